// Smooth activations with an int8 derivative tape, one pass each way (sm_100a).
//
// A smooth activation of the reference's packed family (GELU, SiLU, Tanh, Sigmoid, ELU, CELU,
// SELU, Softplus, Mish, Hardswish) keeps, instead of its input, its local derivative as int8
// against one fp32 scale per row (src/qste/nn.py:483-507 of the reference):
//
//   forward   y = f(x);  d = f'(x);  scale[r] = max(max_c |d[r, c]|, 1e-8) / 127
//             q[r, c] = clamp(rint(d[r, c] / scale[r]), -127, 127)
//   backward  grad_in = grad_out * (q * scale)
//
// The reference does this with a dozen element-wise torch kernels over the activation.  Here
// the forward is ONE kernel: a block walks one row, computes y and d in fp32, writes y, keeps d
// in shared memory while the row maximum is reduced, then writes the int8 row (x is read once:
// 2 + 2 + 1 bytes per element for a 16-bit dtype).  The backward is one element-wise kernel.
//
// HBM-bound on paper (5 bytes per element forward, 5 backward); the transcendental functions
// make the forward about as expensive in issue slots as in bytes.
#include "common.cuh"

namespace qste {
namespace {

enum Act {
  ACT_GELU = 0, ACT_GELU_TANH = 1, ACT_SILU = 2, ACT_TANH = 3, ACT_SIGMOID = 4, ACT_ELU = 5,
  ACT_CELU = 6, ACT_SELU = 7, ACT_SOFTPLUS = 8, ACT_MISH = 9, ACT_HARDSWISH = 10, ACT_COUNT = 11
};

constexpr float kSeluAlpha = 1.6732632423543772f;
constexpr float kSeluScale = 1.0507009873554805f;

template <typename T> __device__ __forceinline__ float round_through(float v) {
  T stored;
  DType<T>::store(&stored, v);
  return DType<T>::load(&stored);
}

// 1 / (1 + e^-x).  For a 16-bit tensor the fast exponential and division are exact to well inside
// the type's last bit (2^-21 relative against 2^-9 / 2^-11) and take a third of the instructions.
template <typename T>
__device__ __forceinline__ float sigmoidf(float x) {
  if (sizeof(T) == 2) return __fdividef(1.0f, 1.0f + __expf(-x));
  return 1.0f / (1.0f + expf(-x));
}

// y = f(x) and d = f'(x).  Where the reference forms the derivative from the activation's
// OUTPUT (tanh, sigmoid, elu, celu, selu: nn.py:414-470) it uses the output as stored, i.e.
// rounded to the tensor's dtype; `T` reproduces that rounding.
template <typename T, int kKind>
__device__ __forceinline__ void activate(float x, float a, float& y, float& d) {
  if (kKind == ACT_GELU) {
    const float cdf = 0.5f * (1.0f + erff(x * 0.70710678118654752440f));
    y = x * cdf;
    d = cdf + x * expf(-0.5f * x * x) * 0.39894228040143267794f;
  } else if (kKind == ACT_GELU_TANH) {
    const float c = 0.79788456080286535588f, k = 0.044715f;
    const float t = tanhf(c * (x + k * x * x * x));
    y = 0.5f * x * (1.0f + t);
    d = 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * c * (1.0f + 3.0f * k * x * x);
  } else if (kKind == ACT_SILU) {
    const float s = sigmoidf<T>(x);
    y = x * s;
    d = s * (1.0f + x * (1.0f - s));
  } else if (kKind == ACT_TANH) {
    y = tanhf(x);
    const float stored = round_through<T>(y);
    d = 1.0f - stored * stored;
  } else if (kKind == ACT_SIGMOID) {
    y = sigmoidf<T>(x);
    const float stored = round_through<T>(y);
    d = stored * (1.0f - stored);
  } else if (kKind == ACT_ELU) {
    y = x > 0.0f ? x : a * expm1f(x);
    d = x > 0.0f ? 1.0f : round_through<T>(y) + a;
  } else if (kKind == ACT_CELU) {
    y = fmaxf(0.0f, x) + fminf(0.0f, a * expm1f(x / a));
    d = x > 0.0f ? 1.0f : round_through<T>(y) / a + 1.0f;
  } else if (kKind == ACT_SELU) {
    y = kSeluScale * (x > 0.0f ? x : kSeluAlpha * expm1f(x));
    d = x > 0.0f ? kSeluScale : round_through<T>(y) + kSeluScale * kSeluAlpha;
  } else if (kKind == ACT_SOFTPLUS) {
    y = x * a > 20.0f ? x : log1pf(expf(x * a)) / a;
    d = sigmoidf<T>(a * x);
  } else if (kKind == ACT_MISH) {
    const float softplus = x > 20.0f ? x : log1pf(expf(x));
    const float t = tanhf(softplus);
    y = x * t;
    d = t + x * (1.0f - t * t) * sigmoidf<T>(x);
  } else {  // ACT_HARDSWISH
    y = x * fminf(fmaxf(x + 3.0f, 0.0f), 6.0f) * (1.0f / 6.0f);
    d = x <= -3.0f ? 0.0f : (x >= 3.0f ? 1.0f : (2.0f * x + 3.0f) * (1.0f / 6.0f));
  }
}

constexpr int kActThreads = 256;

// One block per row (rows are walked grid-stride).  Dynamic shared memory: `columns` floats.
template <typename T, int kKind, int kVec>
__global__ void __launch_bounds__(kActThreads)
smooth_forward_kernel(const T* __restrict__ x, long long rows, long long columns, float a, T* __restrict__ y,
                      int8_t* __restrict__ q, float* __restrict__ scale) {
  extern __shared__ float derivative[];
  __shared__ float warp_max[kActThreads / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* source = x + row * columns;
    T* target = y + row * columns;
    float largest = 0.0f;
    for (long long c = (long long)threadIdx.x * kVec; c < columns; c += (long long)kActThreads * kVec) {
      T in[kVec], out[kVec];
      if (kVec > 1) *reinterpret_cast<uint4*>(in) = *reinterpret_cast<const uint4*>(source + c);
      else in[0] = source[c];
#pragma unroll
      for (int e = 0; e < kVec; ++e) {
        float value, slope;
        activate<T, kKind>(DType<T>::load(in + e), a, value, slope);
        DType<T>::store(out + e, value);
        derivative[c + e] = slope;
        largest = fmaxf(largest, fabsf(slope));
      }
      if (kVec > 1) *reinterpret_cast<uint4*>(target + c) = *reinterpret_cast<const uint4*>(out);
      else target[c] = out[0];
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) largest = fmaxf(largest, __shfl_xor_sync(0xffffffffu, largest, offset));
    if (lane == 0) warp_max[warp] = largest;
    __syncthreads();
    largest = warp_max[0];
#pragma unroll
    for (int w = 1; w < kActThreads / 32; ++w) largest = fmaxf(largest, warp_max[w]);
    const float step = fmaxf(largest, 1e-8f) / 127.0f;
    if (threadIdx.x == 0) scale[row] = step;
    // one reciprocal per row instead of a division per element: the quotient moves by an ulp, the
    // int8 value only where it sat within that of a half
    const float inverse = 1.0f / step;
    int8_t* tape = q + row * columns;
    // each thread quantises what it wrote itself: no barrier needed before, one after (the
    // next row reuses the buffer and warp_max)
    for (long long c = (long long)threadIdx.x * kVec; c < columns; c += (long long)kActThreads * kVec) {
      int8_t packed[kVec];
#pragma unroll
      for (int e = 0; e < kVec; ++e)
        packed[e] = (int8_t)fminf(127.0f, fmaxf(-127.0f, rintf(derivative[c + e] * inverse)));
      if (kVec == 8) *reinterpret_cast<uint2*>(tape + c) = *reinterpret_cast<const uint2*>(packed);
      else if (kVec == 4) *reinterpret_cast<uint32_t*>(tape + c) = *reinterpret_cast<const uint32_t*>(packed);
      else tape[c] = packed[0];
    }
    __syncthreads();
  }
}

// grad_in = grad_out * round(q * round(scale)), every product rounded to the tensor's dtype as
// the reference's torch expression rounds it (nn.py:504-507).
template <typename T, int kVec>
__global__ void __launch_bounds__(256)
smooth_backward_kernel(const T* __restrict__ grad, const int8_t* __restrict__ q, const float* __restrict__ scale,
                       long long rows, long long columns, T* __restrict__ out) {
  const long long per_row = columns / kVec;
  const long long total = rows * per_row;
  for (long long index = blockIdx.x * (long long)blockDim.x + threadIdx.x; index < total;
       index += (long long)gridDim.x * blockDim.x) {
    const long long row = index / per_row;
    const long long at = row * columns + (index - row * per_row) * kVec;
    const float step = round_through<T>(scale[row]);
    T in[kVec], result[kVec];
    int8_t tape[kVec];
    if (kVec == 8) {
      *reinterpret_cast<uint4*>(in) = *reinterpret_cast<const uint4*>(grad + at);
      *reinterpret_cast<uint2*>(tape) = *reinterpret_cast<const uint2*>(q + at);
    } else if (kVec == 4) {
      *reinterpret_cast<uint4*>(in) = *reinterpret_cast<const uint4*>(grad + at);
      *reinterpret_cast<uint32_t*>(tape) = *reinterpret_cast<const uint32_t*>(q + at);
    } else {
      in[0] = grad[at];
      tape[0] = q[at];
    }
#pragma unroll
    for (int e = 0; e < kVec; ++e)
      DType<T>::store(result + e, DType<T>::load(in + e) * round_through<T>((float)tape[e] * step));
    if (kVec > 1) *reinterpret_cast<uint4*>(out + at) = *reinterpret_cast<const uint4*>(result);
    else out[at] = result[0];
  }
}

template <typename T, int kVec>
int launch_forward(int kind, const T* x, long long rows, long long columns, float a, T* y, int8_t* q, float* scale,
                   cudaStream_t stream) {
  const size_t shared = (size_t)columns * sizeof(float);
  long long grid = rows;
  const long long cap = (long long)sm_count() * 8;
  if (grid > cap) grid = cap;
#define QSTE_ACT_CASE(K)                                                                                   \
  case K: {                                                                                                \
    auto kernel = smooth_forward_kernel<T, K, kVec>;                                                       \
    if (shared > 48 * 1024) {                                                                              \
      const cudaError_t error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared); \
      if (error != cudaSuccess) { set_last_cuda_error(error, "cudaFuncSetAttribute(smooth_forward)"); return QSTE_ERR_CUDA; } \
    }                                                                                                      \
    kernel<<<(unsigned)grid, kActThreads, shared, stream>>>(x, rows, columns, a, y, q, scale);             \
    break;                                                                                                 \
  }
  switch (kind) {
    QSTE_ACT_CASE(ACT_GELU) QSTE_ACT_CASE(ACT_GELU_TANH) QSTE_ACT_CASE(ACT_SILU) QSTE_ACT_CASE(ACT_TANH)
    QSTE_ACT_CASE(ACT_SIGMOID) QSTE_ACT_CASE(ACT_ELU) QSTE_ACT_CASE(ACT_CELU) QSTE_ACT_CASE(ACT_SELU)
    QSTE_ACT_CASE(ACT_SOFTPLUS) QSTE_ACT_CASE(ACT_MISH) QSTE_ACT_CASE(ACT_HARDSWISH)
    default: return QSTE_ERR_UNSUPPORTED;
  }
#undef QSTE_ACT_CASE
  note_launches(1);
  return launch_status("smooth_forward");
}

template <typename T>
int forward_for(int kind, const void* x, long long rows, long long columns, float a, void* y, int8_t* q, float* scale,
                cudaStream_t stream) {
  constexpr int kWide = 16 / (int)sizeof(T);
  const bool wide = columns % kWide == 0 && aligned(x, 16) && aligned(y, 16) && aligned(q, 8);
  if (wide)
    return launch_forward<T, kWide>(kind, static_cast<const T*>(x), rows, columns, a, static_cast<T*>(y), q, scale, stream);
  return launch_forward<T, 1>(kind, static_cast<const T*>(x), rows, columns, a, static_cast<T*>(y), q, scale, stream);
}

template <typename T>
int backward_for(const void* grad, const int8_t* q, const float* scale, long long rows, long long columns, void* out,
                 cudaStream_t stream) {
  constexpr int kWide = 16 / (int)sizeof(T);
  const bool wide = columns % kWide == 0 && aligned(grad, 16) && aligned(out, 16) && aligned(q, 8);
  const long long items = wide ? rows * (columns / kWide) : rows * columns;
  long long grid = ceil_div(items, 256);
  const long long cap = (long long)sm_count() * 16;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  if (wide)
    smooth_backward_kernel<T, kWide><<<(unsigned)grid, 256, 0, stream>>>(static_cast<const T*>(grad), q, scale, rows, columns,
                                                                        static_cast<T*>(out));
  else
    smooth_backward_kernel<T, 1><<<(unsigned)grid, 256, 0, stream>>>(static_cast<const T*>(grad), q, scale, rows, columns,
                                                                    static_cast<T*>(out));
  note_launches(1);
  return launch_status("smooth_backward");
}

}  // namespace
}  // namespace qste

using namespace qste;

extern "C" {

int qste_b200_smooth_forward(const void* inputs, int dtype, int64_t rows, int64_t columns, int kind, double parameter,
                             void* outputs, int8_t* derivative, float* scale, qste_stream_t stream) {
  if (rows < 0 || columns < 0) return QSTE_ERR_SHAPE;
  if (dtype_size(dtype) == 0) return QSTE_ERR_DTYPE;
  if (kind < 0 || kind >= ACT_COUNT) return QSTE_ERR_UNSUPPORTED;
  if (rows == 0 || columns == 0) return QSTE_OK;
  if (!inputs || !outputs || !derivative || !scale) return QSTE_ERR_NULL;
  if ((size_t)columns * sizeof(float) > 200 * 1024) return QSTE_ERR_LIMIT;  // the row's derivatives sit in shared memory
  if (check_arch() != QSTE_OK) return QSTE_ERR_ARCH;
  QSTE_DISPATCH_DTYPE(dtype, T, return forward_for<T>(kind, inputs, rows, columns, (float)parameter, outputs, derivative,
                                                      scale, as_stream(stream)));
  return QSTE_ERR_DTYPE;
}

int qste_b200_smooth_backward(const void* grad, int dtype, const int8_t* derivative, const float* scale, int64_t rows,
                              int64_t columns, void* grad_inputs, qste_stream_t stream) {
  if (rows < 0 || columns < 0) return QSTE_ERR_SHAPE;
  if (dtype_size(dtype) == 0) return QSTE_ERR_DTYPE;
  if (rows == 0 || columns == 0) return QSTE_OK;
  if (!grad || !derivative || !scale || !grad_inputs) return QSTE_ERR_NULL;
  if (check_arch() != QSTE_OK) return QSTE_ERR_ARCH;
  QSTE_DISPATCH_DTYPE(dtype, T, return backward_for<T>(grad, derivative, scale, rows, columns, grad_inputs, as_stream(stream)));
  return QSTE_ERR_DTYPE;
}

}  // extern "C"
