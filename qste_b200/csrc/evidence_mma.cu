// Coordinate evidence of a converted Linear for batches of 17..128 samples: warp-level MMAs with
// the activation signs expanded in registers, bound by the tensor pipe's legacy path and by
// writing the rows x columns fp32 result (sm_100a).
//
//   E0[n, k]   = sum_m dY[m, n] * act_scale[m] * sign(act_bits)[m, k]
//   v[n, k]    = E0[n, k] + sum_m dY[m, n] * offset[m]
//   g_scale[n] = sum_k v[n, k] * sign(W)[n, k]
//   g_bias[n]  = sum_m dY[m, n]
//   E[n, k]    = v[n, k] * weight_scale[n]
//
// The contraction (the samples) is short and the result is large, so the tensor-core tiles spend
// such a product in their epilogue, where a lane owns a row and every store instruction of a warp
// touches 32 lines (135-160 us at 14336 x 4096 for 33..128 samples).  Here the product is a
// `mma.sync.m16n8k16` per 16 weight rows x 8 columns x 16 samples:
//
//   * A = dY^T * act_scale for the CTA's rows, staged once in shared memory as fp16 with ONE
//     power of two per output row (the row's largest term lands in [2^13, 2^14), which the
//     epilogue takes back out): a term is rounded once, to 2^-11 of the row's largest;
//   * B = the activation signs.  Every CTA turns the activation bits of a chunk of columns round
//     in shared memory (pattern[w][k]: bit j = sample 32w + j of column k, by 8 x 8 bit-matrix
//     transposes), and a lane turns bits j and j + 16 of a pattern word into a B register with
//     one shift and one logic operation, as the small-batch forward does with weight bits.  The
//     order of the samples inside an MMA is chosen to suit (A is staged in the matching order);
//   * the order of the COLUMNS inside a group of four MMAs is chosen so that a lane ends up with
//     eight consecutive columns of its two rows: the four lanes of a row store 128 contiguous
//     bytes, a warp's store instruction touches 8 lines instead of 32;
//   * a CTA owns a few slabs of 16 rows and walks the columns in chunks of 4096; its warps share
//     out the 32-column blocks of a chunk, so every warp works whatever the row count;
//   * offset term, bias gradient and exponents come from the staging pass (four threads per row,
//     fp32); g_scale is summed per lane, then over the quad and over the warps in a fixed order.
//
// No workspace, no atomics, one launch.
// Algorithmic bytes: 4*N*K (written) + N*K/8 (weight bits) + M*K/8 + M*N*e + 12N + 8M.
#include <cuda.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "gemm.h"

namespace qste {
namespace {

constexpr int kEvThreads = 512;
constexpr int kEvWarps = kEvThreads / 32;
constexpr int kEvChunk = 4096;            // columns per pass of the pattern planes
constexpr int kEvPlane = kEvChunk + 1;    // words between planes: planes fall in different banks
constexpr int kEvMaxSlabs = 8;            // slabs of 16 rows per CTA

struct EvMmaParams {
  const void* dy;              // [M, N]
  const uint8_t* act_bits;     // [M, K / 8]
  const float* offset;         // [M]
  const float* act_scale;      // [M]
  const uint8_t* weight_bits;  // [N, K / 8]
  const float* weight_scale;   // [N]
  float* evidence;             // [N, K]
  float* g_scale;              // [N] or null
  float* g_bias;               // [N] or null
  long long M, N, K, pitch;    // pitch = K / 8
  int slabs_per_cta;
};

__device__ __forceinline__ void ev_ldmatrix_x4(uint32_t (&r)[4], uint32_t address) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
// 32 bytes from one lane in one instruction: whole sectors, not two half-sector writes for L2 to merge
__device__ __forceinline__ void ev_store8(float* destination, const float (&v)[8]) {
  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(destination), "f"(v[0]), "f"(v[1]),
               "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
               : "memory");
}
__device__ __forceinline__ void ev_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Position of sample s' (0..31) of a 32-sample word in the staged A operand.  An MMA step h takes
// 16 positions; lane q of a quad supplies B for positions 2q, 2q+1 (a pair of samples 16 apart,
// bits j and j + 16 of the pattern word) and 2q+8, 2q+9 (the pair four further on).
__device__ __forceinline__ int ev_position(int sample) {
  const int e = sample >> 4, h = (sample >> 3) & 1, c = (sample >> 2) & 1, q = sample & 3;
  return 16 * h + 8 * c + 2 * q + e;
}

// kWords: 32-sample words of the contraction (1..4)
template <typename T, int kWords>
__global__ void __launch_bounds__(kEvThreads)
evidence_mma_kernel(const __grid_constant__ EvMmaParams p) {
  constexpr int kSamples = 32 * kWords;
  constexpr int kAPitch = kSamples * 2 + 16;        // bytes between rows of A: ldmatrix without bank conflicts
  extern __shared__ __align__(16) unsigned char ev_shared[];
  uint32_t* planes = reinterpret_cast<uint32_t*>(ev_shared);                              // [kWords][kEvPlane]
  unsigned char* a_rows = ev_shared + (size_t)kWords * kEvPlane * 4 + 12;                 // [rows][kAPitch], 16-byte aligned
  a_rows += (16 - (reinterpret_cast<uintptr_t>(a_rows) & 15)) & 15;
  const int rows_cta = p.slabs_per_cta * 16;
  float* unscale = reinterpret_cast<float*>(a_rows + (size_t)rows_cta * kAPitch);        // [rows]
  float* correction = unscale + rows_cta;                                                // [rows]
  float* inner_parts = correction + rows_cta;                                            // [warps][rows]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, q = lane & 3;
  const long long row0 = (long long)blockIdx.x * rows_cta;
  const T* dy = static_cast<const T*>(p.dy);

  // -- staging: four threads per row, each a quarter of the samples (the loads of a thread are a
  //    chain of trips to L2, so the chain is what has to be short).  Largest term, offset term and
  //    bias gradient in fp32, then the row as fp16 in the MMA's sample order, scaled by the row's
  //    power of two.
  for (int r0 = 0; r0 < rows_cta; r0 += kEvThreads / 4) {
    const int r = r0 + (threadIdx.x >> 2), part = threadIdx.x & 3;
    const long long n = row0 + r;
    const bool live = r < rows_cta && n < p.N;
    float largest = 0.0f, add = 0.0f, bias = 0.0f;
    if (live) {
#pragma unroll 4
      for (int m = part; m < (int)p.M; m += 4) {
        const float gradient = DType<T>::load(dy + (long long)m * p.N + n);
        largest = fmaxf(largest, fabsf(gradient * p.act_scale[m]));
        add = fmaf(gradient, p.offset[m], add);
        bias += gradient;
      }
    }
#pragma unroll
    for (int offset = 1; offset <= 2; offset <<= 1) {
      largest = fmaxf(largest, __shfl_xor_sync(0xffffffffu, largest, offset));
      add += __shfl_xor_sync(0xffffffffu, add, offset);
      bias += __shfl_xor_sync(0xffffffffu, bias, offset);
    }
    int exponent = 0;
    if (largest > 0.0f) frexpf(largest, &exponent);       // largest = f * 2^exponent, f in [0.5, 1)
    const float up = largest > 0.0f ? scalbnf(1.0f, 14 - exponent) : 1.0f;
    if (r < rows_cta) {
      if (part == 0) {
        if (live && p.g_bias) p.g_bias[n] = bias;
        unscale[r] = largest > 0.0f ? scalbnf(1.0f, exponent - 14) : 1.0f;
        correction[r] = add;
      }
      __half* row = reinterpret_cast<__half*>(a_rows + (size_t)r * kAPitch);
#pragma unroll 4
      for (int m = part; m < kSamples; m += 4) {
        float value = 0.0f;
        if (live && m < p.M) value = DType<T>::load(dy + (long long)m * p.N + n) * p.act_scale[m] * up;
        row[(m & ~31) + ev_position(m & 31)] = __float2half_rn(value);
      }
    }
  }

  // per-lane g_scale sums of rows g and g + 8 of each slab, over this warp's blocks of all chunks
  float inner[kEvMaxSlabs][2];
#pragma unroll
  for (int s = 0; s < kEvMaxSlabs; ++s) inner[s][0] = inner[s][1] = 0.0f;

  const uint32_t a_base = (uint32_t)__cvta_generic_to_shared(a_rows);
  // ldmatrix of an A fragment: lanes 0-7 rows 0-7 at positions 0-7, 8-15 rows 8-15 at 0-7, 16-23
  // rows 0-7 at positions 8-15, 24-31 rows 8-15 at 8-15
  const uint32_t a_lane = a_base + (uint32_t)((lane & 7) + ((lane >> 3) & 1) * 8) * kAPitch + (lane >> 4) * 16;
  const int column_in_block = 8 * (g >> 1) + (g & 1);      // the column this lane supplies B for, of tile 0

  for (long long chunk0 = 0; chunk0 < p.K; chunk0 += kEvChunk) {
    const int chunk_columns = (int)((p.K - chunk0) < kEvChunk ? (p.K - chunk0) : kEvChunk);
    __syncthreads();            // the previous chunk's planes are done with (and the staging, first time round)
    // -- pattern planes of the chunk: an item is eight samples x 32 columns -- eight 4-byte loads (all
    //    in flight together: the build is a chain of trips to L2 otherwise), four 8 x 8 transposes
    {
      const int quads = chunk_columns / 32;                      // runs of four byte columns
      const int items = quads * (kSamples / 8);
      const uint8_t* bits0 = p.act_bits + (chunk0 >> 3);
      for (int item = threadIdx.x; item < items; item += blockDim.x) {
        const int group = item % (kSamples / 8), quad = item / (kSamples / 8);   // group: eight samples
        uint32_t rows8[8];
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          const int m = group * 8 + s;
          rows8[s] = m < p.M ? __ldg(reinterpret_cast<const uint32_t*>(bits0 + (long long)m * p.pitch) + quad) : 0u;
        }
        unsigned char* plane = reinterpret_cast<unsigned char*>(planes + (size_t)(group >> 2) * kEvPlane + quad * 32) + (group & 3);
#pragma unroll
        for (int byte = 0; byte < 4; ++byte) {
          unsigned long long z = 0;
#pragma unroll
          for (int s = 0; s < 8; ++s) z |= (unsigned long long)((rows8[s] >> (8 * byte)) & 0xffu) << (8 * s);
          // bit (8 s + j) -> bit (8 j + s)
          unsigned long long t = (z ^ (z >> 7)) & 0x00AA00AA00AA00AAull;  z ^= t ^ (t << 7);
          t = (z ^ (z >> 14)) & 0x0000CCCC0000CCCCull;                    z ^= t ^ (t << 14);
          t = (z ^ (z >> 28)) & 0x00000000F0F0F0F0ull;                    z ^= t ^ (t << 28);
#pragma unroll
          for (int j = 0; j < 8; ++j) plane[4 * (8 * byte + j)] = (unsigned char)(z >> (8 * j));
        }
      }
    }
    __syncthreads();

    const int blocks = chunk_columns / 32;
    for (int slab = 0; slab < p.slabs_per_cta; ++slab) {
      const long long n_low = row0 + slab * 16 + g, n_high = n_low + 8;
      if (row0 + slab * 16 >= p.N) break;
      // the slab's A operand: eight registers per 32-sample word
      uint32_t a[kWords][2][4];
#pragma unroll
      for (int w = 0; w < kWords; ++w)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          ev_ldmatrix_x4(a[w][h], a_lane + (uint32_t)(slab * 16) * kAPitch + (uint32_t)(w * 64 + h * 32));
      const float unscale_low = unscale[slab * 16 + g], unscale_high = unscale[slab * 16 + 8 + g];
      const float add_low = correction[slab * 16 + g], add_high = correction[slab * 16 + 8 + g];
      const float scale_low = n_low < p.N ? p.weight_scale[n_low] : 0.0f;
      const float scale_high = n_high < p.N ? p.weight_scale[n_high] : 0.0f;
      float sum_low = 0.0f, sum_high = 0.0f;
      // the weight's sign byte of this lane's eight columns, fetched one block ahead (a trip to L2
      // that nothing in a block's own work is long enough to hide)
      const uint8_t* signs_low = p.weight_bits + (n_low < p.N ? n_low : 0) * p.pitch + (chunk0 >> 3) + q;
      const uint8_t* signs_high = p.weight_bits + (n_high < p.N ? n_high : 0) * p.pitch + (chunk0 >> 3) + q;
      // a warp takes a run of consecutive blocks: a row's 128-byte pieces then follow one another in
      // time as they do in memory, which DRAM likes better than pieces 2 KB apart
      const int per_warp = (blocks + kEvWarps - 1) / kEvWarps;
      const int first_block = warp * per_warp;
      const int end_block = first_block + per_warp < blocks ? first_block + per_warp : blocks;
      uint32_t ahead_low = first_block < end_block ? signs_low[first_block * 4] : 0u;
      uint32_t ahead_high = first_block < end_block ? signs_high[first_block * 4] : 0u;
      for (int block = first_block; block < end_block; ++block) {
        const uint32_t minus_low = ~ahead_low, minus_high = ~ahead_high;
        if (block + 1 < end_block) {
          ahead_low = signs_low[(block + 1) * 4];
          ahead_high = signs_high[(block + 1) * 4];
        }
        float acc[4][4];
#pragma unroll
        for (int t = 0; t < 4; ++t)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[t][i] = 0.0f;
        const uint32_t* source = planes + block * 32 + column_in_block;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
#pragma unroll
          for (int w = 0; w < kWords; ++w) {
            // bit 3 of `shifted` is this lane's first sample of the word
            const uint32_t shifted = source[(size_t)w * kEvPlane + 2 * t] << (3 - q);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint32_t b0 = 0xBC00BC00u ^ ((shifted << (12 - 8 * h)) & 0x80008000u);
              const uint32_t b1 = 0xBC00BC00u ^ ((shifted << (8 - 8 * h)) & 0x80008000u);
              ev_mma(acc[t], a[w][h], b0, b1);
            }
          }
        }
        // this lane's eight consecutive columns of rows g and g + 8: column 8q + 2t + e is acc[t][e]
        const long long column = chunk0 + block * 32 + 8 * q;
        float low[8], high[8];
#pragma unroll
        for (int t = 0; t < 4; ++t)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float v_low = fmaf(acc[t][e], unscale_low, add_low);
            const float v_high = fmaf(acc[t][2 + e], unscale_high, add_high);
            sum_low += __uint_as_float(__float_as_uint(v_low) ^ ((minus_low << (31 - (2 * t + e))) & 0x80000000u));
            sum_high += __uint_as_float(__float_as_uint(v_high) ^ ((minus_high << (31 - (2 * t + e))) & 0x80000000u));
            low[2 * t + e] = v_low * scale_low;
            high[2 * t + e] = v_high * scale_high;
          }
        if (n_low < p.N) ev_store8(p.evidence + n_low * p.K + column, low);
        if (n_high < p.N) ev_store8(p.evidence + n_high * p.K + column, high);
      }
#pragma unroll
      for (int s = 0; s < kEvMaxSlabs; ++s)
        if (s == slab) { inner[s][0] += sum_low; inner[s][1] += sum_high; }
    }
  }

  // -- g_scale: the quad's four column groups, then the warps, in a fixed order
  if (p.g_scale) {
#pragma unroll
    for (int s = 0; s < kEvMaxSlabs; ++s) {
      if (s >= p.slabs_per_cta) break;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float value = inner[s][half];
        value += __shfl_xor_sync(0xffffffffu, value, 1);
        value += __shfl_xor_sync(0xffffffffu, value, 2);
        if (q == 0) inner_parts[warp * rows_cta + s * 16 + half * 8 + g] = value;
      }
    }
    __syncthreads();
    for (int r = threadIdx.x; r < rows_cta; r += blockDim.x) {
      const long long n = row0 + r;
      if (n >= p.N) continue;
      float total = 0.0f;
      for (int w = 0; w < kEvWarps; ++w) total += inner_parts[w * rows_cta + r];
      p.g_scale[n] = total;
    }
  }
}

template <int kWords>
size_t ev_mma_shared(int slabs_per_cta) {
  const int rows = slabs_per_cta * 16;
  return (size_t)kWords * kEvPlane * 4 + 32 + (size_t)rows * (32 * kWords * 2 + 16) + (size_t)rows * 4 * (2 + kEvWarps);
}

template <typename T, int kWords>
int launch_ev_mma(EvMmaParams params, cudaStream_t stream) {
  auto kernel = evidence_mma_kernel<T, kWords>;
  const long long slabs = ceil_div(params.N, 16);
  long long per_cta = ceil_div(slabs, sm_count());
  if (per_cta < 1) per_cta = 1;
  if (per_cta > kEvMaxSlabs) return QSTE_ERR_UNSUPPORTED;
  params.slabs_per_cta = (int)per_cta;
  const long long grid = ceil_div(slabs, per_cta);
  const size_t shared = ev_mma_shared<kWords>((int)per_cta);
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 64 || !configured[device]) {
    const cudaError_t error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (error != cudaSuccess) { set_last_cuda_error(error, "cudaFuncSetAttribute(evidence_mma)"); return QSTE_ERR_CUDA; }
    if (device >= 0 && device < 64) configured[device] = true;
  }
  kernel<<<(unsigned)grid, kEvThreads, shared, stream>>>(params);
  note_launches(1);
  return launch_status("evidence_mma");
}

}  // namespace

bool evidence_mma_supported(int64_t samples, int64_t rows, int64_t columns, int dtype, const void* grad,
                            const void* act_bits, const float* evidence) {
  if (samples < 1 || samples > 128 || rows < 1 || columns < 128 || columns % 128 != 0) return false;
  if (dtype_size(dtype) == 0) return false;
  if (!aligned(evidence, 32) || !aligned(grad, dtype_size(dtype)) || !aligned(act_bits, 4)) return false;
  if (ceil_div(ceil_div(rows, 16), sm_count()) > kEvMaxSlabs) return false;
  return check_arch() == QSTE_OK;
}

int evidence_mma(const void* grad, int dtype, int64_t samples, int64_t rows, const uint8_t* act_bits, const float* aux,
                 int64_t columns, const uint8_t* weight_bits, const float* weight_scale, float* evidence, float* g_scale,
                 float* g_bias, cudaStream_t stream) {
  EvMmaParams params = {};
  params.dy = grad; params.act_bits = act_bits; params.offset = aux; params.act_scale = aux + samples;
  params.weight_bits = weight_bits; params.weight_scale = weight_scale;
  params.evidence = evidence; params.g_scale = g_scale; params.g_bias = g_bias;
  params.M = samples; params.N = rows; params.K = columns; params.pitch = columns / 8;
  const int words = (int)((samples + 31) / 32);
  int status = QSTE_ERR_DTYPE;
  QSTE_DISPATCH_DTYPE(dtype, T, {
    switch (words) {
      case 1: status = launch_ev_mma<T, 1>(params, stream); break;
      case 2: status = launch_ev_mma<T, 2>(params, stream); break;
      case 3: status = launch_ev_mma<T, 3>(params, stream); break;
      default: status = launch_ev_mma<T, 4>(params, stream); break;
    }
  });
  return status;
}

}  // namespace qste
