// Shared helpers for the qste_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qste_b200.h"

namespace qste {

// -- host side ------------------------------------------------------------------

void set_last_cuda_error(cudaError_t error, const char* where);
// Adds to the process-wide count of kernels this library has launched.
void note_launches(int count);
// Records which kernel family served the calling thread's forward (a string literal).
void note_forward_kernel(const char* name);

// Checks the launch that was just enqueued; returns a qste_status.
inline int launch_status(const char* where) {
  cudaError_t error = cudaGetLastError();
  if (error != cudaSuccess) {
    set_last_cuda_error(error, where);
    return QSTE_ERR_CUDA;
  }
  return QSTE_OK;
}

inline bool aligned(const void* pointer, size_t bytes) {
  return (reinterpret_cast<uintptr_t>(pointer) % bytes) == 0;
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline size_t align_up(size_t value, size_t to) { return (value + to - 1) / to * to; }

inline size_t dtype_size(int dtype) {
  switch (dtype) {
    case QSTE_F32: return 4;
    case QSTE_F16: return 2;
    case QSTE_BF16: return 2;
    default: return 0;
  }
}

inline cudaStream_t as_stream(qste_stream_t stream) { return reinterpret_cast<cudaStream_t>(stream); }

// Number of SMs of the current device (cached per device id).
int sm_count();
// SMs the calling thread's persistent GEMMs leave free (qste_b200_set_reserved_sms).
int reserved_sms();
// QSTE_OK when the current device is compute capability 10.x.
int check_arch();

// -- device side ------------------------------------------------------------------

template <typename T> struct DType;
template <> struct DType<float> {
  static constexpr int id = QSTE_F32;
  __device__ static float load(const float* p) { return *p; }
  __device__ static void store(float* p, float v) { *p = v; }
};
template <> struct DType<__half> {
  static constexpr int id = QSTE_F16;
  __device__ static float load(const __half* p) { return __half2float(*p); }
  __device__ static void store(__half* p, float v) { *p = __float2half_rn(v); }
};
template <> struct DType<__nv_bfloat16> {
  static constexpr int id = QSTE_BF16;
  __device__ static float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  __device__ static void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

__device__ __forceinline__ float sign_of_bit(unsigned byte, int bit) {
  return ((byte >> bit) & 1u) ? 1.0f : -1.0f;
}

// +x when the bit is set, -x otherwise, without a multiply.
__device__ __forceinline__ float apply_sign(float x, unsigned bit) {
  return __uint_as_float(__float_as_uint(x) ^ ((bit ^ 1u) << 31));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}

}  // namespace qste

// Dispatch a templated call over the three activation dtypes.
#define QSTE_DISPATCH_DTYPE(dtype, T, ...)                           \
  switch (dtype) {                                                   \
    case QSTE_F32: { using T = float; __VA_ARGS__; break; }          \
    case QSTE_F16: { using T = __half; __VA_ARGS__; break; }         \
    case QSTE_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
    default: return QSTE_ERR_DTYPE;                                  \
  }
