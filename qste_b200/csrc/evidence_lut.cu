// Coordinate evidence of a converted Linear for batches of 1..32 samples, on the CUDA cores,
// bound by writing the rows x columns fp32 result (sm_100a).
//
//   E0[n, k]   = sum_m dY[m, n] * act_scale[m] * sign(act_bits)[m, k]
//   v[n, k]    = E0[n, k] + sum_m dY[m, n] * offset[m]            (the saved activations' offset)
//   g_scale[n] = sum_k v[n, k] * sign(W)[n, k]
//   g_bias[n]  = sum_m dY[m, n]
//   E[n, k]    = v[n, k] * weight_scale[n]
//
// With so few samples the contraction is nothing and the output is everything: 4 bytes per
// coordinate have to be written once (235 MB at 14336 x 4096: 36 us of HBM time), and each takes
// M multiply-adds.  The tensor-core tiles spend such a product entirely in their epilogue, one
// k-block per 128 x 256 tile, four warps draining tensor memory with a row per lane (106-130 us),
// behind four small kernels that prepare their operands (another 30 us).  Here one kernel does all
// of it:
//
//   * every CTA first turns the activation bits round in shared memory: pattern[k] has bit m set
//     when sample m's bit of column k is set (M x K bits read, K words written);
//   * a WARP owns a weight row n.  Lane m holds dY[m, n] * act_scale[m]; the warp tabulates, for
//     every group g of four samples, the 16 signed sums of its four values (the look-up-table idea
//     of the small-batch forward, with the samples as the contraction) -- 16 words per group, so
//     lanes looking up the same group never conflict;
//   * each lane then walks four consecutive columns at a time: one 16-byte load of their four
//     patterns, one look-up and add per group (the offset term rides the first group's entries),
//     the product with the weight's sign for g_scale, the row scale, and one 16-byte store -- a
//     warp stores 512 contiguous bytes per step;
//   * g_bias, the offset term and g_scale are warp sums of one value per lane.
//
// Everything is fp32 from the 16-bit gradient on (no re-encoding), no workspace, no atomics.
// Algorithmic bytes: 4*N*K (written) + N*K/8 (weight bits) + M*K/8 + M*N*e + 12N + 8M.
#include <cuda.h>

#include "common.cuh"
#include "gemm.h"

namespace qste {
namespace {

constexpr int kEvidenceThreads = 512;

struct EvidenceParams {
  const void* dy;            // [M, N]
  const uint8_t* act_bits;   // [M, K / 8]
  const float* offset;       // [M]
  const float* act_scale;    // [M]
  const uint8_t* weight_bits;  // [N, K / 8]
  const float* weight_scale;   // [N]
  float* evidence;           // [N, K]
  float* g_scale;            // [N] or null
  float* g_bias;             // [N] or null
  long long M, N, K, pitch;  // pitch = K / 8
};

// sum + the entries that the nibbles kGroup.. of `word` select in their groups' tables.  The table
// starts on a 64-byte boundary of the shared window, so "base + 4 * nibble" is an OR that folds
// into the mask, and a group's 64 bytes are the load's immediate offset: shift, one logic
// operation, load, add per group.
template <int kGroup, int kGroups>
__device__ __forceinline__ float add_lookups(float sum, uint32_t word, uint32_t table_base) {
  if constexpr (kGroup == kGroups) {
    return sum;
  } else {
    const uint32_t shifted = kGroup == 0 ? word << 2 : word >> (4 * kGroup - 2);
    const uint32_t address = (shifted & 60u) | table_base;
    float entry;
    asm volatile("ld.shared.f32 %0, [%1 + %2];" : "=f"(entry) : "r"(address), "n"(kGroup * 64) : "memory");
    return add_lookups<kGroup + 1, kGroups>(sum + entry, word, table_base);
  }
}

// kGroups: groups of four samples (1..8)
template <typename T, int kGroups>
__global__ void __launch_bounds__(kEvidenceThreads)
evidence_lut_kernel(const __grid_constant__ EvidenceParams p) {
  extern __shared__ __align__(16) uint32_t evidence_shared[];
  uint32_t* pattern = evidence_shared;                                   // [K]
  // [warps][kGroups * 16], on a 64-byte boundary of the shared window (the look-ups rely on it)
  const uint32_t after_patterns = (uint32_t)__cvta_generic_to_shared(evidence_shared + p.K);
  float* tables = reinterpret_cast<float*>(reinterpret_cast<char*>(evidence_shared + p.K) + ((64u - (after_patterns & 63u)) & 63u));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;

  // -- pattern[k]: bit m = sample m's activation bit of column k.  A thread turns one byte column
  //    (eight columns) at a time; for a fixed sample the threads read consecutive bytes.
  for (long long byte = threadIdx.x; byte < p.pitch; byte += blockDim.x) {
    uint32_t word[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
    for (int m = 0; m < (int)p.M; ++m) {
      const uint32_t bits = p.act_bits[m * p.pitch + byte];
#pragma unroll
      for (int j = 0; j < 8; ++j) word[j] |= ((bits >> j) & 1u) << m;
    }
    uint4* out = reinterpret_cast<uint4*>(pattern + byte * 8);
    out[0] = make_uint4(word[0], word[1], word[2], word[3]);
    out[1] = make_uint4(word[4], word[5], word[6], word[7]);
  }
  // this lane's sample
  const bool has_sample = lane < p.M;
  const float my_scale = has_sample ? p.act_scale[lane] : 0.0f;
  const float my_offset = has_sample ? p.offset[lane] : 0.0f;
  __syncthreads();

  float* table = tables + warp * (kGroups * 16);
  const T* dy = static_cast<const T*>(p.dy);
  const long long total_warps = (long long)gridDim.x * warps;
  for (long long n = (long long)blockIdx.x * warps + warp; n < p.N; n += total_warps) {
    const float gradient = has_sample ? DType<T>::load(dy + (long long)lane * p.N + n) : 0.0f;
    const float value = gradient * my_scale;
    const float add = warp_sum(gradient * my_offset);          // sum_m dY[m, n] * offset[m]
    if (p.g_bias) {
      const float bias = warp_sum(gradient);
      if (lane == 0) p.g_bias[n] = bias;
    }
    // -- the 16 signed sums of every group of four samples: lane 4g + s builds patterns 4s..4s+3 of group g
    {
      const int g = lane >> 2, first = (lane & 3) * 4;
      float v[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) v[b] = __shfl_sync(0xffffffffu, value, (4 * g + b) & 31);
      if (g < kGroups) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int pt = first + e;
          // (the offset term rides the first group's entries: one add per coordinate less)
          table[g * 16 + pt] = ((pt & 1) ? v[0] : -v[0]) + ((pt & 2) ? v[1] : -v[1]) + ((pt & 4) ? v[2] : -v[2]) +
                               ((pt & 8) ? v[3] : -v[3]) + (g == 0 ? add : 0.0f);
        }
      }
    }
    __syncwarp();
    const float row_scale = p.weight_scale[n];
    const uint8_t* weight_row = p.weight_bits + n * p.pitch;
    float* out_row = p.evidence + n * p.K;
    const uint32_t table_base = (uint32_t)__cvta_generic_to_shared(table);
    float inner = 0.0f;
    // -- four consecutive columns per lane and step, 128 per warp
    const int columns = (int)p.K;
    for (int k0 = 4 * lane; k0 < columns; k0 += 128) {
      const uint4 words = *reinterpret_cast<const uint4*>(pattern + k0);
      // bits 0..3: where the weight's sign of the four columns is MINUS
      const uint32_t minus = ~((uint32_t)weight_row[k0 >> 3] >> (k0 & 4));
      const uint32_t word[4] = {words.x, words.y, words.z, words.w};
      float out[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float v = add_lookups<0, kGroups>(0.0f, word[e], table_base);
        // v with its sign flipped where the weight's sign is minus
        inner += __uint_as_float(__float_as_uint(v) ^ ((minus << (31 - e)) & 0x80000000u));
        out[e] = v * row_scale;
      }
      *reinterpret_cast<float4*>(out_row + k0) = make_float4(out[0], out[1], out[2], out[3]);
    }
    inner = warp_sum(inner);
    if (p.g_scale && lane == 0) p.g_scale[n] = inner;
    __syncwarp();   // the table is rewritten for the next row
  }
}

template <typename T, int kGroups>
int launch_evidence(const EvidenceParams& params, cudaStream_t stream) {
  auto kernel = evidence_lut_kernel<T, kGroups>;
  const size_t shared = (size_t)params.K * sizeof(uint32_t) + 64 + (size_t)(kEvidenceThreads / 32) * kGroups * 16 * sizeof(float);
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (shared > 48 * 1024 && (device < 0 || device >= 64 || !configured[device])) {
    const cudaError_t error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    if (error != cudaSuccess) { set_last_cuda_error(error, "cudaFuncSetAttribute(evidence_lut)"); return QSTE_ERR_CUDA; }
    if (device >= 0 && device < 64) configured[device] = true;
  }
  // two CTAs per SM when the patterns leave room, rows dealt round-robin to the warps
  const int warps = kEvidenceThreads / 32;
  long long grid = (long long)sm_count() * (shared <= 100 * 1024 ? 2 : 1);
  const long long needed = ceil_div(params.N, warps);
  if (grid > needed) grid = needed;
  kernel<<<(unsigned)grid, kEvidenceThreads, shared, stream>>>(params);
  note_launches(1);
  return launch_status("evidence_lut");
}

}  // namespace

bool evidence_lut_supported(int64_t samples, int64_t rows, int64_t columns, int dtype, const void* grad,
                            const float* evidence) {
  if (samples < 1 || samples > 32 || rows < 1 || columns < 128 || columns % 128 != 0 || columns > 16384) return false;
  if (dtype_size(dtype) == 0) return false;
  if (!aligned(evidence, 16) || !aligned(grad, dtype_size(dtype))) return false;
  return check_arch() == QSTE_OK;
}

int evidence_lut(const void* grad, int dtype, int64_t samples, int64_t rows, const uint8_t* act_bits, const float* aux,
                 int64_t columns, const uint8_t* weight_bits, const float* weight_scale, float* evidence, float* g_scale,
                 float* g_bias, cudaStream_t stream) {
  EvidenceParams params = {};
  params.dy = grad; params.act_bits = act_bits; params.offset = aux; params.act_scale = aux + samples;
  params.weight_bits = weight_bits; params.weight_scale = weight_scale;
  params.evidence = evidence; params.g_scale = g_scale; params.g_bias = g_bias;
  params.M = samples; params.N = rows; params.K = columns; params.pitch = columns / 8;
  const int groups = (int)((samples + 3) / 4);
  int status = QSTE_ERR_DTYPE;
  QSTE_DISPATCH_DTYPE(dtype, T, {
    switch (groups) {
      case 1: status = launch_evidence<T, 1>(params, stream); break;
      case 2: status = launch_evidence<T, 2>(params, stream); break;
      case 3: status = launch_evidence<T, 3>(params, stream); break;
      case 4: status = launch_evidence<T, 4>(params, stream); break;
      case 5: status = launch_evidence<T, 5>(params, stream); break;
      case 6: status = launch_evidence<T, 6>(params, stream); break;
      case 7: status = launch_evidence<T, 7>(params, stream); break;
      default: status = launch_evidence<T, 8>(params, stream); break;
    }
  });
  return status;
}

}  // namespace qste
