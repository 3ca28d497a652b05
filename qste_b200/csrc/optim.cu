// The int8 coordinate optimizer: one step for one surface.
//
// Compiled with -fmad=false.  The step's integer outputs (int8 coordinates, int8
// moments, packed sign bits, flip count) are decided by fp32 comparisons, so the
// kernels below reproduce the reference's CPU kernel
// (src/qste/kernels/cpu.cpp:578-808) operation by operation:
//
//   * every fp32 sum the reference forms sequentially -- a row's sum of squares
//     over ascending columns, a column's over ascending rows, the four strided
//     lanes of the update norm, a moment block's sum of squares -- is formed here
//     by ONE thread in the same order.  Parallelism comes from running many such
//     chains at once (one lane per row / column / block), not from splitting a
//     chain;
//   * rows and blocks are walked through 32x32 shared-memory tiles filled with
//     cp.async, eight tiles deep per warp, so global traffic stays coalesced and
//     the chains never wait on DRAM;
//   * the three sums the reference accumulates in double (row mean, update norm,
//     moment norm) are reduced in double with a fixed tree.  Their result is
//     rounded to fp32 once, so it can differ from the reference's sequential
//     double sum only when the exact value lies within ~1e-16 (relative) of an
//     fp32 rounding boundary.
//
// The reference's hand-written loops run on one thread (its extension is built
// without OpenMP, so at::parallel_for is a plain call); that single-thread order
// is the one reproduced.
#include <stdlib.h>

#include "common.cuh"

namespace qste {

constexpr int kStages = 8;
constexpr int kTile = 32;
constexpr int kPitch = kTile + 1;

struct UpdateScalars {           // lives at the start of the workspace
  unsigned long long reserved;   // +0  (the GEMM kernels count their abandoned waits here)
  long long flips;               // +8
  float gain;                    // +16  (1 - beta1) / update_divisor
  float coordinate_step;         // +20  coordinate_lr / moment_rms
  float sqrt_row_mean;           // +24
  float update_rms;              // +28
  float moment_rms;              // +32
  float pad[7];
};

__device__ __forceinline__ void cp_async4(void* smem, const void* global) {
  const unsigned address = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(address), "l"(global) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ bool disabled(const uint8_t* update_enabled) {
  return update_enabled != nullptr && *update_enabled == 0;
}

// Fill one 32x32 tile: rows r0.., columns c0.. of a matrix with row pitch `ld`;
// lane l fetches column c0 + l of each row (a 128-byte line per row).  Elements
// outside [R, C) or at/after flat index `limit` become +0.
__device__ __forceinline__ void issue_tile(float (*slot)[kPitch], const float* __restrict__ g,
                                           int64_t ld, int64_t r0, int64_t c0, int64_t R, int64_t C,
                                           int64_t limit, int lane) {
  const int64_t col = c0 + lane;
#pragma unroll 8
  for (int i = 0; i < kTile; ++i) {
    const int64_t row = r0 + i;
    const int64_t flat = row * ld + col;
    if (row < R && col < C && flat < limit)
      cp_async4(&slot[i][lane], g + flat);
    else
      slot[i][lane] = 0.0f;
  }
  cp_async_commit();
}

// ---------------------------------------------------------------------------
// Pass 1a: row sums of squares (cpu.cpp:629-641), one lane per row
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(32)
row_squares_kernel(const float* __restrict__ g, int64_t R, int64_t C, uint16_t* __restrict__ row_v,
                   float* __restrict__ row_stats, float beta2, const uint8_t* update_enabled) {
  if (disabled(update_enabled)) return;
  __shared__ float ring[kStages][kTile][kPitch];
  const int lane = threadIdx.x;
  const int64_t r0 = (int64_t)blockIdx.x * kTile;
  const int64_t tiles = (C + kTile - 1) / kTile;
  const int64_t limit = R * C;
  // the prologue always commits kStages - 1 groups (empty ones past the last tile), so
  // that "at most kStages - 1 groups pending" below means "tile t has landed"
  for (int64_t t = 0; t < kStages - 1; ++t) {
    if (t < tiles) issue_tile(ring[t % kStages], g, C, r0, t * kTile, R, C, limit, lane);
    else cp_async_commit();
  }
  float total = 0.0f;
  for (int64_t t = 0; t < tiles; ++t) {
    if (t + kStages - 1 < tiles)
      issue_tile(ring[(t + kStages - 1) % kStages], g, C, r0, (t + kStages - 1) * kTile, R, C, limit, lane);
    else
      cp_async_commit();
    cp_async_wait<kStages - 1>();
    __syncwarp();
    const float* line = ring[t % kStages][lane];
#pragma unroll
    for (int c = 0; c < kTile; ++c) {
      const float square = line[c] * line[c];
      total += square;
    }
    __syncwarp();
  }
  const int64_t row = r0 + lane;
  if (row < R) {
    const float previous = __half2float(__ushort_as_half(row_v[row]));
    const float updated = previous * beta2 + (total / (float)C + 1e-12f) * (1.0f - beta2);
    row_stats[row] = updated;
    row_v[row] = __half_as_ushort(__float2half_rn(updated));
  }
}

// ---------------------------------------------------------------------------
// Pass 1b: column sums of squares over ascending rows (cpu.cpp:632-636, 643-648)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(32)
column_squares_kernel(const float* __restrict__ g, int64_t R, int64_t C,
                      float* __restrict__ column_sum, const uint8_t* update_enabled) {
  if (disabled(update_enabled)) return;
  __shared__ float ring[kStages][kTile][kPitch];
  const int lane = threadIdx.x;
  const int64_t c0 = (int64_t)blockIdx.x * kTile;
  const int64_t tiles = (R + kTile - 1) / kTile;
  const int64_t limit = R * C;
  for (int64_t t = 0; t < kStages - 1; ++t) {
    if (t < tiles) issue_tile(ring[t % kStages], g, C, t * kTile, c0, R, C, limit, lane);
    else cp_async_commit();
  }
  float total = 0.0f;
  for (int64_t t = 0; t < tiles; ++t) {
    if (t + kStages - 1 < tiles)
      issue_tile(ring[(t + kStages - 1) % kStages], g, C, (t + kStages - 1) * kTile, c0, R, C, limit, lane);
    else
      cp_async_commit();
    cp_async_wait<kStages - 1>();
    __syncwarp();
    float (*slot)[kPitch] = ring[t % kStages];
#pragma unroll
    for (int i = 0; i < kTile; ++i) {
      const float value = slot[i][lane];
      const float square = value * value;
      total += square;
    }
    __syncwarp();
  }
  if (c0 + lane < C) column_sum[c0 + lane] = total;
}

// ---------------------------------------------------------------------------
// Deterministic block-wide double sum (fixed strided order, fixed tree)
// ---------------------------------------------------------------------------
__device__ double block_sum_double(double value, double* shared) {
  const int tid = threadIdx.x;
  shared[tid] = value;
  __syncthreads();
  for (int width = blockDim.x >> 1; width > 0; width >>= 1) {
    if (tid < width) shared[tid] += shared[tid + width];
    __syncthreads();
  }
  const double total = shared[0];
  __syncthreads();
  return total;
}

// Finish pass 1: column EMA (cpu.cpp:649-652), row mean in double (656-660), the
// two normalisation vectors (661-667).  One block.
__global__ void __launch_bounds__(1024)
finish_factors_kernel(const float* __restrict__ column_sum, uint16_t* __restrict__ col_v,
                      const float* __restrict__ row_stats, float* __restrict__ row_factor,
                      float* __restrict__ column_factor, int64_t R, int64_t C, float beta2,
                      UpdateScalars* scalars, const uint8_t* update_enabled) {
  if (disabled(update_enabled)) return;
  __shared__ double shared[1024];
  const int tid = threadIdx.x;
  for (int64_t c = tid; c < C; c += blockDim.x) {
    const float previous = __half2float(__ushort_as_half(col_v[c]));
    const float updated = previous * beta2 + (column_sum[c] / (float)R + 1e-12f) * (1.0f - beta2);
    col_v[c] = __half_as_ushort(__float2half_rn(updated));
    column_factor[c] = 1.0f / sqrtf(fmaxf(updated, 1e-10f));
  }
  double local = 0.0;
  for (int64_t r = tid; r < R; r += blockDim.x) local += (double)row_stats[r];
  const double accumulated = block_sum_double(local, shared);
  const float row_mean = fmaxf((float)(accumulated / (double)R), 1e-10f);
  const float sqrt_row_mean = sqrtf(row_mean);
  for (int64_t r = tid; r < R; r += blockDim.x)
    row_factor[r] = sqrt_row_mean / sqrtf(fmaxf(row_stats[r], 1e-10f));
  if (tid == 0) {
    scalars->sqrt_row_mean = sqrt_row_mean;
    scalars->flips = 0;
  }
}

// ---------------------------------------------------------------------------
// Pass 2: normalise in place, four strided sums of squares per row (cpu.cpp:670-699)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(32)
precondition_kernel(float* __restrict__ g, int64_t R, int64_t C, const float* __restrict__ row_factor,
                    const float* __restrict__ column_factor, double* __restrict__ row_partial,
                    const uint8_t* update_enabled) {
  if (disabled(update_enabled)) return;
  __shared__ float ring[kStages][kTile][kPitch];
  const int lane = threadIdx.x;
  const int64_t r0 = (int64_t)blockIdx.x * kTile;
  const int64_t tiles = (C + kTile - 1) / kTile;
  const int64_t limit = R * C;
  const int64_t main4 = C & ~(int64_t)3;
  const int64_t row = r0 + lane;
  const float multiplier = row < R ? row_factor[row] : 0.0f;
  for (int64_t t = 0; t < kStages - 1; ++t) {
    if (t < tiles) issue_tile(ring[t % kStages], g, C, r0, t * kTile, R, C, limit, lane);
    else cp_async_commit();
  }
  float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
  for (int64_t t = 0; t < tiles; ++t) {
    // The slot refilled here was drained (read back to global) in iteration t - 1.
    if (t + kStages - 1 < tiles)
      issue_tile(ring[(t + kStages - 1) % kStages], g, C, r0, (t + kStages - 1) * kTile, R, C, limit, lane);
    else
      cp_async_commit();
    cp_async_wait<kStages - 1>();
    __syncwarp();
    float (*slot)[kPitch] = ring[t % kStages];
    const int64_t c0 = t * kTile;
    const float my_factor = (c0 + lane < C) ? column_factor[c0 + lane] : 0.0f;
    float* line = slot[lane];
#pragma unroll
    for (int c = 0; c < kTile; ++c) {
      const float factor = __shfl_sync(0xffffffffu, my_factor, c);
      const float update = line[c] * multiplier * factor;
      line[c] = update;
      const float square = update * update;
      if (c0 + c >= main4) a0 += square;          // ragged tail lands in lane 0
      else if ((c & 3) == 0) a0 += square;
      else if ((c & 3) == 1) a1 += square;
      else if ((c & 3) == 2) a2 += square;
      else a3 += square;
    }
    __syncwarp();
    const int64_t col = c0 + lane;
    if (col < C) {
#pragma unroll 8
      for (int i = 0; i < kTile; ++i)
        if (r0 + i < R) g[(r0 + i) * C + col] = slot[i][lane];
    }
    __syncwarp();
  }
  if (row < R) row_partial[row] = (double)(a0 + a1) + (double)(a2 + a3);
}

// Global update RMS and clip divisor (cpu.cpp:702-707).  One block.
__global__ void __launch_bounds__(1024)
finish_update_norm_kernel(const double* __restrict__ row_partial, int64_t R, int64_t count,
                          float beta1, float update_clip, UpdateScalars* scalars,
                          const uint8_t* update_enabled) {
  if (disabled(update_enabled)) return;
  __shared__ double shared[1024];
  double local = 0.0;
  for (int64_t r = threadIdx.x; r < R; r += blockDim.x) local += row_partial[r];
  const double square_sum = block_sum_double(local, shared);
  if (threadIdx.x == 0) {
    const float update_rms = sqrtf(fmaxf((float)(square_sum / (double)count), 1e-16f));
    const float update_divisor = fmaxf(1.0f, update_rms / update_clip);
    const float inverse_divisor = 1.0f / update_divisor;
    scalars->update_rms = update_rms;
    scalars->gain = (1.0f - beta1) * inverse_divisor;
  }
}

// ---------------------------------------------------------------------------
// Pass 3: first moment per block (cpu.cpp:714-735), one lane per block
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(32)
moment_kernel(float* __restrict__ g, const int8_t* __restrict__ moment_q,
              uint16_t* __restrict__ moment_scale, int64_t count, int64_t block_size, int64_t blocks,
              float beta1, const UpdateScalars* __restrict__ scalars,
              double* __restrict__ block_partial, const uint8_t* update_enabled) {
  if (disabled(update_enabled)) return;
  __shared__ float ring[kStages][kTile][kPitch];
  const int lane = threadIdx.x;
  const int64_t b0 = (int64_t)blockIdx.x * kTile;
  const int64_t tiles = (block_size + kTile - 1) / kTile;
  const int64_t block = b0 + lane;
  const bool live = block < blocks;
  const float old_scale = live ? __half2float(__ushort_as_half(moment_scale[block])) : 0.0f;
  const float decay = old_scale * beta1;
  const float gain = scalars->gain;
  for (int64_t t = 0; t < kStages - 1; ++t) {
    if (t < tiles) issue_tile(ring[t % kStages], g, block_size, b0, t * kTile, blocks, block_size, count, lane);
    else cp_async_commit();
  }
  float maximum = 1e-6f;
  float block_square = 0.0f;
  for (int64_t t = 0; t < tiles; ++t) {
    if (t + kStages - 1 < tiles)
      issue_tile(ring[(t + kStages - 1) % kStages], g, block_size, b0, (t + kStages - 1) * kTile,
                 blocks, block_size, count, lane);
    else
      cp_async_commit();
    // this lane's 32 int8 moments for the tile, fetched while the tile lands
    const int64_t t0 = t * kTile;
    const int64_t start = block * block_size + t0;
    int width = 0;
    if (live) {
      int64_t left = block_size - t0;
      if (count - start < left) left = count - start;
      width = left <= 0 ? 0 : (left < kTile ? (int)left : kTile);
    }
    __align__(16) int8_t previous[kTile];
    if (width == kTile && ((reinterpret_cast<uintptr_t>(moment_q + start) & 15) == 0)) {
      const uint4 lo = *reinterpret_cast<const uint4*>(moment_q + start);
      const uint4 hi = *reinterpret_cast<const uint4*>(moment_q + start + 16);
      *reinterpret_cast<uint4*>(previous) = lo;
      *reinterpret_cast<uint4*>(previous + 16) = hi;
    } else {
#pragma unroll
      for (int e = 0; e < kTile; ++e) previous[e] = e < width ? moment_q[start + e] : (int8_t)0;
    }
    cp_async_wait<kStages - 1>();
    __syncwarp();
    float (*slot)[kPitch] = ring[t % kStages];
    float* line = slot[lane];
#pragma unroll
    for (int e = 0; e < kTile; ++e) {
      if (e < width) {
        const float moment = (float)previous[e] * decay + line[e] * gain;
        line[e] = moment;
        block_square += moment * moment;
        maximum = fmaxf(maximum, fabsf(moment));
      }
    }
    __syncwarp();
    const int64_t col = t0 + lane;
    if (col < block_size) {
#pragma unroll 8
      for (int i = 0; i < kTile; ++i) {
        const int64_t flat = (b0 + i) * block_size + col;
        if (b0 + i < blocks && flat < count) g[flat] = slot[i][lane];
      }
    }
    __syncwarp();
  }
  // the 32 block sums of this warp, added in double by a fixed butterfly: one value per warp
  // for the final reduction instead of one per block
  double warp_square = live ? (double)block_square : 0.0;
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) warp_square += __shfl_xor_sync(0xffffffffu, warp_square, offset);
  if (lane == 0) block_partial[blockIdx.x] = warp_square;
  if (live) {
    moment_scale[block] = __half_as_ushort(__float2half_rn(maximum / 127.0f));
  }
}

// Global moment RMS and the coordinate step (cpu.cpp:736-741).  One block.
__global__ void __launch_bounds__(1024)
finish_moment_norm_kernel(const double* __restrict__ block_partial, int64_t partials, int64_t blocks,
                          int64_t block_size, float coordinate_lr, UpdateScalars* scalars,
                          const uint8_t* update_enabled) {
  if (disabled(update_enabled)) return;
  __shared__ double shared[1024];
  double local = 0.0;
  for (int64_t b = threadIdx.x; b < partials; b += blockDim.x) local += block_partial[b];
  const double moment_square_sum = block_sum_double(local, shared);
  if (threadIdx.x == 0) {
    const float moment_rms =
        sqrtf(fmaxf((float)(moment_square_sum / (double)(blocks * block_size)), 1e-16f));
    scalars->moment_rms = moment_rms;
    scalars->coordinate_step = coordinate_lr / moment_rms;
  }
}

// ---------------------------------------------------------------------------
// Pass 4: stochastic rounding, moment requantisation, sign repack, flips
// (cpu.cpp:746-807).  One thread per packed byte: 8 coordinates.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t scramble(uint32_t value) {
  value = (value ^ 61u) ^ (value >> 16);
  value += value << 3;
  value ^= value >> 4;
  value *= 0x27d4eb2du;
  value ^= value >> 15;
  return value;
}

// Pass 4 for whole bytes (C % 8 == 0) and power-of-two blocks of at least 8 elements: byte q
// holds elements 8q .. 8q + 7 of one block.  Same arithmetic as coordinate_and_pack_kernel below,
// without its index bookkeeping, and with the loads of a thread's next byte issued before the
// current one is worked on: the kernel is bound by memory latency, not by bandwidth or issue.
//
// Conversions and roundings go through the few XU lanes of an SM, so they are done with fp32
// additions wherever those give the same value: adding and subtracting 1.5 * 2^23 rounds a float
// of magnitude < 2^22 to the nearest-even integer (what rintf does), and the low mantissa bits of
// integer + 1.5 * 2^23 are that integer.
struct PackInputs {
  float4 lo, hi;
  uint2 coordinate;
  unsigned short scale;
  uint8_t bits;
};

__global__ void __launch_bounds__(256)
coordinate_and_pack_fast_kernel(const float* __restrict__ moment, int8_t* __restrict__ coordinate,
                                uint8_t* __restrict__ packed, int8_t* __restrict__ moment_q,
                                const uint16_t* __restrict__ moment_scale, int64_t total, int block_shift,
                                uint32_t seed_hash, int64_t step_host, const int64_t* __restrict__ step_device,
                                UpdateScalars* scalars, const uint8_t* update_enabled) {
  if (disabled(update_enabled)) return;
  const int64_t step = step_device ? *step_device : step_host;
  const uint32_t hash_seed = seed_hash ^ scramble((uint32_t)step ^ 0x2545f491u);
  const float coordinate_step = scalars->coordinate_step;
  constexpr float kMagic = 12582912.0f;
  constexpr int kMagicBits = 0x4b400000;
  auto load = [&](int64_t q) {
    PackInputs in;
    const int64_t base = q * 8;
    in.lo = *reinterpret_cast<const float4*>(moment + base);
    in.hi = *reinterpret_cast<const float4*>(moment + base + 4);
    in.coordinate = *reinterpret_cast<const uint2*>(coordinate + base);
    in.scale = moment_scale[base >> block_shift];
    in.bits = packed[q];
    return in;
  };
  int local_flips = 0;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t q = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  PackInputs current = {}, following = {};
  if (q < total) current = load(q);
  while (q < total) {
    const int64_t next_q = q + stride;
    if (next_q < total) following = load(next_q);
    const int64_t base = q * 8;
    const float m[8] = {current.lo.x, current.lo.y, current.lo.z, current.lo.w,
                        current.hi.x, current.hi.y, current.hi.z, current.hi.w};  // constant indices below
    const uint2 old_c = current.coordinate;
    const float inverse_scale = 1.0f / fmaxf(__half2float(__ushort_as_half(current.scale)), 1e-12f);
    const uint32_t index = (uint32_t)base;
    unsigned next = 0;
    uint32_t c_lo = 0u, c_hi = 0u, m_lo = 0u, m_hi = 0u;  // scalars: arrays here end up in local memory
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int old_value = (int)(int8_t)(((e < 4 ? old_c.x : old_c.y) >> (8 * (e & 3))) & 0xffu);
      const float old_float = __int_as_float(kMagicBits + old_value) - kMagic;
      const float target = old_float - m[e] * coordinate_step;
      float lower;
      if (fabsf(target) < 4194304.0f) {
        const float nearest = (target + kMagic) - kMagic;
        lower = nearest - (nearest > target ? 1.0f : 0.0f);
      } else {
        lower = floorf(target);
      }
      const float uniform = __uint2float_rn(scramble((index + e) ^ hash_seed)) * (1.0f / 4294967296.0f);
      const float rounded = lower + (uniform < (target - lower) ? 1.0f : 0.0f);
      const int new_c = __float_as_int(fminf(127.0f, fmaxf(-127.0f, rounded)) + kMagic) - kMagicBits;
      // clamping before rounding gives the same integer: the bounds are integers themselves
      const float scaled = fminf(127.0f, fmaxf(-127.0f, m[e] * inverse_scale));
      const int new_m = __float_as_int(scaled + kMagic) - kMagicBits;
      if (new_c >= 0) next |= 1u << e;
      const uint32_t c_byte = ((uint32_t)new_c & 0xffu) << (8 * (e & 3));
      const uint32_t m_byte = ((uint32_t)new_m & 0xffu) << (8 * (e & 3));
      if (e < 4) { c_lo |= c_byte; m_lo |= m_byte; } else { c_hi |= c_byte; m_hi |= m_byte; }
    }
    *reinterpret_cast<uint2*>(coordinate + base) = make_uint2(c_lo, c_hi);
    *reinterpret_cast<uint2*>(moment_q + base) = make_uint2(m_lo, m_hi);
    local_flips += __popc((unsigned)current.bits ^ next);
    packed[q] = (uint8_t)next;
    current = following;
    q = next_q;
  }
  // integer sum: any order gives the same total
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1)
    local_flips += __shfl_xor_sync(0xffffffffu, local_flips, offset);
  if ((threadIdx.x & 31) == 0 && local_flips)
    atomicAdd(reinterpret_cast<unsigned long long*>(&scalars->flips), (unsigned long long)local_flips);
}

// The same step when the moment pass did NOT write the moments back (moment_vec_kernel<true,
// false>): `evidence` still holds the reduced evidence, and the moment of an element is formed
// again here, operation for operation as the moment pass formed it --
//     u = (g * row_factor) * column_factor,   m = moment_q * (old_scale * beta1) + u * gain
// -- so the bits are the same and the matrix of fp32 moments (4 bytes per coordinate written by
// one kernel and read by the next) never exists.  `new_scale` holds the block scales the moment
// pass derived; `moment_scale` still holds the old ones and is overwritten afterwards
// (commit_scales_kernel).  Needs C % 8 == 0 and a power-of-two block of at least 8.
struct LeanInputs {
  float4 lo, hi, factor_lo, factor_hi;
  uint2 coordinate, moment;
  float row_factor;
  unsigned short old_scale, new_scale;
  uint8_t bits;
};

__global__ void __launch_bounds__(256)
coordinate_and_pack_lean_kernel(const float* __restrict__ evidence, int8_t* __restrict__ coordinate,
                                uint8_t* __restrict__ packed, int8_t* __restrict__ moment_q,
                                const uint16_t* __restrict__ moment_scale, const uint16_t* __restrict__ new_scale,
                                const float* __restrict__ row_factor, const float* __restrict__ column_factor,
                                int64_t total, int64_t C8, int block_shift, float beta1, uint32_t seed_hash,
                                int64_t step_host, const int64_t* __restrict__ step_device, UpdateScalars* scalars,
                                const uint8_t* update_enabled) {
  if (disabled(update_enabled)) return;
  const int64_t step = step_device ? *step_device : step_host;
  const uint32_t hash_seed = seed_hash ^ scramble((uint32_t)step ^ 0x2545f491u);
  const float coordinate_step = scalars->coordinate_step;
  const float gain = scalars->gain;
  constexpr float kMagic = 12582912.0f;
  constexpr int kMagicBits = 0x4b400000;
  auto load = [&](int64_t q, int64_t row, int64_t column8) {
    LeanInputs in;
    const int64_t base = q * 8;
    in.lo = *reinterpret_cast<const float4*>(evidence + base);
    in.hi = *reinterpret_cast<const float4*>(evidence + base + 4);
    in.factor_lo = *reinterpret_cast<const float4*>(column_factor + column8 * 8);
    in.factor_hi = *reinterpret_cast<const float4*>(column_factor + column8 * 8 + 4);
    in.row_factor = row_factor[row];
    in.coordinate = *reinterpret_cast<const uint2*>(coordinate + base);
    in.moment = *reinterpret_cast<const uint2*>(moment_q + base);
    in.old_scale = moment_scale[base >> block_shift];
    in.new_scale = new_scale[base >> block_shift];
    in.bits = packed[q];
    return in;
  };
  int local_flips = 0;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t stride_rows = stride / C8, stride_columns = stride - stride_rows * C8;
  int64_t q = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t row = q / C8, column8 = q - row * C8;
  LeanInputs current = {}, following = {};
  if (q < total) current = load(q, row, column8);
  while (q < total) {
    const int64_t next_q = q + stride;
    row += stride_rows;
    column8 += stride_columns;
    if (column8 >= C8) { column8 -= C8; ++row; }
    if (next_q < total) following = load(next_q, row, column8);
    const int64_t base = q * 8;
    const float g[8] = {current.lo.x, current.lo.y, current.lo.z, current.lo.w,
                        current.hi.x, current.hi.y, current.hi.z, current.hi.w};  // constant indices below
    const float cf[8] = {current.factor_lo.x, current.factor_lo.y, current.factor_lo.z, current.factor_lo.w,
                         current.factor_hi.x, current.factor_hi.y, current.factor_hi.z, current.factor_hi.w};
    const uint2 old_c = current.coordinate, old_m = current.moment;
    const float decay = __half2float(__ushort_as_half(current.old_scale)) * beta1;
    const float inverse_scale = 1.0f / fmaxf(__half2float(__ushort_as_half(current.new_scale)), 1e-12f);
    const float rf = current.row_factor;
    const uint32_t index = (uint32_t)base;
    unsigned next = 0;
    uint32_t c_lo = 0u, c_hi = 0u, m_lo = 0u, m_hi = 0u;  // scalars: arrays here end up in local memory
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int old_value = (int)(int8_t)(((e < 4 ? old_c.x : old_c.y) >> (8 * (e & 3))) & 0xffu);
      const int old_moment = (int)(int8_t)(((e < 4 ? old_m.x : old_m.y) >> (8 * (e & 3))) & 0xffu);
      const float update = g[e] * rf * cf[e];
      const float m = (float)old_moment * decay + update * gain;
      const float old_float = __int_as_float(kMagicBits + old_value) - kMagic;
      const float target = old_float - m * coordinate_step;
      float lower;
      if (fabsf(target) < 4194304.0f) {
        const float nearest = (target + kMagic) - kMagic;
        lower = nearest - (nearest > target ? 1.0f : 0.0f);
      } else {
        lower = floorf(target);
      }
      const float uniform = __uint2float_rn(scramble((index + e) ^ hash_seed)) * (1.0f / 4294967296.0f);
      const float rounded = lower + (uniform < (target - lower) ? 1.0f : 0.0f);
      const int new_c = __float_as_int(fminf(127.0f, fmaxf(-127.0f, rounded)) + kMagic) - kMagicBits;
      const float scaled = fminf(127.0f, fmaxf(-127.0f, m * inverse_scale));
      const int new_m = __float_as_int(scaled + kMagic) - kMagicBits;
      if (new_c >= 0) next |= 1u << e;
      const uint32_t c_byte = ((uint32_t)new_c & 0xffu) << (8 * (e & 3));
      const uint32_t m_byte = ((uint32_t)new_m & 0xffu) << (8 * (e & 3));
      if (e < 4) { c_lo |= c_byte; m_lo |= m_byte; } else { c_hi |= c_byte; m_hi |= m_byte; }
    }
    *reinterpret_cast<uint2*>(coordinate + base) = make_uint2(c_lo, c_hi);
    *reinterpret_cast<uint2*>(moment_q + base) = make_uint2(m_lo, m_hi);
    local_flips += __popc((unsigned)current.bits ^ next);
    packed[q] = (uint8_t)next;
    current = following;
    q = next_q;
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1)
    local_flips += __shfl_xor_sync(0xffffffffu, local_flips, offset);
  if ((threadIdx.x & 31) == 0 && local_flips)
    atomicAdd(reinterpret_cast<unsigned long long*>(&scalars->flips), (unsigned long long)local_flips);
}

// the block scales of this step take the place of the old ones once every element has used both
__global__ void __launch_bounds__(256)
commit_scales_kernel(const uint16_t* __restrict__ new_scale, uint16_t* __restrict__ moment_scale, int64_t blocks,
                     const uint8_t* update_enabled) {
  if (disabled(update_enabled)) return;
  for (int64_t b = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; b < blocks; b += (int64_t)gridDim.x * blockDim.x)
    moment_scale[b] = new_scale[b];
}

__global__ void __launch_bounds__(256)
coordinate_and_pack_kernel(const float* __restrict__ moment, int8_t* __restrict__ coordinate,
                           uint8_t* __restrict__ packed, int8_t* __restrict__ moment_q,
                           const uint16_t* __restrict__ moment_scale, int64_t R, int64_t C,
                           int block_shift, int64_t block_size, uint32_t seed_hash, int64_t step_host,
                           const int64_t* __restrict__ step_device, UpdateScalars* scalars,
                           const uint8_t* update_enabled) {
  if (disabled(update_enabled)) return;
  const int64_t stride = (C + 7) >> 3;
  const int64_t total = R * stride;
  const int64_t step = step_device ? *step_device : step_host;
  const uint32_t hash_seed = seed_hash ^ scramble((uint32_t)step ^ 0x2545f491u);
  const float coordinate_step = scalars->coordinate_step;
  const bool vector_ok = (C & 7) == 0;
  int local_flips = 0;
  for (int64_t q = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; q < total;
       q += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = q / stride, byte = q - row * stride;
    const int64_t column0 = byte * 8;
    const int64_t base = row * C + column0;
    const int limit = (C - column0) < 8 ? (int)(C - column0) : 8;
    float m[8];
    int8_t c8[8];
    if (vector_ok) {
      const float4 lo = *reinterpret_cast<const float4*>(moment + base);
      const float4 hi = *reinterpret_cast<const float4*>(moment + base + 4);
      m[0] = lo.x; m[1] = lo.y; m[2] = lo.z; m[3] = lo.w;
      m[4] = hi.x; m[5] = hi.y; m[6] = hi.z; m[7] = hi.w;
      *reinterpret_cast<uint2*>(c8) = *reinterpret_cast<const uint2*>(coordinate + base);
    } else {
      for (int e = 0; e < 8; ++e) {
        m[e] = e < limit ? moment[base + e] : 0.0f;
        c8[e] = e < limit ? coordinate[base + e] : (int8_t)0;
      }
    }
    int8_t new_c[8], new_m[8];
    unsigned next = 0;
    int64_t cached_block = -1;
    float inverse_scale = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      if (e < limit) {
        const int64_t i = base + e;
        const int64_t block = block_shift >= 0 ? (i >> block_shift) : (i / block_size);
        if (block != cached_block) {
          cached_block = block;
          inverse_scale =
              1.0f / fmaxf(__half2float(__ushort_as_half(moment_scale[block])), 1e-12f);
        }
        const float target = (float)c8[e] - m[e] * coordinate_step;
        const float lower = floorf(target);
        const float uniform = __uint2float_rn(scramble((uint32_t)i ^ hash_seed)) * (1.0f / 4294967296.0f);
        const float rounded = lower + (uniform < (target - lower) ? 1.0f : 0.0f);
        new_c[e] = (int8_t)fminf(127.0f, fmaxf(-127.0f, rounded));
        new_m[e] = (int8_t)fminf(127.0f, fmaxf(-127.0f, rintf(m[e] * inverse_scale)));
        if (new_c[e] >= 0) next |= 1u << e;
      } else {
        new_c[e] = 0;
        new_m[e] = 0;
      }
    }
    if (vector_ok) {
      *reinterpret_cast<uint2*>(coordinate + base) = *reinterpret_cast<const uint2*>(new_c);
      *reinterpret_cast<uint2*>(moment_q + base) = *reinterpret_cast<const uint2*>(new_m);
    } else {
      for (int e = 0; e < limit; ++e) {
        coordinate[base + e] = new_c[e];
        moment_q[base + e] = new_m[e];
      }
    }
    const unsigned mask = limit >= 8 ? 0xffu : ((1u << limit) - 1u);
    const unsigned previous = packed[q];
    local_flips += __popc((previous ^ next) & mask);
    packed[q] = (uint8_t)((previous & ~mask & 0xffu) | next);
  }
  // integer sum: any order gives the same total
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1)
    local_flips += __shfl_xor_sync(0xffffffffu, local_flips, offset);
  if ((threadIdx.x & 31) == 0 && local_flips)
    atomicAdd(reinterpret_cast<unsigned long long*>(&scalars->flips), (unsigned long long)local_flips);
}

// ---------------------------------------------------------------------------
// Vectorised variants of the four tile-walking kernels
// ---------------------------------------------------------------------------
//
// Same chains, same arithmetic, same order -- only the data movement differs.  When rows are
// 16-byte aligned (columns % 4 == 0, block_size % 32 == 0) a 32 x 32 tile is filled with eight
// 16-byte cp.async per lane (four full 128-byte lines per instruction) instead of 32 four-byte
// ones, into an unpadded tile whose 16-byte chunks are XOR-swizzled by (row % 8):
//     element (r, c) lives at word  ((c / 4) ^ (r % 8)) * 4 + c % 4  of row r.
// A lane that owns ROW r then reads its 32 values with eight conflict-free 128-bit loads, a lane
// that owns COLUMN c reads one word per row, also conflict-free, and tiles that are rewritten
// (normalised evidence, moments) go back to global memory as full 128-byte lines.

__device__ __forceinline__ void cp_async16(void* smem, const void* global) {
  const unsigned address = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(address), "l"(global) : "memory");
}

__device__ __forceinline__ void issue_tile16(float (*slot)[kTile], const float* __restrict__ g,
                                             int64_t ld, int64_t r0, int64_t c0, int64_t R, int64_t C,
                                             int64_t limit, int lane) {
  const int chunk = lane & 7;
  const int64_t col = c0 + chunk * 4;
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const int row = q * 4 + (lane >> 3);
    const int64_t flat = (r0 + row) * ld + col;
    float* destination = &slot[row][(chunk ^ (row & 7)) << 2];
    if (r0 + row < R && col < C && flat < limit)
      cp_async16(destination, g + flat);
    else
      *reinterpret_cast<float4*>(destination) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  }
  cp_async_commit();
}

// full 128-byte lines of a rewritten tile back to global memory
__device__ __forceinline__ void drain_tile16(float (*slot)[kTile], float* __restrict__ g, int64_t ld,
                                             int64_t r0, int64_t c0, int64_t R, int64_t C,
                                             int64_t limit, int lane) {
  const int chunk = lane & 7;
  const int64_t col = c0 + chunk * 4;
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const int row = q * 4 + (lane >> 3);
    const int64_t flat = (r0 + row) * ld + col;
    if (r0 + row < R && col < C && flat < limit)
      *reinterpret_cast<float4*>(g + flat) =
          *reinterpret_cast<const float4*>(&slot[row][(chunk ^ (row & 7)) << 2]);
  }
}

#define QSTE_TILE_LOOP(ISSUE)                                              \
  for (int64_t t = 0; t < kStages - 1; ++t) {                              \
    if (t < tiles) { ISSUE(t); } else cp_async_commit();                   \
  }                                                                        \
  for (int64_t t = 0; t < tiles; ++t) {                                    \
    if (t + kStages - 1 < tiles) { ISSUE(t + kStages - 1); } else cp_async_commit(); \
    cp_async_wait<kStages - 1>();                                          \
    __syncwarp();

// one warp: the sums of squares of rows 32 * tile .. + 31, and their moving average
__device__ __forceinline__ void row_squares_tile(float (*ring)[kTile][kTile], const float* __restrict__ g, int64_t R,
                                                 int64_t C, uint16_t* __restrict__ row_v,
                                                 float* __restrict__ row_stats, float beta2, int64_t tile, int lane) {
  const int64_t r0 = tile * kTile;
  const int64_t tiles = (C + kTile - 1) / kTile;
  const int64_t limit = R * C;
  float total = 0.0f;
#define ISSUE_ROW(T) issue_tile16(ring[(T) % kStages], g, C, r0, (T) * kTile, R, C, limit, lane)
  QSTE_TILE_LOOP(ISSUE_ROW)
    const float* line = ring[t % kStages][lane];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 v = *reinterpret_cast<const float4*>(line + ((j ^ (lane & 7)) << 2));
      float square = v.x * v.x; total += square;
      square = v.y * v.y; total += square;
      square = v.z * v.z; total += square;
      square = v.w * v.w; total += square;
    }
    __syncwarp();
  }
#undef ISSUE_ROW
  const int64_t row = r0 + lane;
  if (row < R) {
    const float previous = __half2float(__ushort_as_half(row_v[row]));
    const float updated = previous * beta2 + (total / (float)C + 1e-12f) * (1.0f - beta2);
    row_stats[row] = updated;
    row_v[row] = __half_as_ushort(__float2half_rn(updated));
  }
}

__global__ void __launch_bounds__(32)
row_squares_vec_kernel(const float* __restrict__ g, int64_t R, int64_t C, uint16_t* __restrict__ row_v,
                       float* __restrict__ row_stats, float beta2, const uint8_t* update_enabled) {
  if (disabled(update_enabled)) return;
  __shared__ __align__(16) float ring[kStages][kTile][kTile];
  row_squares_tile(ring, g, R, C, row_v, row_stats, beta2, blockIdx.x, threadIdx.x);
}

__global__ void __launch_bounds__(32)
column_squares_vec_kernel(const float* __restrict__ g, int64_t R, int64_t C,
                          float* __restrict__ column_sum, const uint8_t* update_enabled) {
  if (disabled(update_enabled)) return;
  __shared__ __align__(16) float ring[kStages][kTile][kTile];
  const int lane = threadIdx.x;
  const int64_t c0 = (int64_t)blockIdx.x * kTile;
  const int64_t tiles = (R + kTile - 1) / kTile;
  const int64_t limit = R * C;
  float total = 0.0f;
#define ISSUE_COLUMN(T) issue_tile16(ring[(T) % kStages], g, C, (T) * kTile, c0, R, C, limit, lane)
  QSTE_TILE_LOOP(ISSUE_COLUMN)
    float (*slot)[kTile] = ring[t % kStages];
#pragma unroll
    for (int i = 0; i < kTile; ++i) {
      const float value = slot[i][(((lane >> 2) ^ (i & 7)) << 2) | (lane & 3)];
      const float square = value * value;
      total += square;
    }
    __syncwarp();
  }
#undef ISSUE_COLUMN
  if (c0 + lane < C) column_sum[c0 + lane] = total;
}

// column_squares_vec_kernel for matrices whose sides are multiples of 32: no bounds tests, and
// every address that does not depend on the tile is computed once.  With one chain per column
// there are only C / 32 warps, fewer than SMs at the sizes that matter, so what counts is the
// number of instructions a warp spends per row beside the chain's own add.
__device__ __forceinline__ void column_squares_strip(float (*ring)[kTile][kTile], const float* __restrict__ g,
                                                     int64_t R, int64_t C, float* __restrict__ column_sum,
                                                     int64_t strip, int lane) {
  const int64_t c0 = strip * kTile;
  const int tiles = (int)(R / kTile);
  // this lane copies 16 bytes of rows lane / 8, lane / 8 + 4, ... of a tile
  const int chunk = lane & 7, sub = lane >> 3;
  const float* source = g + (int64_t)sub * C + c0 + chunk * 4;
  const int64_t row_step = 4 * C, tile_step = (int64_t)kTile * C;
  const unsigned ring_base = (unsigned)__cvta_generic_to_shared(&ring[0][0][0]);
  unsigned destination[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const int row = q * 4 + sub;
    destination[q] = (unsigned)(row * kTile * 4 + ((chunk ^ (row & 7)) << 4));
  }
  auto issue = [&](int t) {
    const float* tile_source = source + t * tile_step;
    const unsigned slot = ring_base + (unsigned)(t % kStages) * (kTile * kTile * 4);
#pragma unroll
    for (int q = 0; q < 8; ++q)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(slot + destination[q]),
                   "l"(tile_source + q * row_step) : "memory");
    cp_async_commit();
  };
  // word of column `lane` inside row i of a slot: the 16-byte chunks of a row are XOR-swizzled by i % 8
  int word[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) word[k] = (((lane >> 2) ^ k) << 2) | (lane & 3);
  for (int t = 0; t < kStages - 1; ++t) {
    if (t < tiles) issue(t); else cp_async_commit();
  }
  float total = 0.0f;
  for (int t = 0; t < tiles; ++t) {
    if (t + kStages - 1 < tiles) issue(t + kStages - 1); else cp_async_commit();
    cp_async_wait<kStages - 1>();
    __syncwarp();
    const float* slot = &ring[t % kStages][0][0];
#pragma unroll
    for (int i = 0; i < kTile; ++i) {
      const float value = slot[i * kTile + word[i & 7]];
      const float square = value * value;
      total += square;
    }
    __syncwarp();
  }
  column_sum[c0 + lane] = total;
}

__global__ void __launch_bounds__(32)
column_squares_interior_kernel(const float* __restrict__ g, int64_t R, int64_t C,
                               float* __restrict__ column_sum, const uint8_t* update_enabled) {
  if (disabled(update_enabled)) return;
  __shared__ __align__(16) float ring[kStages][kTile][kTile];
  column_squares_strip(ring, g, R, C, column_sum, blockIdx.x, threadIdx.x);
}

// Both factor sums in one launch: CTAs [0, C / 32) are the column strips -- few, long, and light
// on bandwidth -- and the rest the row tiles, which are many, short and bandwidth-hungry, in the
// SMs' spare room.  The two read the evidence independently, so side by side they take about as
// long as the slower one instead of the sum of both.
__global__ void __launch_bounds__(32)
factor_sums_kernel(const float* __restrict__ g, int64_t R, int64_t C, float* __restrict__ column_sum,
                   uint16_t* __restrict__ row_v, float* __restrict__ row_stats, float beta2,
                   const uint8_t* update_enabled) {
  if (disabled(update_enabled)) return;
  __shared__ __align__(16) float ring[kStages][kTile][kTile];
  const int64_t column_tiles = C / kTile;
  if (blockIdx.x < column_tiles)
    column_squares_strip(ring, g, R, C, column_sum, blockIdx.x, threadIdx.x);
  else
    row_squares_tile(ring, g, R, C, row_v, row_stats, beta2, blockIdx.x - column_tiles, threadIdx.x);
}

__global__ void __launch_bounds__(32)
precondition_vec_kernel(float* __restrict__ g, int64_t R, int64_t C, const float* __restrict__ row_factor,
                        const float* __restrict__ column_factor, double* __restrict__ row_partial,
                        const uint8_t* update_enabled) {
  if (disabled(update_enabled)) return;
  __shared__ __align__(16) float ring[kStages][kTile][kTile];
  const int lane = threadIdx.x;
  const int64_t r0 = (int64_t)blockIdx.x * kTile;
  const int64_t tiles = (C + kTile - 1) / kTile;
  const int64_t limit = R * C;
  const int64_t row = r0 + lane;
  const float multiplier = row < R ? row_factor[row] : 0.0f;
  float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;  // columns % 4 == 0: no ragged tail
#define ISSUE_ROW(T) issue_tile16(ring[(T) % kStages], g, C, r0, (T) * kTile, R, C, limit, lane)
  QSTE_TILE_LOOP(ISSUE_ROW)
    float (*slot)[kTile] = ring[t % kStages];
    float* line = slot[lane];
    const int64_t c0 = t * kTile;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float4 factor = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (c0 + 4 * j < C) factor = *reinterpret_cast<const float4*>(column_factor + c0 + 4 * j);
      float4* cell = reinterpret_cast<float4*>(line + ((j ^ (lane & 7)) << 2));
      const float4 v = *cell;
      float4 u;
      u.x = v.x * multiplier * factor.x;
      u.y = v.y * multiplier * factor.y;
      u.z = v.z * multiplier * factor.z;
      u.w = v.w * multiplier * factor.w;
      *cell = u;
      float square = u.x * u.x; a0 += square;
      square = u.y * u.y; a1 += square;
      square = u.z * u.z; a2 += square;
      square = u.w * u.w; a3 += square;
    }
    __syncwarp();
    drain_tile16(slot, g, C, r0, c0, R, C, limit, lane);
    __syncwarp();
  }
#undef ISSUE_ROW
  if (row < R) row_partial[row] = (double)(a0 + a1) + (double)(a2 + a3);
}

// Pass 2 without a write-back, four lanes per row.  The reference splits a row's sum of squares
// into four strided chains (columns 4i + j, j = 0..3); here lane (r, j) = (lane / 4, lane % 4) of a
// warp owns chain j of row r, so a warp covers 8 rows and there are four times as many warps as
// with one lane per row -- the kernel is bound by the latency of those chains, and the number of
// warps is what hides it.  A stage holds 128 columns of the 8 rows plus the 128 column factors
// (a ninth "row"); rows are 16 bytes further apart than their length, which keeps the quads of
// the 8 rows on different banks.
constexpr int kQuadStages = 3;
constexpr int kQuadColumns = 128;
constexpr int kQuadPitch = kQuadColumns + 4;

__global__ void __launch_bounds__(32)
precondition_quad_kernel(const float* __restrict__ g, int64_t R, int64_t C, const float* __restrict__ row_factor,
                         const float* __restrict__ column_factor, double* __restrict__ row_partial,
                         const uint8_t* update_enabled) {
  if (disabled(update_enabled)) return;
  __shared__ __align__(16) float ring[kQuadStages][9][kQuadPitch];
  const int lane = threadIdx.x;
  const int r = lane >> 2, j = lane & 3;
  const int64_t r0 = (int64_t)blockIdx.x * 8;
  const int64_t row = r0 + r;
  const int64_t tiles = (C + kQuadColumns - 1) / kQuadColumns;
  const float multiplier = row < R ? row_factor[row] : 0.0f;
  // lane l fetches 16-byte chunk l of each of the 8 rows and of the factors; past C: zeros
  auto issue = [&](int64_t t) {
    float (*slot)[kQuadPitch] = ring[t % kQuadStages];
    const int64_t c = t * kQuadColumns + lane * 4;
#pragma unroll
    for (int rr = 0; rr < 9; ++rr) {
      float* destination = &slot[rr][lane * 4];
      const bool inside = c < C && (rr == 8 || r0 + rr < R);
      if (inside)
        cp_async16(destination, rr == 8 ? column_factor + c : g + (r0 + rr) * C + c);
      else
        *reinterpret_cast<float4*>(destination) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    cp_async_commit();
  };
  for (int64_t t = 0; t < kQuadStages - 1; ++t) {
    if (t < tiles) issue(t); else cp_async_commit();
  }
  float a = 0.0f;
  for (int64_t t = 0; t < tiles; ++t) {
    if (t + kQuadStages - 1 < tiles) issue(t + kQuadStages - 1); else cp_async_commit();
    cp_async_wait<kQuadStages - 1>();
    __syncwarp();
    const float* line = ring[t % kQuadStages][r] + j;
    const float* factors = ring[t % kQuadStages][8] + j;
#pragma unroll
    for (int i = 0; i < kQuadColumns / 4; ++i) {
      const float update = line[4 * i] * multiplier * factors[4 * i];
      const float square = update * update;
      a += square;
    }
    __syncwarp();
  }
  const int base = lane & ~3;
  const float a0 = __shfl_sync(0xffffffffu, a, base);
  const float a1 = __shfl_sync(0xffffffffu, a, base + 1);
  const float a2 = __shfl_sync(0xffffffffu, a, base + 2);
  const float a3 = __shfl_sync(0xffffffffu, a, base + 3);
  if (j == 0 && row < R) row_partial[row] = (double)(a0 + a1) + (double)(a2 + a3);
}

// kRecompute = true: g still holds the evidence; the normalised update (g * row_factor) *
// column_factor is formed here, exactly as precondition_vec_kernel forms it (needs C % 4 == 0,
// so that four consecutive elements share a row).
// kWriteBack = false (only with kRecompute): the moments are not stored -- the last pass forms them
// again from the evidence (coordinate_and_pack_lean_kernel) -- and the new block scales go to
// `scale_out` instead of replacing the old ones, which that pass still needs.
template <bool kRecompute, bool kWriteBack>
__global__ void __launch_bounds__(32)
moment_vec_kernel(float* __restrict__ g, const int8_t* __restrict__ moment_q,
                  uint16_t* __restrict__ moment_scale, uint16_t* __restrict__ scale_out, int64_t count, int64_t block_size, int64_t blocks,
                  float beta1, const UpdateScalars* __restrict__ scalars,
                  double* __restrict__ block_partial, const uint8_t* update_enabled, int64_t C,
                  const float* __restrict__ row_factor, const float* __restrict__ column_factor) {
  if (disabled(update_enabled)) return;
  // A block is only block_size / 32 tiles long and there are many blocks: a shallow ring leaves
  // room for three times as many warps per SM, which is what hides the latency here.
  constexpr int kStages = 3;
  __shared__ __align__(16) float ring[kStages][kTile][kTile];
  const int lane = threadIdx.x;
  const int64_t b0 = (int64_t)blockIdx.x * kTile;
  const int64_t tiles = block_size / kTile;  // block_size % 32 == 0
  const int64_t block = b0 + lane;
  const bool live = block < blocks;
  const float old_scale = live ? __half2float(__ushort_as_half(moment_scale[block])) : 0.0f;
  const float decay = old_scale * beta1;
  const float gain = scalars->gain;
  float maximum = 1e-6f;
  float block_square = 0.0f;
  // int8 moments of this lane's block for one tile: 32 contiguous bytes
  auto load_previous = [&](int64_t tile, uint4& lo, uint4& hi, int& width) {
    const int64_t start = block * block_size + tile * kTile;
    width = 0;
    lo = make_uint4(0, 0, 0, 0);
    hi = lo;
    if (live && tile < tiles && start < count) {
      const int64_t left = count - start;
      width = left < kTile ? (int)left : kTile;
      if (width == kTile) {
        lo = *reinterpret_cast<const uint4*>(moment_q + start);
        hi = *reinterpret_cast<const uint4*>(moment_q + start + 16);
      } else {
        __align__(16) int8_t scratch[kTile];
        for (int e = 0; e < kTile; ++e) scratch[e] = e < width ? moment_q[start + e] : (int8_t)0;
        lo = *reinterpret_cast<const uint4*>(scratch);
        hi = *reinterpret_cast<const uint4*>(scratch + 16);
      }
    }
  };
  uint4 next_lo, next_hi;
  int next_width;
  load_previous(0, next_lo, next_hi, next_width);
  // row and column of the next group of four elements of this lane's block
  int64_t walk_row = 0, walk_column = 0;
  float walk_factor = 0.0f;
  if (kRecompute && live) {
    const int64_t start = block * block_size;
    walk_row = start / C;
    walk_column = start - walk_row * C;
    walk_factor = start < count ? row_factor[walk_row] : 0.0f;
  }
#define ISSUE_BLOCK(T) issue_tile16(ring[(T) % kStages], g, block_size, b0, (T) * kTile, blocks, block_size, count, lane)
  QSTE_TILE_LOOP(ISSUE_BLOCK)
    const uint4 lo = next_lo, hi = next_hi;
    const int width = next_width;
    load_previous(t + 1, next_lo, next_hi, next_width);
    __align__(16) int8_t previous[kTile];
    *reinterpret_cast<uint4*>(previous) = lo;
    *reinterpret_cast<uint4*>(previous + 16) = hi;
    float (*slot)[kTile] = ring[t % kStages];
    float* line = slot[lane];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float4* cell = reinterpret_cast<float4*>(line + ((j ^ (lane & 7)) << 2));
      const float4 v = *cell;
      float values[4] = {v.x, v.y, v.z, v.w};
      if (kRecompute && 4 * j < width) {
        const float4 factor = *reinterpret_cast<const float4*>(column_factor + walk_column);
        values[0] = values[0] * walk_factor * factor.x;
        values[1] = values[1] * walk_factor * factor.y;
        values[2] = values[2] * walk_factor * factor.z;
        values[3] = values[3] * walk_factor * factor.w;
        walk_column += 4;
        if (walk_column >= C) {
          walk_column = 0;
          ++walk_row;
          walk_factor = walk_row * C < count ? row_factor[walk_row] : 0.0f;
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (4 * j + e < width) {
          const float moment = (float)previous[4 * j + e] * decay + values[e] * gain;
          values[e] = moment;
          block_square += moment * moment;
          maximum = fmaxf(maximum, fabsf(moment));
        }
      }
      if (kWriteBack) *cell = make_float4(values[0], values[1], values[2], values[3]);
    }
    __syncwarp();
    if (kWriteBack) {
      drain_tile16(slot, g, block_size, b0, t * kTile, blocks, block_size, count, lane);
      __syncwarp();
    }
  }
#undef ISSUE_BLOCK
  // the 32 block sums of this warp, added in double by a fixed butterfly: one value per warp
  // for the final reduction instead of one per block
  double warp_square = live ? (double)block_square : 0.0;
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) warp_square += __shfl_xor_sync(0xffffffffu, warp_square, offset);
  if (lane == 0) block_partial[blockIdx.x] = warp_square;
  if (live) {
    (kWriteBack ? moment_scale : scale_out)[block] = __half_as_ushort(__float2half_rn(maximum / 127.0f));
  }
}
#undef QSTE_TILE_LOOP

// ---------------------------------------------------------------------------
// The moment pass when nothing is written back, by direct loads (no shared-memory tiles)
// ---------------------------------------------------------------------------
//
// Once the moments are not stored (the lean path), the pass only READS: 4 bytes of evidence and
// one of the old moment per coordinate.  A lane still owns one block of 256 coordinates -- its
// sum of squares is one fp32 chain over the block in index order, as the reference forms it --
// but it now fetches its kilobyte of evidence itself, 32 bytes per load (a whole sector: lanes
// are a kilobyte apart, so nothing is shared between them), four loads of evidence and one of
// moments in flight per 32 coordinates.  No tile ring means no shared memory per warp beyond the
// column factors (staged once per CTA, padded by four floats per 256 so that the 32 lanes, whose
// blocks start 256 columns apart, read them without bank conflicts), so the SM holds as many
// warps as registers allow.  Requires block_size == 256 and columns % 256 == 0 (a block then
// lies inside one row).
__device__ __forceinline__ void ld_global_v8(const void* address, uint32_t* r) {
  asm volatile("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "l"(address));
}

constexpr int kDirectThreads = 256;

__global__ void __launch_bounds__(kDirectThreads)
moment_direct_kernel(const float* __restrict__ g, const int8_t* __restrict__ moment_q,
                     const uint16_t* __restrict__ moment_scale, uint16_t* __restrict__ scale_out, int64_t blocks,
                     int64_t C, float beta1, const UpdateScalars* __restrict__ scalars,
                     double* __restrict__ block_partial, const uint8_t* update_enabled,
                     const float* __restrict__ row_factor, const float* __restrict__ column_factor) {
  if (disabled(update_enabled)) return;
  extern __shared__ float factors[];   // column c at c + 4 * (c / 256)
  for (int64_t c = threadIdx.x * 4; c < C; c += kDirectThreads * 4)
    *reinterpret_cast<float4*>(factors + c + 4 * (c >> 8)) = *reinterpret_cast<const float4*>(column_factor + c);
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (kDirectThreads / 32) + (threadIdx.x >> 5);
  const int64_t block = warp * 32 + lane;
  const bool live = block < blocks;
  const int64_t start = (live ? block : 0) * 256;
  const int64_t row = start / C;
  const int64_t column0 = start - row * C;
  const float multiplier = row_factor[row];
  const float decay = __half2float(__ushort_as_half(moment_scale[live ? block : 0])) * beta1;
  const float gain = scalars->gain;
  const float* source = g + start;
  const int8_t* previous = moment_q + start;
  const float* factor = factors + column0 + 4 * (column0 >> 8);
  float maximum = 1e-6f;
  float block_square = 0.0f;
#pragma unroll 2
  for (int piece = 0; piece < 8; ++piece) {      // 32 coordinates per piece
    uint32_t raw[4][8], old[8];
#pragma unroll
    for (int v = 0; v < 4; ++v) ld_global_v8(source + piece * 32 + v * 8, raw[v]);
    ld_global_v8(previous + piece * 32, old);
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const float4 f0 = *reinterpret_cast<const float4*>(factor + piece * 32 + v * 8);
      const float4 f1 = *reinterpret_cast<const float4*>(factor + piece * 32 + v * 8 + 4);
      const float cf[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int index = v * 8 + e;
        const int q = (int)(int8_t)((old[index >> 2] >> (8 * (index & 3))) & 0xffu);
        const float update = __uint_as_float(raw[v][e]) * multiplier * cf[e];
        const float moment = (float)q * decay + update * gain;
        block_square += moment * moment;
        maximum = fmaxf(maximum, fabsf(moment));
      }
    }
  }
  // the 32 block sums of this warp, added in double by the same fixed butterfly as the tiled kernel
  double warp_square = live ? (double)block_square : 0.0;
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) warp_square += __shfl_xor_sync(0xffffffffu, warp_square, offset);
  if (lane == 0 && warp * 32 < blocks) block_partial[warp] = warp_square;
  if (live) scale_out[block] = __half_as_ushort(__float2half_rn(maximum / 127.0f));
}

__global__ void publish_flips_kernel(const UpdateScalars* scalars, int64_t* flips_out,
                                     const uint8_t* update_enabled) {
  if (disabled(update_enabled)) { *flips_out = 0; return; }
  *flips_out = scalars->flips;
}

struct UpdateLayout {
  size_t scalars, column_sum, row_stats, row_factor, column_factor, row_partial, block_partial, new_scale, total;
};

static UpdateLayout layout_for(int64_t R, int64_t C, int64_t blocks) {
  UpdateLayout l;
  size_t at = 0;
  l.scalars = at; at = align_up(at + sizeof(UpdateScalars), 256);
  l.column_sum = at; at = align_up(at + sizeof(float) * (size_t)C, 256);
  l.row_stats = at; at = align_up(at + sizeof(float) * (size_t)R, 256);
  l.row_factor = at; at = align_up(at + sizeof(float) * (size_t)R, 256);
  l.column_factor = at; at = align_up(at + sizeof(float) * (size_t)C, 256);
  l.row_partial = at; at = align_up(at + sizeof(double) * (size_t)R, 256);
  l.block_partial = at; at = align_up(at + sizeof(double) * (size_t)blocks, 256);
  l.new_scale = at; at = align_up(at + sizeof(uint16_t) * (size_t)blocks, 256);
  l.total = at;
  return l;
}

// QSTE_B200_FACTOR_SUMS=separate: the row and the column sums of squares as two launches even when
// both sides are multiples of 32 (for A/B timing; one launch is 30 us faster at 14336 x 4096).
static bool separate_factor_sums() {
  static const bool separate = getenv("QSTE_B200_FACTOR_SUMS") != nullptr;
  return separate;
}

uint32_t host_scramble(uint32_t value) {
  value = (value ^ 61u) ^ (value >> 16);
  value += value << 3;
  value ^= value >> 4;
  value *= 0x27d4eb2du;
  value ^= value >> 15;
  return value;
}

// Enqueue the whole step with every scratch array carved out of `base`.
int run_coordinate_update(float* gradient, int8_t* coordinate, uint8_t* packed, int8_t* moment_q,
                          uint16_t* moment_scale, uint16_t* row_v, uint16_t* col_v, int64_t R,
                          int64_t C, double beta1_in, double beta2_in, double update_clip_in,
                          double coordinate_lr_in, int64_t block_size, int64_t seed, int64_t step,
                          const int64_t* step_device, const uint8_t* update_enabled,
                          int64_t* flips_out, char* base, cudaStream_t stream) {
  const int64_t count = R * C;
  const int64_t blocks = ceil_div(count, block_size);
  const UpdateLayout l = layout_for(R, C, blocks);
  UpdateScalars* scalars = reinterpret_cast<UpdateScalars*>(base + l.scalars);
  float* column_sum = reinterpret_cast<float*>(base + l.column_sum);
  float* row_stats = reinterpret_cast<float*>(base + l.row_stats);
  float* row_factor = reinterpret_cast<float*>(base + l.row_factor);
  float* column_factor = reinterpret_cast<float*>(base + l.column_factor);
  double* row_partial = reinterpret_cast<double*>(base + l.row_partial);
  double* block_partial = reinterpret_cast<double*>(base + l.block_partial);
  uint16_t* new_scale = reinterpret_cast<uint16_t*>(base + l.new_scale);
  const float beta1 = (float)beta1_in, beta2 = (float)beta2_in;
  const float update_clip = (float)update_clip_in, coordinate_lr = (float)coordinate_lr_in;

  const unsigned row_tiles = (unsigned)ceil_div(R, kTile);
  const unsigned column_tiles = (unsigned)ceil_div(C, kTile);
  const unsigned block_tiles = (unsigned)ceil_div(blocks, kTile);
  int launched_less = 0;

  // 16-byte aligned rows (of the matrix and of the [blocks, block_size] view): vectorised tiles
  const bool vec_rows = (C % 4 == 0) && aligned(gradient, 16);
  const bool vec_blocks = (block_size % 32 == 0) && (count % 4 == 0) && aligned(gradient, 16) &&
                          aligned(moment_q, 16);
  const bool interior = R % kTile == 0 && C % kTile == 0;
  if (vec_rows && interior && !separate_factor_sums()) {
    factor_sums_kernel<<<column_tiles + row_tiles, 32, 0, stream>>>(gradient, R, C, column_sum, row_v, row_stats, beta2,
                                                                    update_enabled);
    launched_less = 1;
  } else if (vec_rows) {
    row_squares_vec_kernel<<<row_tiles, 32, 0, stream>>>(gradient, R, C, row_v, row_stats, beta2, update_enabled);
    if (interior)
      column_squares_interior_kernel<<<column_tiles, 32, 0, stream>>>(gradient, R, C, column_sum, update_enabled);
    else
      column_squares_vec_kernel<<<column_tiles, 32, 0, stream>>>(gradient, R, C, column_sum, update_enabled);
  } else {
    row_squares_kernel<<<row_tiles, 32, 0, stream>>>(gradient, R, C, row_v, row_stats, beta2, update_enabled);
    column_squares_kernel<<<column_tiles, 32, 0, stream>>>(gradient, R, C, column_sum, update_enabled);
  }
  finish_factors_kernel<<<1, 1024, 0, stream>>>(column_sum, col_v, row_stats, row_factor, column_factor,
                                                R, C, beta2, scalars, update_enabled);
  const bool recompute = vec_rows && vec_blocks;  // the update is formed twice, never stored
  if (recompute)
    precondition_quad_kernel<<<(unsigned)((R + 7) / 8), 32, 0, stream>>>(gradient, R, C, row_factor, column_factor,
                                                                         row_partial, update_enabled);
  else if (vec_rows)
    precondition_vec_kernel<<<row_tiles, 32, 0, stream>>>(gradient, R, C, row_factor, column_factor,
                                                                row_partial, update_enabled);
  else
    precondition_kernel<<<row_tiles, 32, 0, stream>>>(gradient, R, C, row_factor, column_factor,
                                                      row_partial, update_enabled);
  finish_update_norm_kernel<<<1, 1024, 0, stream>>>(row_partial, R, count, beta1, update_clip, scalars,
                                                    update_enabled);
  int block_shift = -1;
  if ((block_size & (block_size - 1)) == 0) {
    block_shift = 0;
    while (((int64_t)1 << block_shift) < block_size) ++block_shift;
  }
  // lean: the fp32 moments are never stored; the last pass forms them again from the evidence
  const bool lean = recompute && (C & 7) == 0 && block_shift >= 3;
  const size_t factor_bytes = (size_t)(C + C / 64 + 8) * sizeof(float);
  const bool direct = lean && block_size == 256 && C % 256 == 0 && aligned(gradient, 32) && aligned(moment_q, 32) &&
                      factor_bytes <= 96 * 1024;
  if (direct) {
    static bool configured[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (factor_bytes > 48 * 1024 && (device < 0 || device >= 64 || !configured[device])) {
      const cudaError_t error = cudaFuncSetAttribute(moment_direct_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     96 * 1024);
      if (error != cudaSuccess) { set_last_cuda_error(error, "cudaFuncSetAttribute(moment_direct)"); return QSTE_ERR_CUDA; }
      if (device >= 0 && device < 64) configured[device] = true;
    }
    const unsigned grid = (unsigned)ceil_div(blocks, kDirectThreads);
    moment_direct_kernel<<<grid, kDirectThreads, factor_bytes, stream>>>(gradient, moment_q, moment_scale, new_scale, blocks,
                                                                         C, beta1, scalars, block_partial, update_enabled,
                                                                         row_factor, column_factor);
  } else if (lean)
    moment_vec_kernel<true, false><<<block_tiles, 32, 0, stream>>>(gradient, moment_q, moment_scale, new_scale, count,
                                                                   block_size, blocks, beta1, scalars, block_partial,
                                                                   update_enabled, C, row_factor, column_factor);
  else if (recompute)
    moment_vec_kernel<true, true><<<block_tiles, 32, 0, stream>>>(gradient, moment_q, moment_scale, new_scale, count,
                                                                  block_size, blocks, beta1, scalars, block_partial,
                                                                  update_enabled, C, row_factor, column_factor);
  else if (vec_blocks)
    moment_vec_kernel<false, true><<<block_tiles, 32, 0, stream>>>(gradient, moment_q, moment_scale, new_scale, count,
                                                                   block_size, blocks, beta1, scalars, block_partial,
                                                                   update_enabled, C, row_factor, column_factor);
  else
    moment_kernel<<<block_tiles, 32, 0, stream>>>(gradient, moment_q, moment_scale, count, block_size,
                                                  blocks, beta1, scalars, block_partial, update_enabled);
  finish_moment_norm_kernel<<<1, 1024, 0, stream>>>(block_partial, (int64_t)block_tiles, blocks, block_size,
                                                    coordinate_lr, scalars, update_enabled);
  const int64_t bytes = R * ((C + 7) / 8);
  int64_t grid = ceil_div(bytes, 256);
  const int64_t cap = (int64_t)sm_count() * 16;
  if (grid > cap) grid = cap;
  int launched = 8;
  if (lean) {
    coordinate_and_pack_lean_kernel<<<(unsigned)grid, 256, 0, stream>>>(
        gradient, coordinate, packed, moment_q, moment_scale, new_scale, row_factor, column_factor, bytes, C / 8,
        block_shift, beta1, host_scramble((uint32_t)seed), step, step_device, scalars, update_enabled);
    int64_t commit_grid = ceil_div(blocks, 256);
    if (commit_grid > cap) commit_grid = cap;
    commit_scales_kernel<<<(unsigned)commit_grid, 256, 0, stream>>>(new_scale, moment_scale, blocks, update_enabled);
    launched = 9;
  } else if ((C & 7) == 0 && block_shift >= 3)
    coordinate_and_pack_fast_kernel<<<(unsigned)grid, 256, 0, stream>>>(
        gradient, coordinate, packed, moment_q, moment_scale, bytes, block_shift,
        host_scramble((uint32_t)seed), step, step_device, scalars, update_enabled);
  else
    coordinate_and_pack_kernel<<<(unsigned)grid, 256, 0, stream>>>(
        gradient, coordinate, packed, moment_q, moment_scale, R, C, block_shift, block_size,
        host_scramble((uint32_t)seed), step, step_device, scalars, update_enabled);
  if (flips_out) publish_flips_kernel<<<1, 1, 0, stream>>>(scalars, flips_out, update_enabled);
  note_launches((flips_out ? launched + 1 : launched) - launched_less);
  return launch_status("coordinate_update");
}

int check_update_arguments(const float* gradient, const int8_t* coordinate, const uint8_t* packed,
                           const int8_t* moment_q, const uint16_t* moment_scale,
                           const uint16_t* row_v, const uint16_t* col_v, int64_t R, int64_t C,
                           int64_t block_size) {
  if (R <= 0 || C <= 0 || block_size <= 0) return QSTE_ERR_SHAPE;
  if (!gradient || !coordinate || !packed || !moment_q || !moment_scale || !row_v || !col_v)
    return QSTE_ERR_NULL;
  if (!aligned(gradient, 4)) return QSTE_ERR_ALIGNMENT;
  return QSTE_OK;
}

// ---------------------------------------------------------------------------
// Scratch that lives in the library image, for callers that cannot allocate
// ---------------------------------------------------------------------------
//
// The same step as above, with its scratch arrays carved out of one file-scope device
// array instead of a caller-provided workspace.  Every GPU that loads the library holds
// these bytes until the process exits, so the array is sized for a stated maximum
// rather than for the largest conceivable surface.
constexpr int64_t kStaticMaxRows = 16384;
constexpr int64_t kStaticMaxColumns = 16384;
constexpr int64_t kStaticMaxBlocks = 262144;  // ceil(rows * columns / block_size)
constexpr size_t kStaticScratchBytes =
    256 /*scalars*/ + 2 * 4 * kStaticMaxColumns + 2 * 4 * kStaticMaxRows + 8 * kStaticMaxRows +
    8 * kStaticMaxBlocks + 2 * kStaticMaxBlocks + 8 * 256 /*alignment of each array*/;

static __device__ __align__(256) unsigned char g_update_scratch[kStaticScratchBytes];

// In host code `g_update_scratch` is only a handle for the symbol, not a device address;
// the address has to be asked for, once per device, with that device current.
static int static_scratch_address(char** address) {
  static char* cached[64] = {};
  int device = 0;
  cudaError_t error = cudaGetDevice(&device);
  if (error != cudaSuccess) {
    set_last_cuda_error(error, "cudaGetDevice");
    return QSTE_ERR_CUDA;
  }
  if (device < 0 || device >= 64) return QSTE_ERR_LIMIT;
  if (!cached[device]) {
    void* pointer = nullptr;
    error = cudaGetSymbolAddress(&pointer, g_update_scratch);
    if (error != cudaSuccess || !pointer) {
      set_last_cuda_error(error, "cudaGetSymbolAddress(g_update_scratch)");
      return QSTE_ERR_CUDA;
    }
    cached[device] = static_cast<char*>(pointer);
  }
  *address = cached[device];
  return QSTE_OK;
}

}  // namespace qste

using namespace qste;

extern "C" {

int qste_b200_coordinate_update_static(float* gradient, int8_t* coordinate, uint8_t* packed,
                                       int8_t* moment_q, uint16_t* moment_scale, uint16_t* row_v,
                                       uint16_t* col_v, int64_t rows, int64_t columns, double beta1,
                                       double beta2, double update_clip, double coordinate_lr,
                                       int64_t block_size, int64_t seed, int64_t step,
                                       const int64_t* step_device, const uint8_t* update_enabled,
                                       int64_t* flips_out, qste_stream_t stream) {
  const int status = check_update_arguments(gradient, coordinate, packed, moment_q, moment_scale,
                                            row_v, col_v, rows, columns, block_size);
  if (status != QSTE_OK) return status;
  const int64_t blocks = ceil_div(rows * columns, block_size);
  if (rows > kStaticMaxRows || columns > kStaticMaxColumns || blocks > kStaticMaxBlocks ||
      layout_for(rows, columns, blocks).total > kStaticScratchBytes)
    return QSTE_ERR_LIMIT;
  char* scratch = nullptr;
  const int located = static_scratch_address(&scratch);
  if (located != QSTE_OK) return located;
  // Nothing in the scratch needs clearing here: every array is written in full before it is
  // read within one call, and the flip counter is reset by the call's own third kernel
  // (finish_factors_kernel).
  return run_coordinate_update(gradient, coordinate, packed, moment_q, moment_scale, row_v, col_v,
                               rows, columns, beta1, beta2, update_clip, coordinate_lr, block_size,
                               seed, step, step_device, update_enabled, flips_out, scratch,
                               as_stream(stream));
}

size_t qste_b200_coordinate_update_workspace(int64_t rows, int64_t columns, int64_t block_size) {
  if (rows <= 0 || columns <= 0 || block_size <= 0) return 0;
  return layout_for(rows, columns, ceil_div(rows * columns, block_size)).total;
}

int qste_b200_coordinate_update(float* gradient, int8_t* coordinate, uint8_t* packed,
                                int8_t* moment_q, uint16_t* moment_scale, uint16_t* row_v,
                                uint16_t* col_v, int64_t rows, int64_t columns, double beta1,
                                double beta2, double update_clip, double coordinate_lr,
                                int64_t block_size, int64_t seed, int64_t step,
                                const int64_t* step_device, const uint8_t* update_enabled,
                                int64_t* flips_out, void* workspace, size_t workspace_bytes,
                                qste_stream_t stream) {
  const int status = check_update_arguments(gradient, coordinate, packed, moment_q, moment_scale,
                                            row_v, col_v, rows, columns, block_size);
  if (status != QSTE_OK) return status;
  if (!workspace || workspace_bytes < qste_b200_coordinate_update_workspace(rows, columns, block_size))
    return QSTE_ERR_WORKSPACE;
  if (!aligned(workspace, 256)) return QSTE_ERR_ALIGNMENT;
  return run_coordinate_update(gradient, coordinate, packed, moment_q, moment_scale, row_v, col_v,
                               rows, columns, beta1, beta2, update_clip, coordinate_lr, block_size,
                               seed, step, step_device, update_enabled, flips_out,
                               static_cast<char*>(workspace), as_stream(stream));
}

}  // extern "C"
