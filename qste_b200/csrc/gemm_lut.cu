// Forward of the binary Linear for one or two tokens (up to four of fp32), on the CUDA cores,
// bound by streaming the sign bits (sm_100a).
//
//   Y[m, n] = (sum_k X[m, k] * sign(W)[n, k]) * scale[n] + bias[n]
//
// With one to eight activation rows there is no GEMM to speak of: N*K/8 bytes of bits have to
// cross the memory system once, and every group of four bits selects one of the 16 signed sums
// of four activations.  So each block first tabulates, for its slice of the contraction,
//
//     table[m][g][p] = sum_{b<4} (bit b of p ? +x[m, 4g+b] : -x[m, 4g+b])      p in 0..15
//
// and a thread then owns ONE weight row: it loads the row's bytes of the slice with 16-byte
// loads (all of them in flight at once), walks them a nibble at a time and adds table entries.
// All lanes of a warp look up the same group g with their own pattern p: equal patterns read
// the same word (a broadcast), different ones fall in different banks, because the 16 sums of a
// group are 16 consecutive words -- so the look-ups are conflict-free without any re-ordering of
// the table, and there is no cross-lane reduction at all.
//
// The contraction is cut into S slices (S = 8 when it has that many units of 128 columns) handled by the S
// CTAs of a thread-block CLUSTER; every CTA leaves its partial sums in its own shared memory and,
// after a cluster barrier, each CTA adds the S partials of a share of the rows in rank order
// through distributed shared memory, applies scale and bias and stores.  Deterministic: no
// atomics, no second kernel, no workspace.  Cutting the contraction is what makes the tables small
// (a slice of 1024 columns is 16 KB per token, built by one block in a fraction of a
// microsecond) and what gives every SM work when the matrix has few rows.
//
// Algorithmic bytes: N*K/8 (bits) + 4N (scale) + 4N (bias) + M*K*e + M*N*e.
#include <cuda.h>
#include <stdlib.h>

#include "cluster.cuh"
#include "common.cuh"
#include "gemm.h"

namespace qste {
namespace {

constexpr int kLutMaxThreads = 1024;
constexpr int kLutChunk = 4;   // 16-byte vectors of a weight row per chunk; two chunks are in flight per thread

struct LutParams {
  const void* x;           // [M, K]
  const uint8_t* bits;     // [N, K / 8]
  const float* scale;      // [N]
  const float* bias;       // [N] or null
  void* out;               // [M, N]
  long long M, N, K;
  long long pitch;         // K / 8
  int slices;              // cluster size
  int units;               // K / 128: the contraction in units of 128 columns
  int group_rows;          // weight rows per cluster
  int max_slice_groups;    // nibble groups (4 columns) of the widest slice: the table's extent
};

template <typename T, int kM>
__global__ void __launch_bounds__(kLutMaxThreads)
packed_lut_forward_kernel(const __grid_constant__ LutParams p) {
  extern __shared__ float lut_shared[];
  // [max_slice_groups][16][kM] table (the kM sums of a pattern are adjacent: one vector load per
  // look-up), then [kM][group_rows] partial sums
  float* table = lut_shared;
  float* partial = lut_shared + (size_t)kM * p.max_slice_groups * 16;
  const int rank = (int)cluster_rank();
  const long long cluster = blockIdx.x / p.slices;
  const long long row0 = cluster * p.group_rows;
  int unit_begin, unit_end;
  slice_units(p.units, p.slices, rank, unit_begin, unit_end);
  const int slice_groups = (unit_end - unit_begin) * 32;      // nibble groups in this slice
  const long long column0 = (long long)unit_begin * 128;
  const int rows_here = (int)((p.N - row0) < p.group_rows ? (p.N - row0) : p.group_rows);
  const T* x = static_cast<const T*>(p.x);

  // -- the first chunk of this thread's first row is requested before the table is built, so that
  //    the round trip to DRAM and the table build overlap
  const int slice_vectors = unit_end - unit_begin;            // 16-byte vectors (128 columns) per row in the slice
  const int chunks = (slice_vectors + kLutChunk - 1) / kLutChunk;
  uint4 loaded[kLutChunk], ahead[kLutChunk];
  auto request = [&](uint4* buffer, int row, int chunk) {
    const uint4* source = reinterpret_cast<const uint4*>(p.bits + (row0 + row) * p.pitch + column0 / 8) + chunk * kLutChunk;
#pragma unroll
    for (int i = 0; i < kLutChunk; ++i)
      buffer[i] = (row < rows_here && chunk < chunks && chunk * kLutChunk + i < slice_vectors) ? __ldg(source + i)
                                                                                            : make_uint4(0u, 0u, 0u, 0u);
  };
  request(loaded, (int)threadIdx.x, 0);
  request(ahead, (int)threadIdx.x, 1);
  // ... and so are the scale and bias of the row this thread will finish at the end
  const int share = (p.group_rows + p.slices - 1) / p.slices;   // consecutive rows per CTA in the final sum
  const int final_row = rank * share + (int)(threadIdx.x % (unsigned)share);
  const long long final_n = row0 + final_row;
  const bool final_valid = (int)threadIdx.x < kM * share && final_row < p.group_rows && final_n < p.N;
  const float early_scale = final_valid ? __ldg(p.scale + final_n) : 0.0f;
  const float early_bias = (final_valid && p.bias) ? __ldg(p.bias + final_n) : 0.0f;

  // -- table of the slice.  Groups past the slice (the table's
  //    extent is a whole number of chunks) and tokens past M get all-zero entries: a row's last
  //    chunk is padded with zero bits, which then look up 0.
  //    A thread tabulates one (group, token): it loads the four activations once and writes the 16
  //    sums starting at pattern `g` and wrapping round, which spreads a warp's stores over all banks
  //    (written in pattern order they fell on two).
  for (int e = threadIdx.x; e < kM * p.max_slice_groups; e += blockDim.x) {
    const int g = e / kM, m = e - g * kM;
    float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (m < p.M && g < slice_groups) {
      const T* source = x + (long long)m * p.K + column0 + 4 * g;
#pragma unroll
      for (int b = 0; b < 4; ++b) v[b] = DType<T>::load(source + b);
    }
    float* destination = table + (size_t)g * 16 * kM + m;
#pragma unroll
    for (int step = 0; step < 16; ++step) {
      const int q = (step + g) & 15;
      destination[q * kM] = ((q & 1) ? v[0] : -v[0]) + ((q & 2) ? v[1] : -v[1]) + ((q & 4) ? v[2] : -v[2]) + ((q & 8) ? v[3] : -v[3]);
    }
  }
  __syncthreads();

  // -- one weight row per thread (more than one pass only when a cluster has more rows than threads)
  const char* table_bytes = reinterpret_cast<const char*>(table);
  for (int row = threadIdx.x; row < p.group_rows; row += blockDim.x) {
    float acc[kM];
#pragma unroll
    for (int m = 0; m < kM; ++m) acc[m] = 0.0f;
    if (row != (int)threadIdx.x) {   // a later pass over the rows: nothing was requested ahead for it
      request(loaded, row, 0);
      request(ahead, row, 1);
    }
    for (int chunk = 0; chunk < chunks; ++chunk) {
      // `loaded` holds this chunk, `ahead` the next one (requested a whole chunk of look-ups ago)
      constexpr uint32_t kGroupBytes = 64u * kM;             // 16 patterns x kM floats
      const char* base = table_bytes + (size_t)(chunk * kLutChunk) * 32u * kGroupBytes;
      uint4 current[kLutChunk];
#pragma unroll
      for (int i = 0; i < kLutChunk; ++i) { current[i] = loaded[i]; loaded[i] = ahead[i]; }
      request(ahead, row, chunk + 2);
#pragma unroll
      for (int i = 0; i < kLutChunk; ++i) {
        const uint32_t words[4] = {current[i].x, current[i].y, current[i].z, current[i].w};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            // byte offset of the pattern inside its group: pattern * 4 * kM
            constexpr int kShift = kM == 1 ? 2 : (kM == 2 ? 3 : 4);
            constexpr uint32_t kMask = 15u << kShift;
            const uint32_t pattern = 4 * t >= kShift ? (words[w] >> (4 * t - kShift)) & kMask : (words[w] << (kShift - 4 * t)) & kMask;
            const char* entry = base + pattern + ((i * 4 + w) * 8 + t) * kGroupBytes;
            if (kM == 1) {
              acc[0] += *reinterpret_cast<const float*>(entry);
            } else if (kM == 2) {
              const float2 pair = *reinterpret_cast<const float2*>(entry);
              acc[0] += pair.x; acc[1] += pair.y;
            } else {
              const float4 quad = *reinterpret_cast<const float4*>(entry);
              acc[0] += quad.x; acc[1] += quad.y; acc[2] += quad.z; acc[3] += quad.w;
            }
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < kM; ++m) partial[(size_t)m * p.group_rows + row] = acc[m];
  }

  // -- add the slices in rank order; each CTA finishes a share of the cluster's rows
  cluster_sync();
  for (int e = threadIdx.x; e < kM * share; e += blockDim.x) {
    const int m = e / share, row = rank * share + (e - m * share);
    const long long n = row0 + row;
    if (row >= p.group_rows || n >= p.N || m >= p.M) continue;
    float total = 0.0f;
    for (int s = 0; s < p.slices; ++s) total += ld_cluster_f32(partial + (size_t)m * p.group_rows + row, (uint32_t)s);
    // the first pass over e is the row whose scale and bias were fetched at the start
    const bool early = e == (int)threadIdx.x;
    float value = total * (early ? early_scale : p.scale[n]);
    if (p.bias) value = value + (early ? early_bias : p.bias[n]);
    DType<T>::store(static_cast<T*>(p.out) + (long long)m * p.N + n, value);
  }
  cluster_sync();   // nobody leaves (and frees its shared memory) while a peer may still read it
}

constexpr size_t kLutSharedFloor = 116 * 1024;   // more than half an SM's shared memory: one CTA per SM

// How many clusters of `cluster_size` CTAs of this kernel the device holds at once, every CTA on
// an SM of its own (asked of the driver once per device and size: a GPC holds whole clusters only,
// so it is fewer than SMs / size).
template <typename T, int kM>
int lut_cluster_capacity(int cluster_size) {
  auto kernel = packed_lut_forward_kernel<T, kM>;
  static int cached[64][9] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (cluster_size < 1 || cluster_size > 8) return 0;
  const bool slot = device >= 0 && device < 64;
  const int index = cluster_size;
  if (slot && cached[device][index] > 0) return cached[device][index];
  const int by_count = sm_count() / cluster_size > 0 ? sm_count() / cluster_size : 1;
  int clusters = 0;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) == cudaSuccess) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)(cluster_size * sm_count()), 1, 1);
    config.blockDim = dim3((unsigned)kLutMaxThreads, 1, 1);
    config.dynamicSmemBytes = kLutSharedFloor;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = (unsigned)cluster_size;
    attribute.val.clusterDim.y = 1;
    attribute.val.clusterDim.z = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess) clusters = 0;
  }
  cudaGetLastError();
  if (clusters > by_count) clusters = by_count;
  if (slot && clusters > 0) cached[device][index] = clusters;
  return clusters;    // 0: the driver cannot place such a cluster, the kernel does not apply
}

int lut_cluster_capacity(int dtype, int tokens, int cluster_size) {
  int capacity = 0;
  QSTE_DISPATCH_DTYPE(dtype, T, {
    switch (tokens) {
      case 1: capacity = lut_cluster_capacity<T, 1>(cluster_size); break;
      case 2: capacity = lut_cluster_capacity<T, 2>(cluster_size); break;
      default: capacity = lut_cluster_capacity<T, 4>(cluster_size); break;
    }
  });
  return capacity;
}

template <typename T, int kM>
int launch_lut(const LutParams& params, int clusters, int threads, size_t shared, cudaStream_t stream) {
  auto kernel = packed_lut_forward_kernel<T, kM>;
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 64 || !configured[device]) {
    const cudaError_t error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (error != cudaSuccess) { set_last_cuda_error(error, "cudaFuncSetAttribute(packed_lut_forward)"); return QSTE_ERR_CUDA; }
    if (device >= 0 && device < 64) configured[device] = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)(clusters * params.slices), 1, 1);
  config.blockDim = dim3((unsigned)threads, 1, 1);
  config.dynamicSmemBytes = shared;
  config.stream = stream;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = (unsigned)params.slices;
  attribute.val.clusterDim.y = 1;
  attribute.val.clusterDim.z = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  const cudaError_t error = cudaLaunchKernelEx(&config, kernel, params);
  note_launches(1);
  if (error != cudaSuccess) { set_last_cuda_error(error, "cudaLaunchKernelEx(packed_lut_forward)"); return QSTE_ERR_CUDA; }
  return launch_status("packed_lut_forward");
}

// the cut of one problem: cluster size, rows per cluster, threads, shared memory
struct LutPlan {
  int slices, clusters, group_rows, threads, max_slice_groups, tokens;
  size_t shared;
  bool ok;
};

LutPlan lut_plan(int64_t samples, int64_t rows, int64_t columns, int dtype) {
  LutPlan plan = {};
  plan.ok = false;
  // fp32 activations have no register-expansion kernel to hand over to: the tables serve them up to four tokens
  if (samples < 1 || samples > (dtype == QSTE_F32 ? 4 : lut_max_tokens()) || rows < 1 || columns < 128 || columns % 128 != 0) return plan;
  plan.tokens = samples <= 1 ? 1 : (samples <= 2 ? 2 : 4);
  const int units = (int)(columns / 128);
  // Four slices up to 4096 columns, eight beyond (measured at one token, 4096 -> 14336: 12.8 us with
  // four, 16.0 with eight; 14336 -> 4096: 15.3 against 14.1): a row's slice is then 64-128 bytes of
  // bits, and a matrix with few rows still gives every SM a few hundred threads.
  // QSTE_B200_LUT_SLICES pins the cluster size (for A/B timing).
  static const int pinned = getenv("QSTE_B200_LUT_SLICES") ? atoi(getenv("QSTE_B200_LUT_SLICES")) : 0;
  for (int slices = pinned > 0 ? pinned : (units <= 32 ? 4 : 8); slices <= 8; slices *= 2) {
    int s = slices < units ? slices : units;
    const int widest = (units + s - 1) / s;                 // units of the widest slice
    // the table is indexed a whole chunk (8 vectors = 8 units) at a time: round its extent up
    const int table_units = (widest + kLutChunk - 1) / kLutChunk * kLutChunk;
    const size_t table_bytes = (size_t)plan.tokens * table_units * 32 * 16 * sizeof(float);
    int clusters = lut_cluster_capacity(dtype, plan.tokens, s);   // resident at once, a CTA per SM
    if (clusters < 1) continue;
    int group_rows = (int)ceil_div(rows, clusters);
    clusters = (int)ceil_div(rows, group_rows);
    const size_t partial_bytes = (size_t)plan.tokens * group_rows * sizeof(float);
    if (table_bytes + partial_bytes > 190 * 1024) {
      if (slices == 8) {
        // still too large: more, smaller row groups (several waves of clusters)
        const size_t room = 190 * 1024 > table_bytes ? 190 * 1024 - table_bytes : 0;
        const int fit_rows = (int)(room / (plan.tokens * sizeof(float)));
        if (fit_rows < 32) return plan;
        group_rows = fit_rows;
        clusters = (int)ceil_div(rows, group_rows);
      } else {
        continue;
      }
    }
    plan.slices = s;
    plan.clusters = clusters;
    plan.group_rows = group_rows;
    plan.max_slice_groups = table_units * 32;
    int threads = (group_rows + 31) / 32 * 32;
    if (threads > kLutMaxThreads) threads = kLutMaxThreads;
    if (threads < 128) threads = 128;
    plan.threads = threads;
    plan.shared = (size_t)plan.tokens * plan.max_slice_groups * 16 * sizeof(float) + (size_t)plan.tokens * group_rows * sizeof(float);
    // two CTAs on one SM would each run at half speed while other SMs idle
    if (plan.shared < kLutSharedFloor) plan.shared = kLutSharedFloor;
    plan.ok = true;
    return plan;
  }
  return plan;
}

}  // namespace

int lut_max_tokens() {
  static const int tokens = [] {
    const char* text = getenv("QSTE_B200_LUT_TOKENS");
    const int value = text ? atoi(text) : 2;
    return value < 0 ? 0 : (value > 4 ? 4 : value);
  }();
  return tokens;
}

bool lut_supported(int64_t samples, int64_t rows, int64_t columns, int dtype, const void* x, const void* bits,
                   const void* out, int out_dtype) {
  if (dtype_size(dtype) == 0 || out_dtype != dtype) return false;
  if (!aligned(bits, 16) || !aligned(x, 2) || !aligned(out, 2)) return false;
  if (check_arch() != QSTE_OK) return false;
  return lut_plan(samples, rows, columns, dtype).ok;
}

int lut_forward(const void* x, int dtype, int64_t samples, const uint8_t* packed, const float* scale, const float* bias,
                int64_t rows, int64_t columns, void* out, cudaStream_t stream) {
  const LutPlan plan = lut_plan(samples, rows, columns, dtype);
  if (!plan.ok) return QSTE_ERR_UNSUPPORTED;
  LutParams params = {};
  params.x = x; params.bits = packed; params.scale = scale; params.bias = bias; params.out = out;
  params.M = samples; params.N = rows; params.K = columns;
  params.pitch = columns / 8;
  params.slices = plan.slices;
  params.units = (int)(columns / 128);
  params.group_rows = plan.group_rows;
  params.max_slice_groups = plan.max_slice_groups;
  int status = QSTE_ERR_DTYPE;
  QSTE_DISPATCH_DTYPE(dtype, T, {
    switch (plan.tokens) {
      case 1: status = launch_lut<T, 1>(params, plan.clusters, plan.threads, plan.shared, stream); break;
      case 2: status = launch_lut<T, 2>(params, plan.clusters, plan.threads, plan.shared, stream); break;
      default: status = launch_lut<T, 4>(params, plan.clusters, plan.threads, plan.shared, stream); break;
    }
  });
  return status;
}

}  // namespace qste
