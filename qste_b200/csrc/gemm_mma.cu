// Forward of the binary Linear for 3..32 tokens with the weights held in registers (sm_100a).
//
//   Y[m, n] = (sum_k X[m, k] * sign(W)[n, k]) * scale[n] + bias[n]
//
// At these batch sizes the product is bound by getting N*K/8 bytes of sign bits to the
// arithmetic once; the tokens are few enough that the whole activation slice of a CTA sits in
// shared memory.  tcgen05 does not pay here: an MMA of 128 weight rows by 16 columns occupies the
// tensor pipe for about 160 cycles however few tokens ride along, which puts a floor of 16 us
// under a 4096 x 14336 layer, and its weight operand has to be written out as 16-bit values in
// shared (or tensor) memory first.  The warp-level `mma.sync.m16n8k16` has no such floor and takes
// the weight operand from REGISTERS: a lane turns bits of its two weight rows into an A register
// of the instruction with one shift and one logic operation, straight from the words it loaded
// from global memory, so the expanded weights never exist anywhere.
//
//   * A warp owns a slab of 16 weight rows.  Lane 4g + q holds rows g and g + 8 of it and loads, of
//     every run of 512 columns, the 16 bytes of unit q (128 columns): the four lanes of a row share
//     the run out between them and nothing is loaded twice.  (Two slabs per warp, sharing the
//     activation fragments, were 5-30 % slower: half as many warps to hide latency with.)
//   * The order of the contraction index inside an MMA is free as long as both operands agree, so
//     it is chosen to suit the bits: in step (c, p) of a run -- word c of the unit, p = 0..7 -- lane q
//     supplies columns p, p + 16 (first k-pair of its quad slot) and p + 8, p + 24 (second) of word c
//     of ITS unit.  Bits p and p + 16 of a word move to the sign positions of a pair of 16-bit values
//     with one shift by a constant: (w << (15 - p)) & 0x80008000, XORed onto a pair of -1.  No lane
//     needs a word another lane holds, so there are no shuffles.
//   * The activations are the B operand: tokens are the `n` of the instruction (8 per tile, 1-4
//     tiles).  They are staged in shared memory ONCE per CTA in the matching order -- a 16-byte
//     chunk per (step, k-half) holding, for q = 0..3, the two columns lane q pairs up -- and read
//     with `ldmatrix` (rows padded by 16 bytes: no bank conflicts).
//   * The contraction is cut into S slices over the S CTAs of a thread-block cluster (S = 1, 2, 4
//     or 8): partial sums stay in shared memory, and after a cluster barrier every CTA adds the S
//     partials of its share of the rows in rank order through distributed shared memory, applies
//     scale and bias, and stores.  No atomics, no workspace, one launch.  The cut is chosen so
//     that all clusters are resident at once: how many clusters of a size fit is asked of the
//     driver (a GPC holds a whole number of them), and every CTA claims more than half an SM's
//     shared memory so that no SM is given two.
//
// Accumulation is fp32; the products are exact (+-x), so the result differs from the other
// kernels' only in the order of the fp32 additions.
//
// Algorithmic bytes: N*K/8 (bits) + 8N (scale, bias) + M*K*2 + M*N*2.
#include <cuda.h>
#include <stdlib.h>

#include "cluster.cuh"
#include "common.cuh"
#include "gemm.h"

namespace qste {
namespace {

constexpr int kMmaMaxThreads = 1024;
constexpr int kSlabs = 1;                    // slabs of 16 weight rows per warp
constexpr int kWarpRows = 16 * kSlabs;
constexpr size_t kMmaSharedLimit = 200 * 1024;
constexpr size_t kMmaSharedFloor = 116 * 1024;   // more than half an SM's shared memory: one CTA per SM

struct MmaParams {
  const void* x;           // [M, K], 16-bit
  const uint8_t* bits;     // [N, K / 8]
  const float* scale;      // [N]
  const float* bias;       // [N] or null
  void* out;               // [M, N]
  long long M, N, K;
  long long pitch;         // K / 8
  int slices;              // cluster size
  int units;               // K / 128
  int group_rows;          // weight rows per cluster, a multiple of 16
  int x_pitch;             // bytes between tokens of the activation slice in shared memory
};

template <typename T> struct MmaType;
template <> struct MmaType<__half> {
  static constexpr uint32_t kMinusOnes = 0xBC00BC00u;
  __device__ static void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
template <> struct MmaType<__nv_bfloat16> {
  static constexpr uint32_t kMinusOnes = 0xBF80BF80u;
  __device__ static void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t address) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}

// Bits `pair` and `pair` + 16 of `word` (pair < 16, a constant after unrolling) as a pair of
// 16-bit values, -1 where the bit is clear and +1 where it is set: the shift puts them on the sign
// bits of the two halves.
template <typename T>
__device__ __forceinline__ uint32_t sign_pair(uint32_t word, int pair) {
  return MmaType<T>::kMinusOnes ^ ((word << (15 - pair)) & 0x80008000u);
}

// kTiles: tiles of eight tokens (1, 2 or 4)
template <typename T, int kTiles>
__global__ void __launch_bounds__(kMmaMaxThreads)
packed_mma_forward_kernel(const __grid_constant__ MmaParams p) {
  constexpr int kTokenRows = (kTiles < 2 ? 2 : kTiles) * 8;   // ldmatrix.x4 reads 16 tokens at a time
  extern __shared__ __align__(16) unsigned char mma_shared[];
  // [kTokenRows][x_pitch] activations of the slice, then [kTiles * 8][group_rows] partial sums
  unsigned char* xs = mma_shared;
  float* partial = reinterpret_cast<float*>(mma_shared + (size_t)kTokenRows * p.x_pitch);
  const int rank = (int)cluster_rank();
  const long long cluster = blockIdx.x / p.slices;
  const long long row0 = cluster * p.group_rows;
  int unit_begin, unit_end;
  slice_units(p.units, p.slices, rank, unit_begin, unit_end);
  const int units_here = unit_end - unit_begin;               // units of 128 columns in this slice
  const int runs = (units_here + 3) / 4;                      // runs of 512 columns
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int g = lane >> 2, q = lane & 3;

  // -- this lane's unit of run `run` of its rows of the slabs starting at `first_row`
  auto request = [&](uint4 (&buffer)[kSlabs][2], int first_row, int run) {
    const int unit = run * 4 + q;
#pragma unroll
    for (int s = 0; s < kSlabs; ++s)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int row = first_row + s * 16 + h * 8 + g;
        const long long n = row0 + row;
        const bool valid = row < p.group_rows && n < p.N && unit < units_here;
        buffer[s][h] = valid ? __ldg(reinterpret_cast<const uint4*>(p.bits + n * p.pitch) + unit_begin + unit)
                             : make_uint4(0u, 0u, 0u, 0u);
      }
  };
  // the first two runs of the warp's first rows are requested before the activations are staged
  uint4 current[kSlabs][2], ahead[kSlabs][2];
  request(current, warp * kWarpRows, 0);
  request(ahead, warp * kWarpRows, 1);

  // -- the activation slice, in the order the MMA steps consume it.  A token's run is 1024 bytes:
  //    64 chunks of 16 bytes, chunk 2 * (8c + p) + w holding for q = 0..3 the pair
  //    (column 32c + 8w + p, the same + 16) of unit q.  A thread takes one (token, unit, c, w): two
  //    16-byte loads (columns 8w.. and 16 + 8w.. of word c) become eight 4-byte stores 32 bytes apart.
  //    Lanes run over q and eight tokens, which puts a warp's stores in 32 different banks.  Units
  //    past the slice and tokens past M are zero (their weights then count for nothing).
  {
    const int token_blocks = kTokenRows / 8;
    const int items = token_blocks * runs * 8;                 // (token block, run, c, w), 32 lanes each
    const unsigned char* source = static_cast<const unsigned char*>(p.x) + (size_t)unit_begin * 256;
    for (int item = warp; item < items; item += warps) {
      const int w = item & 1, c = (item >> 1) & 3;
      const int run = (item >> 3) % runs, block = (item >> 3) / runs;
      const int token = block * 8 + g;
      const int unit = run * 4 + q;
      uint4 low = make_uint4(0u, 0u, 0u, 0u), high = make_uint4(0u, 0u, 0u, 0u);
      if (token < p.M && unit < units_here) {
        const unsigned char* from = source + (size_t)token * p.K * 2 + (size_t)unit * 256 + c * 64 + w * 16;
        low = __ldg(reinterpret_cast<const uint4*>(from));
        high = __ldg(reinterpret_cast<const uint4*>(from + 32));
      }
      unsigned char* to = xs + (size_t)token * p.x_pitch + run * 1024 + c * 256 + w * 16 + q * 4;
      const uint32_t lows[4] = {low.x, low.y, low.z, low.w}, highs[4] = {high.x, high.y, high.z, high.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        // two columns per word: (2e, 2e + 1) of the eight
        *reinterpret_cast<uint32_t*>(to + (2 * e) * 32) = __byte_perm(lows[e], highs[e], 0x5410);
        *reinterpret_cast<uint32_t*>(to + (2 * e + 1) * 32) = __byte_perm(lows[e], highs[e], 0x7632);
      }
    }
  }
  __syncthreads();

  // ldmatrix: lanes 0-7 address tokens 0-7 at the step's first chunk, lanes 8-15 the same tokens at
  // its second chunk, lanes 16-31 likewise for tokens 8-15
  const uint32_t fragment_lane = (uint32_t)__cvta_generic_to_shared(xs) +
                                 (uint32_t)((lane >> 4) * 8 + (lane & 7)) * p.x_pitch + ((lane >> 3) & 1) * 16;
  const uint32_t pair_stride = 16u * (uint32_t)p.x_pitch;

  for (int first_row = warp * kWarpRows; first_row < p.group_rows; first_row += warps * kWarpRows) {
    float acc[kSlabs][kTiles][4];
#pragma unroll
    for (int s = 0; s < kSlabs; ++s)
#pragma unroll
      for (int t = 0; t < kTiles; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[s][t][i] = 0.0f;
    if (first_row != warp * kWarpRows) {   // a later pass over the rows: nothing was requested ahead for it
      request(current, first_row, 0);
      request(ahead, first_row, 1);
    }
    uint32_t fragment = fragment_lane;
    for (int run = 0; run < runs; ++run) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t word[kSlabs][2];
#pragma unroll
        for (int s = 0; s < kSlabs; ++s)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint4 mine = current[s][h];
            word[s][h] = c == 0 ? mine.x : (c == 1 ? mine.y : (c == 2 ? mine.z : mine.w));
          }
#pragma unroll
        for (int pair = 0; pair < 8; ++pair) {
          uint32_t b[kTokenRows / 8][2];
#pragma unroll
          for (int half = 0; half < kTokenRows / 16; ++half) {
            uint32_t r[4];
            ldmatrix_x4(r, fragment + (uint32_t)half * pair_stride + (uint32_t)(c * 8 + pair) * 32u);
            b[2 * half][0] = r[0]; b[2 * half][1] = r[1];
            b[2 * half + 1][0] = r[2]; b[2 * half + 1][1] = r[3];
          }
#pragma unroll
          for (int s = 0; s < kSlabs; ++s) {
            // rows g and g + 8; first k-pair of the quad slot (columns pair, pair + 16), then the second (+ 8)
            const uint32_t a[4] = {sign_pair<T>(word[s][0], pair), sign_pair<T>(word[s][1], pair),
                                   sign_pair<T>(word[s][0], pair + 8), sign_pair<T>(word[s][1], pair + 8)};
#pragma unroll
            for (int t = 0; t < kTiles; ++t) MmaType<T>::mma(acc[s][t], a, b[t][0], b[t][1]);
          }
        }
      }
      fragment += 1024u;
#pragma unroll
      for (int s = 0; s < kSlabs; ++s)
#pragma unroll
        for (int h = 0; h < 2; ++h) current[s][h] = ahead[s][h];
      request(ahead, first_row, run + 2);
    }
    // accumulator i of a tile: row g (+8 for i >= 2), token 8t + 2q + (i & 1)
#pragma unroll
    for (int s = 0; s < kSlabs; ++s)
#pragma unroll
      for (int t = 0; t < kTiles; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int row = first_row + s * 16 + (i >> 1) * 8 + g;
          const int token = t * 8 + 2 * q + (i & 1);
          if (row < p.group_rows) partial[(size_t)token * p.group_rows + row] = acc[s][t][i];
        }
  }

  // -- add the slices in rank order; each CTA finishes a share of the cluster's rows
  cluster_sync();
  const int share = (p.group_rows + p.slices - 1) / p.slices;   // consecutive rows per CTA
  for (int e = threadIdx.x; e < (int)p.M * share; e += blockDim.x) {
    const int m = e / share, row = rank * share + (e - m * share);
    const long long n = row0 + row;
    if (row >= p.group_rows || n >= p.N) continue;
    float total = 0.0f;
    for (int s = 0; s < p.slices; ++s) total += ld_cluster_f32(partial + (size_t)m * p.group_rows + row, (uint32_t)s);
    float value = total * p.scale[n];
    if (p.bias) value = value + p.bias[n];
    DType<T>::store(static_cast<T*>(p.out) + (long long)m * p.N + n, value);
  }
  cluster_sync();   // nobody leaves (and frees its shared memory) while a peer may still read it
}

// How many clusters of `cluster_size` CTAs of this kernel the device holds at once, every CTA on
// an SM of its own (asked of the driver once per device and size: a GPC holds whole clusters only).
template <typename T, int kTiles>
int mma_cluster_capacity(int cluster_size) {
  auto kernel = packed_mma_forward_kernel<T, kTiles>;
  static int cached[64][4] = {};
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  const bool slot = device >= 0 && device < 64;
  const int index = cluster_size == 1 ? 0 : (cluster_size == 2 ? 1 : (cluster_size == 4 ? 2 : 3));
  if (slot && cached[device][index] > 0) return cached[device][index];
  if (!slot || !configured[device]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMmaSharedLimit) != cudaSuccess) {
      cudaGetLastError();
      return 0;
    }
    if (slot) configured[device] = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)(cluster_size * sm_count()), 1, 1);
  config.blockDim = dim3((unsigned)kMmaMaxThreads, 1, 1);
  config.dynamicSmemBytes = kMmaSharedFloor;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = (unsigned)cluster_size;
  attribute.val.clusterDim.y = 1;
  attribute.val.clusterDim.z = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess) {
    cudaGetLastError();
    return 0;          // the driver cannot place such a cluster: this kernel does not apply
  }
  const int by_count = sm_count() / cluster_size;
  if (clusters > by_count) clusters = by_count;
  if (slot && clusters > 0) cached[device][index] = clusters;
  return clusters;
}

int mma_cluster_capacity(int dtype, int tiles, int cluster_size) {
#define QSTE_MMA_CAPACITY(T)                                              \
  switch (tiles) {                                                        \
    case 1: return mma_cluster_capacity<T, 1>(cluster_size);              \
    case 2: return mma_cluster_capacity<T, 2>(cluster_size);              \
    default: return mma_cluster_capacity<T, 4>(cluster_size);             \
  }
  if (dtype == QSTE_F16) { QSTE_MMA_CAPACITY(__half) }
  QSTE_MMA_CAPACITY(__nv_bfloat16)
#undef QSTE_MMA_CAPACITY
}

template <typename T, int kTiles>
int launch_mma(const MmaParams& params, int clusters, int threads, size_t shared, cudaStream_t stream) {
  auto kernel = packed_mma_forward_kernel<T, kTiles>;
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 64 || !configured[device]) {
    const cudaError_t error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMmaSharedLimit);
    if (error != cudaSuccess) { set_last_cuda_error(error, "cudaFuncSetAttribute(packed_mma_forward)"); return QSTE_ERR_CUDA; }
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
  if (error != cudaSuccess) { set_last_cuda_error(error, "cudaLaunchKernelEx(packed_mma_forward)"); return QSTE_ERR_CUDA; }
  return launch_status("packed_mma_forward");
}

// the cut of one problem
struct MmaPlan {
  int slices, clusters, group_rows, threads, tiles, x_pitch;
  size_t shared;
  bool ok;
};

// Measured on B200 against the other kernels (CUDA graph over weight copies larger than L2, bf16,
// microseconds, this kernel / tcgen05 tiles; for 1-4 tokens this kernel / look-up tables):
//                      4096->14336   14336->4096   4096->11008   2048->5632   768->3072
//    1 token            12.0 /  9.4   14.9 / 11.7   10.4 /  7.4    5.4 /  4.8   4.9 / 4.1
//    2 tokens           12.1 / 11.6   15.1 / 14.7   10.5 /  9.5    5.4 /  5.7   5.0 / 4.5
//    4 tokens           12.5 / 21.7   15.2 / 27.7   10.9 / 17.6    5.5 /  8.1   5.0 / 5.9
//    5 tokens           12.7 / 31.5   15.4 / 27.0   11.0 / 23.3    5.8 / 14.7   5.0 / 12.1
//   16 tokens           15.1 / 29.6   18.1 / 27.3   12.9 / 23.7    6.4 / 15.3   5.9 / 12.8
//   32 tokens           21.9 / 30.4   31.8 / 27.6   18.9 / 24.7    9.3 / 15.4   8.5 / 13.1
//   64 tokens           57.2 / 31.6       - / 27.9  51.6 / 25.6   20.1 / 16.4  19.2 / 13.3
// (the rows for 64 tokens and 32 tokens at 14336 columns with two slabs per warp).  Hence: 3 to 32
// tokens, 17-32 only for contractions up to 12288 columns.  Four slices were the fastest cut up to
// 11008 columns (two: 8-15 % slower, one: 50-80 %), eight at 14336.
MmaPlan mma_plan(int64_t samples, int64_t rows, int64_t columns, int dtype) {
  MmaPlan plan = {};
  plan.ok = false;
  if (samples <= lut_max_tokens() || samples > 32 || rows < 1 || columns < 128 || columns % 128 != 0) return plan;
  if (samples > 16 && columns > 12288) return plan;
  plan.tiles = samples <= 8 ? 1 : (samples <= 16 ? 2 : 4);
  const int token_rows = (plan.tiles < 2 ? 2 : plan.tiles) * 8;
  const int units = (int)(columns / 128);
  // QSTE_B200_MMA_SLICES pins the cluster size (for A/B timing)
  static const int pinned = getenv("QSTE_B200_MMA_SLICES") ? atoi(getenv("QSTE_B200_MMA_SLICES")) : 0;
  int slices = pinned > 0 ? pinned : (units >= 100 ? 8 : 4);
  if (slices != 1 && slices != 2 && slices != 4 && slices != 8) return plan;
  while (slices > units) slices >>= 1;
  const int widest = (units + slices - 1) / slices;            // units of the widest slice
  const int runs = (widest + 3) / 4;
  const int x_pitch = runs * 1024 + 16;
  const size_t x_bytes = (size_t)token_rows * x_pitch;
  const size_t row_bytes = (size_t)plan.tiles * 8 * sizeof(float);     // partial sums per weight row
  if (x_bytes + 16 * row_bytes > kMmaSharedLimit) return plan;
  const int fit_rows = (int)((kMmaSharedLimit - x_bytes) / row_bytes) / 16 * 16;
  const int capacity = mma_cluster_capacity(dtype, plan.tiles, slices);   // clusters resident at once
  if (capacity <= 0) return plan;
  // one wave of clusters if their row groups fit beside the activations, else two (more: the
  // tensor-core tiles do better)
  for (int waves = 1; waves <= 2; ++waves) {
    const int group_rows = (int)ceil_div(ceil_div(rows, (int64_t)capacity * waves), 16) * 16;
    if (group_rows > fit_rows) continue;
    plan.slices = slices;
    plan.group_rows = group_rows;
    plan.clusters = (int)ceil_div(rows, group_rows);
    plan.x_pitch = x_pitch;
    const size_t need = x_bytes + (size_t)group_rows * row_bytes;
    plan.shared = need < kMmaSharedFloor ? kMmaSharedFloor : need;
    int threads = (group_rows + kWarpRows - 1) / kWarpRows * 32;
    if (threads > kMmaMaxThreads) threads = kMmaMaxThreads;
    if (threads < 64) threads = 64;
    plan.threads = threads;
    plan.ok = true;
    break;
  }
  return plan;
}

}  // namespace

bool mma_supported(int64_t samples, int64_t rows, int64_t columns, int dtype, const void* x, const void* bits,
                   const void* out, int out_dtype) {
  if ((dtype != QSTE_F16 && dtype != QSTE_BF16) || out_dtype != dtype) return false;
  if (!aligned(bits, 16) || !aligned(x, 16) || !aligned(out, 2)) return false;
  if (check_arch() != QSTE_OK) return false;
  return mma_plan(samples, rows, columns, dtype).ok;
}

int mma_forward(const void* x, int dtype, int64_t samples, const uint8_t* packed, const float* scale, const float* bias,
                int64_t rows, int64_t columns, void* out, cudaStream_t stream) {
  const MmaPlan plan = mma_plan(samples, rows, columns, dtype);
  if (!plan.ok) return QSTE_ERR_UNSUPPORTED;
  MmaParams params = {};
  params.x = x; params.bits = packed; params.scale = scale; params.bias = bias; params.out = out;
  params.M = samples; params.N = rows; params.K = columns;
  params.pitch = columns / 8;
  params.slices = plan.slices;
  params.units = (int)(columns / 128);
  params.group_rows = plan.group_rows;
  params.x_pitch = plan.x_pitch;
#define QSTE_MMA_TILES(T)                                                                                    \
  switch (plan.tiles) {                                                                                      \
    case 1: return launch_mma<T, 1>(params, plan.clusters, plan.threads, plan.shared, stream);               \
    case 2: return launch_mma<T, 2>(params, plan.clusters, plan.threads, plan.shared, stream);               \
    default: return launch_mma<T, 4>(params, plan.clusters, plan.threads, plan.shared, stream);              \
  }
  if (dtype == QSTE_F16) { QSTE_MMA_TILES(__half) }
  if (dtype == QSTE_BF16) { QSTE_MMA_TILES(__nv_bfloat16) }
#undef QSTE_MMA_TILES
  return QSTE_ERR_DTYPE;
}

}  // namespace qste
