// Small-batch forward of the binary Linear on the tensor cores, weight-stationary (sm_100a).
//
//   Y[m, n] = (sum_k X[m, k] * sign(W)[n, k]) * scale[n] + bias[n]        1 <= M <= 128 tokens
//
// With few tokens the product is bound by streaming the N*K/8 bytes of sign bits, and the
// large-batch kernel (gemm_tc.cu) is the wrong shape for it: it puts the tokens on the M side
// of the MMA, padded to 128 rows, and pays for 256 expanded weight rows per 64 k-values in
// shared-memory traffic and tensor time whatever M is.  Here the operands are swapped:
//
//   D^T[n, m] = sum_k W(n, k) * X(m, k)      M side = 128 weight rows (a "slab"), N side = tokens
//
// so an MMA costs 128 x Np x 16 with Np = M rounded up to 16, and a CTA owns a slab of weight
// rows for the whole contraction: it reads each of its sign bits exactly once.  The expanded
// +-1 operand never touches shared memory: the expander threads (one weight row each) turn 8
// bytes of bits into 64 bf16/fp16 values in registers and write them straight into TENSOR
// MEMORY (tcgen05.st), from where tcgen05.mma takes its A operand.  Shared memory only carries
// the X tile (Np rows of 64 k-values, by TMA; the same few hundred KB for every CTA, so it
// comes out of L2).  Slabs are sized so that every SM gets one (97 rows at N = 14336), which is
// why no split of the contraction and no second kernel is needed.
//
//   warps 0-15  expanders, four groups of four warps; group g takes k-blocks n = g (mod 4);
//               warp w writes TMEM lanes 32 * (w % 4) .. + 31, one weight row per thread
//   warps 16-19 epilogue: tcgen05.ld, fp32 scale and bias per weight row, transposed store
//   warp 20     TMA producer of the X tiles (one lane; no multicast)
//   warp 21     MMA issuer (one lane): four K = 16 MMAs per k-block, tcgen05.commit
//   warp 22     TMA producer of the sign bits (one lane): chunks of slab rows x 64 bytes (eight
//               k-blocks) into a shared-memory ring, four chunks deep.  The expanders read their
//               8 bytes per k-block from there: with the bits loaded straight from global memory
//               into registers, every expander iteration ended on a ~1.4 us round trip to DRAM
//               (a row per lane, one sector each) and the kernel ran at 0.36 us per k-block
//               whatever the batch -- 27 us at K = 4096 against 7 us of work.
//
// A build switch keeps the expanded operand in shared memory instead (kATmem = false: the
// layout and descriptors of the large-batch kernel), as a cross-check of the tensor-memory path.
//
// Every mbarrier wait is bounded (tcgen05.cuh); on give-up the CTA raises its abort flag, every
// role leaves its loop and tensor memory is freed.
#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"
#include "gemm.h"
#include "tcgen05.cuh"

namespace qste {
namespace {

constexpr int kSlabRows = 128;   // M of the MMA: weight rows per slab (the last ones may be unused)
constexpr int kBK = 64;          // k-values per stage
constexpr int kGroups = 4, kGroupWarps = 4;
constexpr int kExpanderWarps = kGroups * kGroupWarps;
constexpr int kEpilogueWarps = 4;
constexpr int kTmaWarp = kExpanderWarps + kEpilogueWarps, kMmaWarp = kTmaWarp + 1, kBitsWarp = kMmaWarp + 1;
constexpr int kThreads = (kBitsWarp + 1) * 32;
constexpr int kChunkBlocks = 8;                      // k-blocks per chunk of sign bits
constexpr int kChunkRowBytes = kChunkBlocks * 8;     // 64 bytes of a weight row
constexpr int kBitStages = 4;
constexpr uint32_t kBitStageBytes = kSlabRows * kChunkRowBytes;
constexpr int kMaxTokens = 128;
constexpr uint32_t kTmemColumns = 512;
constexpr uint32_t kAccumColumns = 128;     // columns per accumulator (two of them)
constexpr uint32_t kAColumn0 = 256;         // first column of the A stages in tensor memory
constexpr uint32_t kAStageColumns = 32;     // 64 16-bit values per lane

template <bool kATmem> struct WsShape {
  static constexpr int kStages = kATmem ? 8 : 4;
  static constexpr uint32_t kABytes = kATmem ? 0u : (uint32_t)(kSlabRows * kBK * 2);
  static constexpr uint32_t kXBytes = kMaxTokens * kBK * 2;   // room for the largest X tile
  static constexpr uint32_t kStageBytes = kABytes + kXBytes;
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + kBitStages * kBitStageBytes + 1024 /*alignment slack*/ +
                                         256 /*barriers*/;
};

struct WsParams {
  const uint8_t* bits;     // [N, K / 8]
  long long bit_pitch;
  const float* scale;      // [N]
  const float* bias;       // [N] or null
  void* out;               // [M, N] in the activation dtype
  long long M, N, K;
  int tokens_padded;       // Np: M rounded up to 16
  int slab_rows;           // weight rows per slab actually used (<= 128)
  int slabs;
  int kblocks;
  int is_half;             // X (and the expanded weights) are fp16, else bf16
  unsigned long long* diagnostics;
  int profile;             // CTA 0 leaves per-role cycle counts in diagnostics[8..23]
};

__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}

// 32 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_store32(uint32_t address, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(address), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_load16(uint32_t address, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(address) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int e = 0; e < 16; ++e) v[e] = __uint_as_float(r[e]);
}

template <typename TO, bool kATmem>
__global__ void __launch_bounds__(kThreads, 1)
packed_gemm_ws_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_bits,
                      const __grid_constant__ WsParams p) {
  using Shape = WsShape<kATmem>;
  constexpr int kStages = Shape::kStages;
  constexpr uint32_t kStageBytes = Shape::kStageBytes;
#define WAIT(bar, parity) mbar_wait<false>(bar, parity, abort_flag, p.diagnostics, __LINE__)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  // stage s: [expanded A tile (shared-memory variant only)] [X tile]; then the ring of bit chunks
  const uint32_t bits_base = smem_base + kStages * kStageBytes;
  const uint32_t bar_base = bits_base + kBitStages * kBitStageBytes;
  // full(s): the TMA thread (with the X bytes) plus one arrival per warp of the group that wrote
  // the A tile; empty(s): one arrival, from tcgen05.commit
  auto full = [&](int s) { return bar_base + 8u * s; };
  auto empty = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto accum_full = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto accum_empty = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  // bits_full(b): the bits producer (with the chunk's bytes); bits_empty(b): every expander warp
  auto bits_full = [&](int b) { return bar_base + 8u * (2 * kStages + 4 + b); };
  auto bits_empty = [&](int b) { return bar_base + 8u * (2 * kStages + 4 + kBitStages + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_aligned + (bar_base - smem_base) + 8 * (2 * kStages + 4 + 2 * kBitStages));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int np = p.tokens_padded;
  const uint32_t x_bytes = (uint32_t)np * kBK * 2;
  const int chunks = (p.kblocks + kChunkBlocks - 1) / kChunkBlocks;   // per slab

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full(s), 1 + kGroupWarps);
      mbar_init(empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(accum_full(a), 1);
      mbar_init(accum_empty(a), kEpilogueWarps);
    }
    for (int b = 0; b < kBitStages; ++b) {
      mbar_init(bits_full(b), 1);
      mbar_init(bits_empty(b), kExpanderWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == kTmaWarp) tmem_alloc(smem_u32(tmem_slot), kTmemColumns);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == kTmaWarp) {
    // ---- X tiles: Np rows x 64 k-values per k-block, the same for every slab ----------------
    if (lane == 0) {
      int g = 0;
      bool alive = true;
      for (int slab = blockIdx.x; slab < p.slabs && alive; slab += gridDim.x) {
        for (int kb = 0; kb < p.kblocks; ++kb, ++g) {
          const int s = g % kStages;
          if (!WAIT(empty(s), ((g / kStages) & 1) ^ 1)) { alive = false; break; }
          mbar_expect_tx(full(s), x_bytes);
          tma_load_2d(smem_base + s * kStageBytes + Shape::kABytes, &map_x, full(s), kb * kBK, 0);
        }
      }
    }
    __syncwarp();
  } else if (warp == kBitsWarp) {
    // ---- sign bits: slab rows x 64 bytes per chunk (the box is slab_rows tall; bytes past K/8
    // and rows past N read zero) ---------------------------------------------------------------
    if (lane == 0) {
      int h = 0;
      bool alive = true;
      const uint32_t chunk_bytes = (uint32_t)p.slab_rows * kChunkRowBytes;
      for (int slab = blockIdx.x; slab < p.slabs && alive; slab += gridDim.x) {
        for (int c = 0; c < chunks; ++c, ++h) {
          const int b = h % kBitStages;
          if (!WAIT(bits_empty(b), ((h / kBitStages) & 1) ^ 1)) { alive = false; break; }
          mbar_expect_tx(bits_full(b), chunk_bytes);
          tma_load_2d(bits_base + b * kBitStageBytes, &map_bits, bits_full(b), c * kChunkRowBytes, slab * p.slab_rows);
        }
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // ---- MMA issuer -------------------------------------------------------------------------
    if (lane == 0) {
      // D fp32; A and B in one 16-bit format, both K-major; N = Np, M = 128
      const uint32_t format = p.is_half ? 0u : 1u;
      const uint32_t idesc = (1u << 4) | (format << 7) | (format << 10) |
                             ((uint32_t)(np >> 3) << 17) | ((uint32_t)(kSlabRows >> 4) << 24);
      int g = 0, lt = 0;
      bool alive = true;
      const bool prof = p.profile && blockIdx.x == 0 && p.diagnostics;
      long long t_begin = prof ? clock64() : 0, t_wait = 0, t_issue = 0, t_mark = 0;
      for (int slab = blockIdx.x; slab < p.slabs && alive; slab += gridDim.x, ++lt) {
        const int acc = lt & 1;
        if (!WAIT(accum_empty(acc), ((lt >> 1) & 1) ^ 1)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)acc * kAccumColumns;
        for (int kb = 0; kb < p.kblocks; ++kb, ++g) {
          const int s = g % kStages;
          if (prof) t_mark = clock64();
          if (!WAIT(full(s), (g / kStages) & 1)) { alive = false; break; }
          if (prof) { const long long now = clock64(); t_wait += now - t_mark; t_mark = now; }
          tc_fence_after();
          const uint32_t stage = smem_base + s * kStageBytes;
          const uint32_t x_smem = stage + Shape::kABytes;
#pragma unroll
          for (int ks = 0; ks < kBK / 16; ++ks) {
            // K-major, 128-byte swizzle: rows of 64 values = 128 B, 8-row groups 1024 B apart
            const uint64_t desc_x = make_desc(x_smem + ks * 32, 16, 1024);
            const uint32_t d = tmem_d;
            const uint32_t accumulate = (kb | ks) != 0 ? 1u : 0u;
            if (kATmem) {
              // 16 k-values of a lane are 8 columns of 32 bits
              umma_ts(d, tmem_base + kAColumn0 + (uint32_t)s * kAStageColumns + (uint32_t)ks * 8u, desc_x, idesc, accumulate);
            } else {
              umma(d, make_desc(stage + ks * 32, 16, 1024), desc_x, idesc, accumulate);
            }
          }
          umma_commit(empty(s));
          if (prof) t_issue += clock64() - t_mark;
        }
        if (alive) umma_commit(accum_full(acc));
      }
      if (prof) {
        p.diagnostics[8] = (unsigned long long)(clock64() - t_begin);  // MMA thread: whole loop
        p.diagnostics[9] = (unsigned long long)t_wait;                 //   waiting for a full stage
        p.diagnostics[10] = (unsigned long long)t_issue;               //   fence + 4 MMAs + commit
        p.diagnostics[11] = (unsigned long long)g;                     //   k-blocks
      }
    }
    __syncwarp();
  } else if (warp < kExpanderWarps) {
    // ---- expanders: one weight row per thread, 64 k-values per k-block -----------------------
    const int group = warp / kGroupWarps;
    const int quadrant = warp % kGroupWarps;
    const int row_in_slab = quadrant * 32 + lane;
    const uint32_t minus_one = p.is_half ? 0xBC00BC00u : 0xBF80BF80u;
    const uint32_t lane_address = tmem_base + ((uint32_t)(quadrant * 32) << 16) + kAColumn0;
    const uint32_t smem_row = (uint32_t)(row_in_slab * 128);
    const int swizzle = row_in_slab & 7;
    bool alive = true;
    int first = 0;  // k-blocks of the slabs before the current one
    int h = 0;      // chunks of bits before the current one
    // this thread's 8 bytes per k-block sit at row * 64 + (k-block % 8) * 8 of a chunk; rows past
    // the slab read whatever the ring holds there: they are computed and never stored
    const uint32_t my_bits = bits_base + (uint32_t)(row_in_slab < p.slab_rows ? row_in_slab : 0) * kChunkRowBytes;
    const bool prof = p.profile && blockIdx.x == 0 && p.diagnostics && threadIdx.x == 0;
    long long t_begin = prof ? clock64() : 0, t_bits = 0, t_empty = 0, t_store = 0, t_mark = 0;
    for (int slab = blockIdx.x; slab < p.slabs && alive; slab += gridDim.x) {
      for (int c = 0; c < chunks && alive; ++c, ++h) {
        const int b = h % kBitStages;
        if (prof) t_mark = clock64();
        alive = __all_sync(0xffffffffu, WAIT(bits_full(b), (h / kBitStages) & 1));
        if (prof) t_bits += clock64() - t_mark;
        if (!alive) break;
        // both of this group's k-blocks of the chunk (kb = 8c + group and 8c + group + 4) are read
        // now, so the slot can go back to the producer before the expansion starts
        uint32_t words[2][2];
#pragma unroll
        for (int i = 0; i < 2; ++i)
          asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(words[i][0]), "=r"(words[i][1])
                       : "r"(my_bits + b * kBitStageBytes + (uint32_t)(group + kGroups * i) * 8u) : "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(bits_empty(b));
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int kb = c * kChunkBlocks + group + kGroups * i;
          if (kb >= p.kblocks) break;
          const int n = first + kb;
          const int s = n % kStages;
          // warp-uniform: the tensor-memory store below is a warp-wide instruction
          if (prof) t_mark = clock64();
          alive = __all_sync(0xffffffffu, WAIT(empty(s), ((n / kStages) & 1) ^ 1));
          if (prof) { const long long now = clock64(); t_empty += now - t_mark; t_mark = now; }
          if (!alive) break;
          const uint32_t lo = words[i][0], hi = words[i][1];
          if (kATmem) {
            tc_fence_after();
            uint32_t r[32];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const uint4 lower = expand_byte((lo >> (8 * e)) & 0xffu, minus_one);
              const uint4 upper = expand_byte((hi >> (8 * e)) & 0xffu, minus_one);
              r[4 * e] = lower.x; r[4 * e + 1] = lower.y; r[4 * e + 2] = lower.z; r[4 * e + 3] = lower.w;
              r[16 + 4 * e] = upper.x; r[16 + 4 * e + 1] = upper.y; r[16 + 4 * e + 2] = upper.z; r[16 + 4 * e + 3] = upper.w;
            }
            tmem_store32(lane_address + (uint32_t)s * kAStageColumns, r);
            tc_fence_before();
          } else {
            const uint32_t base = smem_base + s * kStageBytes + smem_row;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              st_shared_v4(base + ((e ^ swizzle) << 4), expand_byte((lo >> (8 * e)) & 0xffu, minus_one));
              st_shared_v4(base + (((e + 4) ^ swizzle) << 4), expand_byte((hi >> (8 * e)) & 0xffu, minus_one));
            }
            fence_proxy_async();
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(full(s));
          if (prof) t_store += clock64() - t_mark;
        }
      }
      first += p.kblocks;
    }
    if (prof) {
      p.diagnostics[12] = (unsigned long long)(clock64() - t_begin);  // expander warp 0: whole loop
      p.diagnostics[13] = (unsigned long long)t_bits;                 //   waiting for a chunk of bits
      p.diagnostics[14] = (unsigned long long)t_empty;                //   waiting for a free stage
      p.diagnostics[15] = (unsigned long long)t_store;                //   expand + store + arrive
    }
  } else {
    // ---- epilogue: D^T[weight row, token] -> Y[token, weight row] ----------------------------
    const int quadrant = warp - kExpanderWarps;
    const int row_in_slab = quadrant * 32 + lane;
    TO* out = static_cast<TO*>(p.out);
    int lt = 0;
    for (int slab = blockIdx.x; slab < p.slabs; slab += gridDim.x, ++lt) {
      const int acc = lt & 1;
      if (!WAIT(accum_full(acc), (lt >> 1) & 1)) break;
      tc_fence_after();
      const long long row = (long long)slab * p.slab_rows + row_in_slab;
      const bool valid = row_in_slab < p.slab_rows && row < p.N;
      const float scale = valid ? p.scale[row] : 0.0f;
      const float bias = (valid && p.bias) ? p.bias[row] : 0.0f;
      const uint32_t address = tmem_base + ((uint32_t)(quadrant * 32) << 16) + (uint32_t)acc * kAccumColumns;
      for (int c0 = 0; c0 < np; c0 += 16) {
        float v[16];
        tmem_load16(address + (uint32_t)c0, v);
        if (valid) {
#pragma unroll
          for (int e = 0; e < 16; ++e)
            if (c0 + e < p.M) DType<TO>::store(out + (long long)(c0 + e) * p.N + row, v[e] * scale + bias);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(accum_empty(acc));
    }
  }
#undef WAIT

  tc_fence_before();
  __syncthreads();
  if (warp == kTmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemColumns);
  }
}

typedef CUresult (*EncodeTiledWs)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledWs encode_tiled_ws() {
  static EncodeTiledWs cached = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult query;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &query) == cudaSuccess &&
        query == cudaDriverEntryPointSuccess)
      cached = reinterpret_cast<EncodeTiledWs>(entry);
  }
  return cached;
}

// which variant runs: 0 tensor-memory A operand (default), 1 shared-memory A operand
int ws_variant() {
  static const int variant = getenv("QSTE_B200_WS_VARIANT") ? atoi(getenv("QSTE_B200_WS_VARIANT")) : 0;
  return variant;
}

template <typename TO, bool kATmem>
int launch_ws(const CUtensorMap& map, const CUtensorMap& map_bits, const WsParams& params, int grid, cudaStream_t stream) {
  auto kernel = packed_gemm_ws_kernel<TO, kATmem>;
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 64 || !configured[device]) {
    const cudaError_t error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   (int)WsShape<kATmem>::kSmemBytes);
    if (error != cudaSuccess) {
      set_last_cuda_error(error, "cudaFuncSetAttribute(packed_gemm_ws)");
      return QSTE_ERR_CUDA;
    }
    if (device >= 0 && device < 64) configured[device] = true;
  }
  kernel<<<(unsigned)grid, kThreads, WsShape<kATmem>::kSmemBytes, stream>>>(map, map_bits, params);
  note_launches(1);
  return launch_status("packed_gemm_ws");
}

}  // namespace

bool ws_supported(int64_t samples, int64_t rows, int64_t columns, int dtype, const void* x, const void* bits,
                  const void* out, int out_dtype) {
  if (samples < 1 || samples > kMaxTokens || rows < 1 || columns < kBK) return false;
  if (dtype != QSTE_BF16 && dtype != QSTE_F16) return false;   // fp32 inputs take the three-plane kernel
  if (out_dtype != dtype) return false;
  if (columns % 128 != 0) return false;   // whole k-blocks, and bit rows that start on 16-byte boundaries (TMA)
  if (!aligned(x, 16) || !aligned(bits, 16) || !aligned(out, 2)) return false;
  if (rows > (1ll << 30) || columns > (1ll << 30)) return false;
  return check_arch() == QSTE_OK;
}

// Slabs of weight rows: 128-row slabs when those already give every SM one, else
// ceil(N / SMs) rows each, so that one wave covers the matrix (97 rows at N = 14336 on 148 SMs).
void ws_slabs(int64_t rows, int* slab_rows, int* slabs) {
  const int sms = sm_count();
  long long count = ceil_div(rows, kSlabRows);
  if (count < sms) count = rows < sms ? rows : sms;
  *slab_rows = (int)ceil_div(rows, count);
  *slabs = (int)ceil_div(rows, *slab_rows);
}

// Where the weight-stationary kernel beats the others (graph-replay times over rotating weight
// copies, bf16): its cost is the number of MMAs a CTA issues -- about 160 cycles each at M = 128,
// K = 16, whatever the token count -- so it wins where a slab's contraction is short and the
// matrix is wide enough to give every SM a slab: 4096 -> 14336 takes 25.6-32.3 us for 1..128 tokens
// against 28.9-36.8 us on the 256-column tiles of the large-batch kernel (and 38.4 us for the
// four-token table kernel), while 14336 -> 4096 takes 76 us against 27.
bool ws_preferred(int64_t samples, int64_t rows, int64_t columns) {
  if (columns > 4096) return false;
  return samples <= 4 ? rows >= 8192 : rows >= 12288;
}

int ws_forward(const void* x, int dtype, int64_t samples, const uint8_t* packed, const float* scale, const float* bias,
               int64_t rows, int64_t columns, void* out, int out_dtype, unsigned long long* diagnostics,
               cudaStream_t stream) {
  EncodeTiledWs encode = encode_tiled_ws();
  if (!encode) return QSTE_ERR_CUDA;
  WsParams params = {};
  params.bits = packed;
  params.bit_pitch = (columns + 7) / 8;
  params.scale = scale;
  params.bias = bias;
  params.out = out;
  params.M = samples; params.N = rows; params.K = columns;
  params.tokens_padded = (int)(ceil_div(samples, 16) * 16);
  const int sms = sm_count();
  ws_slabs(rows, &params.slab_rows, &params.slabs);
  params.kblocks = (int)(columns / kBK);
  params.is_half = dtype == QSTE_F16 ? 1 : 0;
  params.diagnostics = diagnostics;
  {
    static const int profile = getenv("QSTE_B200_WS_PROFILE") ? atoi(getenv("QSTE_B200_WS_PROFILE")) : 0;
    params.profile = profile;
  }

  // X as a [M, K] row-major 16-bit matrix; boxes of 64 k-values x Np rows (rows past M read 0)
  CUtensorMap map;
  cuuint64_t dims[2] = {(cuuint64_t)columns, (cuuint64_t)samples};
  cuuint64_t strides[1] = {(cuuint64_t)columns * 2};
  cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)params.tokens_padded};
  cuuint32_t element_strides[2] = {1, 1};
  const CUresult result = encode(&map, dtype == QSTE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                                 2, const_cast<void*>(x), dims, strides, box, element_strides,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (result != CUDA_SUCCESS) {
    set_last_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(ws)");
    return QSTE_ERR_CUDA;
  }
  // the sign bits as a [N, K/8] byte matrix; boxes of 64 bytes (eight k-blocks) x slab_rows rows
  CUtensorMap map_bits;
  cuuint64_t bit_dims[2] = {(cuuint64_t)params.bit_pitch, (cuuint64_t)rows};
  cuuint64_t bit_strides[1] = {(cuuint64_t)params.bit_pitch};
  cuuint32_t bit_box[2] = {(cuuint32_t)kChunkRowBytes, (cuuint32_t)params.slab_rows};
  const CUresult bit_result = encode(&map_bits, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(packed), bit_dims,
                                     bit_strides, bit_box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                     CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (bit_result != CUDA_SUCCESS) {
    set_last_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(ws bits)");
    return QSTE_ERR_CUDA;
  }
  const int grid = params.slabs < sms ? params.slabs : sms;
  const bool a_in_tmem = ws_variant() == 0;
  if (out_dtype == QSTE_F16)
    return a_in_tmem ? launch_ws<__half, true>(map, map_bits, params, grid, stream)
                     : launch_ws<__half, false>(map, map_bits, params, grid, stream);
  return a_in_tmem ? launch_ws<__nv_bfloat16, true>(map, map_bits, params, grid, stream)
                   : launch_ws<__nv_bfloat16, false>(map, map_bits, params, grid, stream);
}

}  // namespace qste
