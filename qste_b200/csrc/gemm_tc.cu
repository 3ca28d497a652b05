// tcgen05 / TMEM packed-sign GEMM for sm_100a.
//
// All three products of the binary Linear are  C[i, j] = sum_k A(i, k) * B(j, k)
// where A is a dense 16-bit activation / gradient operand and B exists in memory
// only as packed sign bits (plus, for two of the products, one fp32 scale per k):
//
//   forward   A = X [I, K] row-major              B(j, k) = sign(W)[j, k]              bits [J, K/8]
//   dX        A = dY [I, K] row-major             B(j, k) = scale[k] * sign(W)[k, j]   bits [K, J/8]
//   evidence  A(i, k) = dY[k, i]  (dY^T)          B(j, k) = x_scale[k] * sign(x)[k, j] bits [K, J/8]
//
// A persistent kernel, at most one CTA of 22 warps per SM, walks tiles of C (three tile
// modes, see TcShape) through a shared-memory ring of stages:
//
//   warps 0-15  expanders, two groups that alternate k-blocks: read the packed bits of the B
//               tile straight from global memory (they are 1/16 of the expanded tile), turn
//               every byte into eight +-1 or +-scale 16-bit values with three integer ops per
//               pair, and store them in the canonical UMMA shared-memory layout (128B
//               swizzle; K-major for the forward, MN-major for the other two, because the
//               packed dimension is then the output dimension); fence.proxy.async, mbarrier
//               arrive.  With 256-row tiles they also take four fifths of the epilogue.
//   warps 16-19 epilogue: tcgen05.ld the accumulator, apply the fp32 per-row / per-column
//               scale, bias and rank-one correction, reduce the row-inner product against the
//               weight bits, and store
//   warp 20     TMA producer: cp.async.bulk.tensor loads of the A tile (128B swizzle), one
//               elected lane, completion on an mbarrier (no multicast anywhere); it also takes
//               the CTA's next work item from a global counter and queues it for the other roles
//   warp 21     MMA issuer: one elected lane issues tcgen05.mma kind::f16 (M = 128, or 256 for a
//               pair of CTAs; N = 256, K = 16) with the fp32 accumulators in TMEM, and
//               tcgen05.commit to hand the stage back
//
// Scales indexed by an OUTPUT dimension stay in fp32 and are applied in the epilogue.
// Scales indexed by the CONTRACTION dimension (dX: row scale; evidence: sample scale)
// ride the expanded operand as fp16(scale * 2^e), e chosen from the largest scale so
// the fp16 range is used fully; the epilogue multiplies by 2^-e.  That costs 2^-12
// relative per term instead of the 2^-9 a bf16 operand would.  kind::f16 needs both
// operands in ONE 16-bit format (a bf16 A with an fp16 B is an illegal instruction), so a
// bf16 gradient is first re-encoded as fp16(dY * 2^a), a from its largest magnitude: the
// 8-bit bf16 mantissa fits the fp16 one, so every element within 2^-28 of the largest
// converts exactly.
// fp32 activations are split by a small pre-pass into three bf16 planes (a contraction
// scale is folded in there, in fp32) that are contracted one after the other, which
// reproduces an fp32 GEMM to ~2^-24.
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls the waiting thread adds 1
// to a diagnostics counter (the first one also leaves its source line, CTA and thread there),
// raises a CTA-wide abort flag, and every role leaves its loop; TMEM is released on every path.
#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"
#include "gemm.h"
#include "tcgen05.cuh"

namespace qste {
namespace {

constexpr int kBM = 128, kBN = 256, kBK = 64;
constexpr int kGroups = 2, kGroupWarps = 8, kGroupThreads = kGroupWarps * 32;
constexpr int kExpanderWarps = kGroups * kGroupWarps;
constexpr int kEpilogueWarps = 4;
constexpr int kTmaWarp = kExpanderWarps + kEpilogueWarps, kMmaWarp = kTmaWarp + 1;
constexpr int kThreads = (kMmaWarp + 1) * 32;
constexpr uint32_t kABytes = kBM * kBK * 2;
constexpr uint32_t kTmemColumns = 512;  // two 128 x 256 fp32 accumulators

// Tile modes.
//   short   one CTA, tiles of 128 x 256, four stages of (A 16 KB + B 32 KB), two alternating
//           accumulators.
//   tall    one CTA, tiles of 256 x 256: two M = 128 MMAs share one expanded B tile; three stages
//           of (A 32 KB + B 32 KB).
//   pair    a cluster of two CTAs, tiles of 512 x 256 (cta_group::2): each CTA holds 256 rows of A
//           and expands 128 of the 256 rows of B; an MMA of the pair (M = 256) takes 128 rows of A
//           and half of B from each CTA's shared memory, so per MMA an SM reads 8 KB of operands
//           instead of 12 and writes half as much expanded B.  Four stages of (A 32 KB + B 16 KB).
//           Shared-memory bandwidth is what bounds the single-CTA modes (160 KB per k-block of a
//           256 x 256 tile at 128 B/clk is the ~1300 cycles measured).
enum TcMode { kModeShort = 0, kModeTall = 1, kModePair = 2 };
template <int kMode> struct TcShape {
  static constexpr bool kIsTall = kMode != kModeShort;
  static constexpr bool kIsPair = kMode == kModePair;
  static constexpr int kTileRows = kIsTall ? 2 * kBM : kBM;           // rows of C per CTA and tile
  static constexpr int kItemRows = kIsPair ? 2 * kTileRows : kTileRows;  // rows of C per tile
  static constexpr uint32_t kABytes = kTileRows * kBK * 2;
  static constexpr int kBRows = kIsPair ? kBN / 2 : kBN;               // rows of B this CTA expands
  static constexpr uint32_t kBBytes = kBRows * kBK * 2;
  static constexpr int kStages = kMode == kModeTall ? 3 : 4;
  static constexpr int kCtas = kIsPair ? 2 : 1;
  // warps per TMEM quadrant that share a tile's epilogue: the epilogue warp, plus (tall tiles)
  // the quadrant's four expander warps
  static constexpr int kMembers = kIsTall ? 5 : 1;
  static constexpr uint32_t kSmemBytes = kStages * (kABytes + kBBytes) + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

struct TcParams {
  const uint8_t* bits;
  long long bit_pitch;
  const float* cs;           // contraction scale or null
  const float* mult;         // device {2^e, 2^-e} of the contraction scale, or null
  const float* a_mult;       // device {2^a, 2^-a} applied to A by the pre-pass, or null
  const float* out_scale;    // per column j
  const float* out_bias;     // per column j
  const float* row_add;      // per row i
  const float* row_scale;    // per row i
  const uint8_t* inner_bits; // [I, J/8]
  long long inner_pitch;
  float* inner_partial;      // [tiles_j * members, I]
  void* out;
  int out_dtype;
  long long I, J, K;
  int kblocks_b;      // k-blocks of the bit operand (= of one plane of A)
  int kblocks_total;  // planes * kblocks_b
  int tiles_i, tiles_j;
  int kind;
  int ab_is_half;     // both operands are fp16 (else bf16)
  unsigned long long* diagnostics;
  // Work items.  Item q < split_begin is tile q, whole.  The tiles from split_begin on are cut
  // along the contraction into `slices` items each; such an item leaves its raw fp32
  // accumulators in partial[slot] (slot = q - split_begin, [tile rows][256]) and a second kernel
  // adds the slices of a tile in a fixed order and applies the epilogue.
  int split_begin, slices, items;
  float* partial;
  // Dynamic hand-out of work items (null: item lt of worker w is w + lt * workers).  schedule[0]
  // counts the items handed out beyond the first one of each worker, schedule[1] the workers
  // that are done; the last one resets both, so the two words are zero between launches.
  unsigned* schedule;
  unsigned long long* profile;   // 16 slots, only read by the profiling instantiation
  int profile_cta;               // the CTA that records them
};

// ---- PTX wrappers ---------------------arp's share of it -------------------------------
//
// A tile's accumulators are cut into units of 32 columns x 128 rows; a warp reads the 32 TMEM
// lanes of its quadrant (warp % 4), one row per lane.  With 128-row tiles the four epilogue warps
// take all units (the next tile's MMAs run meanwhile in the other accumulator).  With 256-row
// tiles both accumulators are in use, the tensor pipe idles until they are drained, and the
// expander warps -- which cannot make progress then either -- take four fifths of the units:
// member 0 is the epilogue warp of the quadrant, members 1-4 its expander warps.  Every member
// arrives on accum_empty after its last TMEM load.
//
// Not inlined: it runs once per tile, and kept out of line it does not compete for registers with
// the expanders' k-block loop, which calls it.
struct WorkItem {
  int tile;
  int kb_begin, kb_count;  // k-blocks [kb_begin, kb_begin + kb_count) of the contraction
  int slot;                // -1: whole tile; else index into TcParams::partial
};
__device__ __forceinline__ WorkItem work_item(const TcParams& p, int q) {
  WorkItem w;
  if (q < p.split_begin) {
    w.tile = q; w.kb_begin = 0; w.kb_count = p.kblocks_total; w.slot = -1;
  } else {
    const int r = q - p.split_begin;
    const int t = r / p.slices, slice = r - t * p.slices;
    const int begin = (int)((long long)slice * p.kblocks_total / p.slices);
    const int end = (int)((long long)(slice + 1) * p.kblocks_total / p.slices);
    w.tile = p.split_begin + t; w.kb_begin = begin; w.kb_count = end - begin; w.slot = r;
  }
  return w;
}

struct DrainContext {
  uint32_t tmem_base;
  uint32_t accum_full, accum_empty;  // barriers of accumulator 0; accumulator 1 is 8 bytes on
  volatile int* abort_flag;
  int worker, workers;
  int rank;             // CTA of the pair (0 otherwise)
  long long* counters;  // profiling instantiation only, else null
};

template <typename TO, bool kProfile, int kMode>
__device__ __forceinline__ bool drain_tile(const TcParams& p, const DrainContext& c, int lt, int q, int member) {
  const WorkItem item = work_item(p, q);  // item q is the lt-th of this CTA (pair)
  constexpr bool kTall = TcShape<kMode>::kIsTall;
  constexpr bool kIsPair = TcShape<kMode>::kIsPair;
  constexpr int kTileRows = TcShape<kMode>::kTileRows;
  constexpr int kItemRows = TcShape<kMode>::kItemRows;
  constexpr int kMembers = TcShape<kMode>::kMembers;
  constexpr int kUnits = (kTileRows / kBM) * (kBN / 32);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int lane_quarter = warp & 3;
  const bool prof = kProfile && c.counters != nullptr;
  long long t_mark = 0;
#define PROF_BEGIN() do { if (kProfile && prof) t_mark = clock64(); } while (0)
#define PROF_END(slot) do { if (kProfile && prof) c.counters[slot] += clock64() - t_mark; } while (0)
  const float unscale = ((p.cs && p.mult) ? p.mult[1] : 1.0f) * (p.a_mult ? p.a_mult[1] : 1.0f);
  const bool vector_ok = ((p.J * (long long)sizeof(TO)) % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
  const bool wide_ok = ((p.J * (long long)sizeof(TO)) % 32 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 31) == 0);
  const bool has_affine = p.out_scale != nullptr || p.out_bias != nullptr;

  const int tile = item.tile;
  const int tile_j = tile % p.tiles_j;
  const int rows_before = c.rank * kTileRows;  // rows of the tile that belong to the other CTA of a pair
  const long long i_tile = (long long)(tile / p.tiles_j) * kItemRows + rows_before, j0 = (long long)tile_j * kBN;
  const int acc = kTall ? 0 : (lt & 1);
  // The per-row terms of this lane's row (two rows with 256-row tiles) and the sign word of its first
  // unit are requested BEFORE the wait for the accumulators, and each further sign word one unit
  // ahead: a unit that asked for them where it uses them waited a trip to L2 per 32 columns, which is
  // what bounded products with a short contraction (coordinate evidence of a small batch: one
  // k-block per tile, all epilogue).
  const long long i_first = i_tile + lane_quarter * 32 + lane, i_second = i_first + kBM;
  const bool first_ok = i_first < p.I, second_ok = kTileRows > kBM && i_second < p.I;
  const float add_first = (p.row_add && first_ok) ? __ldg(p.row_add + i_first) : 0.0f;
  const float add_second = (p.row_add && second_ok) ? __ldg(p.row_add + i_second) : 0.0f;
  const float mul_first = (p.row_scale && first_ok) ? __ldg(p.row_scale + i_first) : 1.0f;
  const float mul_second = (p.row_scale && second_ok) ? __ldg(p.row_scale + i_second) : 1.0f;
  const bool word_loads = (p.inner_pitch & 3) == 0 && (reinterpret_cast<uintptr_t>(p.inner_bits) & 3) == 0;
  auto sign_word_of = [&](int unit) -> uint32_t {
    if (!p.inner_bits || item.slot >= 0 || unit >= kUnits) return 0u;
    const int half = unit / (kBN / 32), chunk = unit % (kBN / 32);
    const long long i = i_tile + half * kBM + lane_quarter * 32 + lane, j = j0 + chunk * 32;
    if (i >= p.I || j >= p.J) return 0u;
    const uint8_t* source = p.inner_bits + i * p.inner_pitch + (j >> 3);
    if (word_loads && j + 32 <= p.J) return __ldg(reinterpret_cast<const uint32_t*>(source));
    uint32_t word = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b)
      if (j + 8 * b < p.J) word |= (uint32_t)source[b] << (8 * b);
    return word;
  };
  uint32_t sign_ahead = sign_word_of(member);
  PROF_BEGIN();
  bool ready = mbar_wait<kIsPair>(c.accum_full + 8u * acc, kTall ? (lt & 1) : ((lt >> 1) & 1), c.abort_flag,
                                  p.diagnostics, __LINE__);
  PROF_END(0);
  ready = __all_sync(0xffffffffu, ready);
  if (!ready) return false;
  tc_fence_after();
  const int last_unit = member + ((kUnits - 1 - member) / kMembers) * kMembers;
  float inner0 = 0.0f, inner1 = 0.0f;
#pragma unroll 1
  for (int unit = member; unit < kUnits; unit += kMembers) {
    const int half = unit / (kBN / 32), chunk = unit % (kBN / 32);
    const long long i = i_tile + half * kBM + lane_quarter * 32 + lane;
    const bool row_ok = i < p.I;
    const float add = half == 0 ? add_first : add_second;
    const float row_mul = half == 0 ? mul_first : mul_second;
    const uint32_t sign_word = sign_ahead;
    sign_ahead = sign_word_of(unit + kMembers);
    const uint32_t tmem_half = c.tmem_base + ((uint32_t)(lane_quarter * 32) << 16) +
                               (uint32_t)((kTall ? half : acc) * kBN);
    const int column = chunk * 32;
    const long long j = j0 + column;
    const int valid = (p.J - j) < 32 ? (int)(p.J - j) : 32;  // <= 0: the chunk lies past J
    // Every index into v[] below is a compile-time constant, so the values stay in registers,
    // and the per-element arithmetic carries no branch: an absent scale, bias or row term is the
    // neutral value.  (A test of p.out_scale per element compiles to a branch per element, which
    // made this loop several times slower than the MMAs it follows.)  Lane e fetches the scale
    // and bias of column j + e -- requested before the TMEM load so that the latencies overlap
    // -- and the warp passes them round by shuffle, which costs no register arrays.
    float scale_e = 1.0f, bias_e = 0.0f;
    if (has_affine) {
      const bool inside = lane < valid;
      if (p.out_scale) scale_e = inside ? __ldg(p.out_scale + j + lane) : 0.0f;
      if (p.out_bias) bias_e = inside ? __ldg(p.out_bias + j + lane) : 0.0f;
      scale_e *= unscale;
    }
    float v[32];
    PROF_BEGIN();
    tmem_load32(tmem_half + (uint32_t)column, v);
    PROF_END(1);
    if (unit == last_unit) {
      // this warp's part of the accumulators is in registers now
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (kIsPair) mbar_arrive_remote(c.accum_empty + 8u * acc, 0);  // the even CTA issues the MMAs
        else mbar_arrive(c.accum_empty + 8u * acc);
      }
    }
    if (valid <= 0) continue;
    if (item.slot >= 0) {
      // a slice of the contraction: the raw sums go to the partial buffer
      if (row_ok) {
        float* raw = p.partial +
                     ((long long)item.slot * kItemRows + rows_before + (half * kBM + lane_quarter * 32 + lane)) * kBN + column;
#pragma unroll
        for (int e = 0; e < 4; ++e) st_global_v8(raw + 8 * e, reinterpret_cast<const uint32_t*>(v) + 8 * e);
      }
      continue;
    }
    PROF_BEGIN();
    if (has_affine) {
#pragma unroll
      for (int e = 0; e < 32; ++e)
        v[e] = v[e] * __shfl_sync(0xffffffffu, scale_e, e) + (__shfl_sync(0xffffffffu, bias_e, e) + add);
    } else {
#pragma unroll
      for (int e = 0; e < 32; ++e) v[e] = v[e] * unscale + add;
    }
    if (p.inner_bits) {
      float sum = 0.0f;
#pragma unroll
      for (int e = 0; e < 32; ++e) sum += (e < valid) ? apply_sign(v[e], (sign_word >> e) & 1u) : 0.0f;
      if (half == 0) inner0 += sum; else inner1 += sum;
    }
    if (p.row_scale) {
#pragma unroll
      for (int e = 0; e < 32; ++e) v[e] *= row_mul;
    }
    PROF_END(2);
    PROF_BEGIN();
    if (row_ok) store_row32<TO>(static_cast<TO*>(p.out) + i * p.J + j, v, vector_ok, wide_ok, valid);
    PROF_END(3);
  }
  if (p.inner_partial && item.slot < 0) {
    // one slot per (column tile, member); a later kernel adds the slots in a fixed order
    float* slot = p.inner_partial + ((long long)tile_j * kMembers + member) * p.I;
#pragma unroll
    for (int half = 0; half < kTileRows / kBM; ++half) {
      const long long i = i_tile + half * kBM + lane_quarter * 32 + lane;
      if (i < p.I) slot[i] = half == 0 ? inner0 : inner1;
    }
  }
#undef PROF_BEGIN
#undef PROF_END
  return true;
}

// ---- the kernel -----------------------------------------------------------------------
//
// Persistent: one CTA per SM walks tiles  blockIdx.x, blockIdx.x + gridDim.x, ...  (tiles are
// numbered with j fastest, so the CTAs of one wave share a few rows of A and all of the
// packed operand through L2).
//
//   warps 0-15   expanders, two groups of eight     warps 16-19  epilogue
//   warp 20      TMA producer                        warp 21      MMA issuer
//
// Tall tiles (256 rows per CTA, the normal case): each k-block brings 256 rows of A (32 KB) and
// ONE expanded B tile; the MMA thread issues two MMAs per 16 k-values, one per accumulator,
// against the same B tile.  The expansion, its shared-memory stores and its ALU work are thereby
// paid once per 256 rows of output instead of once per 128, which is what matters: the tensor
// core's operand reads already take most of the shared-memory bandwidth, so everything else
// that touches shared memory competes with it.  Both accumulators (2 x 256 columns) fill TMEM,
// so the epilogue of a tile does not overlap the next tile's MMAs; the expander warps share it.
// Short tiles (128 rows): two alternating accumulators, the epilogue overlaps the next tile,
// used when the output has few rows or few tiles.
//
// A stage holds the A tile and the B tile behind ONE full barrier (the TMA thread and the
// expander warps all arrive on it), so the MMA thread has a single barrier per k-block, and it
// probes that barrier one k-block early: issuing tcgen05.mma blocks while the tensor pipe is
// busy, so anything else on that thread's path is lost tensor time.
// The two expander groups alternate k-blocks, so the store and proxy-fence latency of one
// k-block hides behind the other group's work; each thread fetches the packed bits (and scale)
// of its next k-block one round ahead, into registers.
//
// kProfile: CTA 0 records, per role, cycles spent in its loop and in each kind of wait
// (p.profile[0..15]).  Off in normal launches.

template <typename TO, bool kProfile, int kMode>
__global__ void __launch_bounds__(kThreads, 1)
packed_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ TcParams p) {
  using Shape = TcShape<kMode>;
  constexpr bool kTall = Shape::kIsTall;
  constexpr bool kIsPair = Shape::kIsPair;
  constexpr int kStages = Shape::kStages;
  constexpr int kTileRows = Shape::kTileRows;
  constexpr uint32_t kTileABytes = Shape::kABytes;
  constexpr uint32_t kBBytes = Shape::kBBytes;
  constexpr uint32_t kStageBytes = kTileABytes + kBBytes;
  const bool prof = kProfile && (int)blockIdx.x == p.profile_cta && p.profile != nullptr;
  long long t_total = 0, t_w0 = 0, t_w1 = 0, t_w2 = 0, t_mark = 0;
#define PROF_BEGIN() do { if (kProfile && prof) t_mark = clock64(); } while (0)
#define PROF_END(acc) do { if (kProfile && prof) acc += clock64() - t_mark; } while (0)
#define WAIT(bar, parity) mbar_wait<kIsPair>(bar, parity, abort_flag, p.diagnostics, __LINE__)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  // stage s: A tile at smem_base + s * kStageBytes, B tile right behind it
  const uint32_t bar_base = smem_base + kStages * kStageBytes;
  // full(s): one arrival of the TMA thread (with the A bytes) plus one per expander warp of the
  // group that wrote the B tile; empty(s): one arrival, from tcgen05.commit
  auto full = [&](int s) { return bar_base + 8u * s; };
  auto empty = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto accum_full = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto accum_empty = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  // ready(s), odd CTA of a pair only: its expander warps arrive here, and one relay thread passes
  // the stage on to the even CTA's full(s) with a single cluster-scope arrive (a release at
  // cluster scope from each of the eight warps cost them ~1000 cycles per k-block)
  auto ready_local = [&](int s) { return bar_base + 8u * (2 * kStages + 4 + s); };
  // The queue of work items: the TMA thread of the (even) CTA takes the next item from a global
  // counter and passes its index to every other role -- of both CTAs of a pair -- through a
  // ring of kQueue words; queue_full(i) says word i is written, queue_empty(i), on the even CTA,
  // that every role has read it.  CTAs that start late (their SM was busy with a kernel of
  // another stream) then simply take fewer items instead of holding the whole launch up.
  constexpr int kQueue = 4;
  auto queue_full = [&](int i) { return bar_base + 8u * (3 * kStages + 4 + i); };
  auto queue_empty = [&](int i) { return bar_base + 8u * (3 * kStages + 4 + kQueue + i); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_aligned + (bar_base - smem_base) + 8 * (3 * kStages + 4 + 2 * kQueue));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile uint32_t* queue_ring = tmem_slot + 2;
  const uint32_t queue_ring_address = smem_u32(tmem_slot + 2);
  // odd CTA of a pair: how many of its readers have read queue word i
  const uint32_t handback_address = smem_u32(tmem_slot + 2 + kQueue);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool a_mn_major = p.kind == TC_EVIDENCE;
  const bool b_mn_major = p.kind != TC_FORWARD;
  // In a pair both CTAs walk the same work items; `rank` selects the 256 rows of A and the 128
  // rows of B this CTA owns.  All cross-CTA signalling goes to the even CTA (rank 0), whose MMA
  // thread issues for both.
  const int rank = kIsPair ? (int)cluster_rank() : 0;
  const int worker = kIsPair ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int workers = kIsPair ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const bool dynamic = p.schedule != nullptr;
  // readers of a queue word: MMA thread (or relay), 16 expander warps, 4 epilogue warps, and the
  // odd CTA's TMA thread
  constexpr int kCtaReaders = 1 + kExpanderWarps + kEpilogueWarps;
  constexpr uint32_t kOddReaders = kCtaReaders + 1;
  // arrivals on queue_empty: this CTA's readers, plus one from the odd CTA of a pair (its last reader)
  constexpr int kQueueReaders = kCtaReaders + (kIsPair ? 1 : 0);
  // accumulator buffers in flight: the tall tile uses both halves of TMEM at once
  constexpr int kMembers = Shape::kMembers;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full(s), 1 + kGroupWarps + (kIsPair ? 1 : 0));
      mbar_init(empty(s), 1);
      mbar_init(ready_local(s), kGroupWarps);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(accum_full(a), 1);
      mbar_init(accum_empty(a), Shape::kCtas * kEpilogueWarps * kMembers);
    }
    for (int i = 0; i < kQueue; ++i) {
      mbar_init(queue_full(i), 1);
      mbar_init(queue_empty(i), kQueueReaders);
    }
    *abort_flag = 0;
    for (int i = 0; i < kQueue; ++i) tmem_slot[2 + kQueue + i] = 0;
    fence_barrier_init();
  }
  if (warp == kTmaWarp) {
    if (kIsPair) tmem_alloc_pair(smem_u32(tmem_slot), kTmemColumns);
    else tmem_alloc(smem_u32(tmem_slot), kTmemColumns);
  }
  tc_fence_before();
  if (kIsPair) cluster_sync_all(); else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  DrainContext drain_context;
  drain_context.tmem_base = tmem_base;
  drain_context.accum_full = accum_full(0);
  drain_context.accum_empty = accum_empty(0);
  drain_context.abort_flag = abort_flag;
  drain_context.worker = worker;
  drain_context.workers = workers;
  drain_context.rank = rank;
  drain_context.counters = nullptr;
  long long drain_counters[4] = {0, 0, 0, 0};  // profiling: wait, TMEM loads, arithmetic, stores
  if (kProfile && prof) drain_context.counters = drain_counters;
  auto drain = [&](int lt, int q, int member) { return drain_tile<TO, kProfile, kMode>(p, drain_context, lt, q, member); };

  // The lt-th item of this CTA (pair), or -1 when there is none (or the kernel is giving up).
  // Called by every lane of a warp role, or by the one active lane of a single-thread role.  One
  // lane waits, reads the word and hands the slot back; a warp role gets the value by shuffle.
  // The producer sits in the even CTA.  A reader there hands back with an arrive on the producer's
  // own barrier (a release at CTA scope, which the producer's wait acquires).  The readers of the
  // odd CTA count themselves in their own shared memory with an acquire-release atomic at CTA
  // scope, and the last of them passes the slot back with ONE remote arrive that releases at
  // cluster scope; the producer's wait acquires at cluster scope.  Every reader's load of the word
  // is thus ordered before the refill by the memory model, and only one thread per item pays for
  // the cluster-scope release (all 22 paying it cost 0.8 % of a large GEMM).  With a CTA-scope
  // remote arrive from each reader, readers of the odd CTA were seen to read a slot AFTER it had
  // been refilled; it took items of a single k-block to show, only then is the producer a full ring
  // ahead.
  auto take = [&](int lt, bool whole_warp) -> int {
    if (!dynamic) {
      const int q = worker + lt * workers;
      return q < p.items ? q : -1;
    }
    const int slot = lt % kQueue;
    int q = -1;
    if (!whole_warp || lane == 0) {
      if (WAIT(queue_full(slot), (lt / kQueue) & 1)) {
        const uint32_t word = queue_ring[slot];
        if (rank == 0) {
          mbar_arrive(queue_empty(slot));
        } else {
          uint32_t before;
          asm volatile("atom.acq_rel.cta.shared::cta.add.u32 %0, [%1], 1;"
                       : "=r"(before) : "r"(handback_address + 4u * slot) : "memory");
          if (before == kOddReaders - 1) {
            asm volatile("st.relaxed.cta.shared::cta.u32 [%0], %1;" ::"r"(handback_address + 4u * slot), "r"(0u) : "memory");
            mbar_arrive_remote_release(queue_empty(slot), 0);
          }
        }
        q = (int)word < p.items ? (int)word : -1;
      }
    }
    if (whole_warp) q = __shfl_sync(0xffffffffu, q, 0);
    return q;
  };

  if (warp == kTmaWarp) {
    // ---- TMA producer ---------------------------------------------------------------
    if (lane == 0) {
      int g = 0;
      bool alive = true;
      if (kProfile && prof) t_total = clock64();
      // hands item q to the other roles as the lt-th of this CTA (pair)
      auto publish = [&](int lt, int q) {
        const int slot = lt % kQueue;
        if (!WAIT(queue_empty(slot), ((lt / kQueue) & 1) ^ 1)) return false;
        queue_ring[slot] = (uint32_t)q;
        mbar_arrive(queue_full(slot));
        if (kIsPair) {
          st_shared_remote_u32(queue_ring_address + 4u * slot, 1, (uint32_t)q);
          mbar_arrive_remote_release(queue_full(slot), 1);
        }
        return true;
      };
      const bool producer = dynamic && rank == 0;
      int upcoming = worker;  // this worker's first item is fixed; the others come from the counter
      if (producer) alive = publish(0, upcoming);
      for (int lt = 0; alive; ++lt) {
        int q;
        unsigned ticket = 0;
        if (producer) {
          q = upcoming;
          if (q >= p.items) break;
          // asked for now, needed only after this item's loads are issued: the round trip of the
          // atomic stays off the path of items that are only a few k-blocks long
          ticket = atomicAdd(p.schedule, 1u);
        } else {
          q = take(lt, false);
          if (q < 0) break;
        }
        const WorkItem item = work_item(p, q);
        const int i0 = (item.tile / p.tiles_j) * Shape::kItemRows + rank * kTileRows;
        for (int kb = item.kb_begin; kb < item.kb_begin + item.kb_count; ++kb, ++g) {
          const int s = g % kStages;
          const uint32_t parity = ((g / kStages) & 1) ^ 1;
          PROF_BEGIN();
          const bool got = WAIT(empty(s), parity);
          PROF_END(t_w0);
          if (!got) { alive = false; break; }
          const uint32_t a_smem = smem_base + s * kStageBytes;
          // a pair: the even CTA expects the bytes of both A tiles on its barrier
          if (rank == 0) mbar_expect_tx(full(s), Shape::kCtas * kTileABytes);
          if (a_mn_major) {
            // boxes of 64 (i) x 64 (k): 8 KB each, i-atoms 8192 B apart
#pragma unroll
            for (int b = 0; b < kTileRows / 64; ++b) {
              if (kIsPair) tma_load_2d_pair(a_smem + b * 8192, &map_a, full(s), i0 + b * 64, kb * kBK);
              else tma_load_2d(a_smem + b * 8192, &map_a, full(s), i0 + b * 64, kb * kBK);
            }
          } else {
            // boxes of 64 (k) x 128 rows: 16 KB each
#pragma unroll
            for (int b = 0; b < kTileRows / kBM; ++b) {
              if (kIsPair) tma_load_2d_pair(a_smem + b * kABytes, &map_a, full(s), kb * kBK, i0 + b * kBM);
              else tma_load_2d(a_smem + b * kABytes, &map_a, full(s), kb * kBK, i0 + b * kBM);
            }
          }
        }
        if (producer && alive) {
          upcoming = workers + (int)ticket;
          alive = publish(lt + 1, upcoming);
        }
      }
      if (dynamic && rank == 0) {
        // the last worker to run out of items leaves the two words zero for the next launch
        __threadfence();
        if (atomicAdd(p.schedule + 1, 1u) == (unsigned)workers - 1u) {
          p.schedule[0] = 0u;
          p.schedule[1] = 0u;
        }
      }
      if (kProfile && prof) { p.profile[0] = clock64() - t_total; p.profile[1] = t_w0; }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // ---- MMA issuer (the even CTA of a pair issues for both) -----------------------------
    if (lane == 0 && rank == 0) {
      // instruction descriptor: D fp32, A and B in one 16-bit format, majors, N = 256, M = 128
      // (256 for a pair: 128 rows from each CTA)
      const uint32_t format = p.ab_is_half ? 0u : 1u;
      const uint32_t idesc = (1u << 4) | (format << 7) | (format << 10) |
                             ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
                             ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)((Shape::kCtas * kBM) >> 4) << 24);
      // MN-major B tile: mn-atoms (64 columns) 1024 B apart, k-groups (8 rows) one row of atoms apart
      constexpr uint32_t kBKGroup = (Shape::kBRows / 64) * 1024;
      int g = 0;
      bool alive = true;
      if (kProfile && prof) t_total = clock64();
      // `ready` is the probe of this k-block's barrier, issued while the previous k-block's
      // MMAs were being issued: in steady state the thread never blocks on a barrier.  (After the
      // last k-block it probes a phase that never comes, which reads false and is not used.)
      bool ready = mbar_test<kIsPair>(full(0), 0);
      for (int lt = 0; alive; ++lt) {
        const int q = take(lt, false);
        if (q < 0) break;
        const WorkItem item = work_item(p, q);
        const int acc = kTall ? 0 : (lt & 1);
        const uint32_t acc_parity = kTall ? ((lt & 1) ^ 1) : (((lt >> 1) & 1) ^ 1);
        PROF_BEGIN();
        const bool free_acc = WAIT(accum_empty(acc), acc_parity);
        PROF_END(t_w2);
        if (!free_acc) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * kBN);
        for (int kb = 0; kb < item.kb_count; ++kb, ++g) {
          const int s = g % kStages;
          if (!ready) {
            PROF_BEGIN();
            const bool got = WAIT(full(s), (g / kStages) & 1);
            PROF_END(t_w0);
            if (!got) { alive = false; break; }
          }
          tc_fence_after();
          ready = mbar_test<kIsPair>(full((g + 1) % kStages), ((g + 1) / kStages) & 1);
          const uint32_t a_smem = smem_base + s * kStageBytes;
          const uint32_t b_smem = a_smem + kTileABytes;
#pragma unroll
          for (int ks = 0; ks < kBK / 16; ++ks) {
            // K-major: 64-element rows of 128 B, 8-row groups 1024 B apart; 16 elements = 32 B.
            // MN-major A: 64(mn) x 8(k) atoms of 1024 B, k-groups 1024 B apart, mn-atoms 8192 B apart.
            // MN-major B: k-groups kBKGroup apart, mn-atoms 1024 B apart.
            const uint64_t desc_b = b_mn_major ? make_desc(b_smem + ks * 2 * kBKGroup, 1024, kBKGroup)
                                               : make_desc(b_smem + ks * 32, 16, 1024);
#pragma unroll
            for (int half = 0; half < kTileRows / kBM; ++half) {
              // rows half * 128 .. + 127 of the tile -> accumulator `half` (tall) or `acc`
              const uint32_t a_half = a_smem + half * kABytes;
              const uint64_t desc_a = a_mn_major ? make_desc(a_half + ks * 2048, 8192, 1024)
                                                 : make_desc(a_half + ks * 32, 16, 1024);
              if (kIsPair) umma_pair(tmem_d + (uint32_t)(half * kBN), desc_a, desc_b, idesc, (kb | ks) != 0 ? 1u : 0u);
              else umma(tmem_d + (uint32_t)(half * kBN), desc_a, desc_b, idesc, (kb | ks) != 0 ? 1u : 0u);
            }
          }
          if (kIsPair) umma_commit_pair(empty(s)); else umma_commit(empty(s));
        }
        if (alive) { if (kIsPair) umma_commit_pair(accum_full(acc)); else umma_commit(accum_full(acc)); }
      }
      if (kProfile && prof) {
        p.profile[2] = clock64() - t_total; p.profile[3] = t_w0; p.profile[4] = 0; p.profile[5] = t_w2;
        p.profile[12] = (unsigned long long)g;
      }
    } else if (kIsPair && lane == 0 && rank == 1) {
      // ---- relay of the odd CTA: stage s of this CTA's B tile is written -> tell the even CTA
      int g = 0;
      bool alive = true;
      for (int lt = 0; alive; ++lt) {
        const int q = take(lt, false);
        if (q < 0) break;
        const WorkItem item = work_item(p, q);
        for (int kb = 0; kb < item.kb_count && alive; ++kb, ++g) {
          const int s = g % kStages;
          PROF_BEGIN();
          alive = mbar_wait<false>(ready_local(s), (g / kStages) & 1, abort_flag, p.diagnostics, __LINE__);
          PROF_END(t_w0);
          PROF_BEGIN();
          if (alive) mbar_arrive_remote(full(s), 0);
          PROF_END(t_w1);
        }
      }
      if (kProfile && prof) { p.profile[3] = t_w0; p.profile[4] = t_w1; p.profile[12] = (unsigned long long)g; }
    }
    __syncwarp();
  } else if (warp < kExpanderWarps) {
    // ---- expanders ------------------------------------------------------------------
    // One group (256 threads) writes the B tile of this CTA, rows of 64 k-values:
    //   single CTA: 256 rows, a thread owns 8 bytes of bits (eight 16-byte chunks)
    //   pair:       128 rows, a thread owns 4 bytes of bits (four chunks): `part` picks which
    const int group = warp / kGroupWarps;
    const int t_group = threadIdx.x - group * kGroupThreads;  // 0..255 inside the group
    const int part = kIsPair ? (t_group >> 7) : 0;
    const int t = kIsPair ? (t_group & 127) : t_group;        // position inside the tile
    const uint32_t minus_one = p.ab_is_half ? 0xBC00BC00u : 0xBF80BF80u;
    const float mult = (p.cs && p.mult) ? p.mult[0] : 1.0f;
    const bool scaled = b_mn_major && p.cs != nullptr;
    const int c = t & 63, q = t >> 6;                      // MN-major: k-row and 64-column atom
    const uint32_t my_offset = b_mn_major ? (uint32_t)(((c >> 3) * (Shape::kBRows / 64) + q) * 1024 + (c & 7) * 128)
                                          : (uint32_t)(t * 128);
    const int swizzle = b_mn_major ? (c & 7) : (t & 7);

    // packed bits (and scale) of this thread for k-block kb of the contraction, column tile j0
    auto fetch = [&](long long j0, int kb, unsigned long long& word, float& value) {
      value = 1.0f;
      const int kb_b = kb % p.kblocks_b;
      const uint8_t* source;
      if (!b_mn_major) {
        long long row = j0 + t;
        if (row >= p.J) row = p.J - 1;  // rows past J are never stored
        source = p.bits + row * p.bit_pitch + (long long)kb_b * 8;
      } else {
        long long krow = (long long)kb_b * kBK + c;
        if (krow >= p.K) krow = p.K - 1;  // A is zero there, any finite value will do
        long long column = j0 + q * 64;
        if (column >= p.J) column = 0;     // columns past J are never stored
        source = p.bits + krow * p.bit_pitch + (column >> 3);
        if (scaled) value = p.cs[krow];
      }
      if (kIsPair) word = *reinterpret_cast<const uint32_t*>(source + 4 * part);
      else word = *reinterpret_cast<const unsigned long long*>(source);
    };
    auto pattern = [&](float value) {
      if (!scaled) return minus_one;
      const uint32_t h = (uint32_t)__half_as_ushort(__float2half_rn(value * mult)) | 0x8000u;
      return h | (h << 16);
    };

    bool alive = true;
    int n = group;  // this group's next k-block, counted over all work items of this CTA
    // Expands this group's k-blocks below `limit`; k-block n of the count is k-block
    // kb_origin + n of the contraction.  No call inside: a call would make the compiler park the
    // prefetched words on the stack, and a store of a value that a load has just requested waits
    // for that load.
    auto run = [&](int limit, long long j0, int kb_origin) {
      if (n >= limit || !alive) return;
      unsigned long long word, next_word;
      float value, next_value;
      fetch(j0, kb_origin + n, word, value);
      for (; n < limit && alive; n += kGroups) {
        fetch(j0, kb_origin + (n + kGroups < limit ? n + kGroups : n), next_word, next_value);
        const int s = n % kStages;
        PROF_BEGIN();
        alive = WAIT(empty(s), ((n / kStages) & 1) ^ 1);
        PROF_END(t_w1);
        PROF_BEGIN();
        if (alive) {
          const uint32_t base = smem_base + s * kStageBytes + kTileABytes + my_offset;
          const uint32_t negative = pattern(value);
          const uint32_t lo = (uint32_t)word, hi = (uint32_t)(word >> 32);
#pragma unroll
          for (int e = 0; e < 4; ++e)
            st_shared_v4(base + (((e + 4 * part) ^ swizzle) << 4), expand_byte((lo >> (8 * e)) & 0xffu, negative));
          if (!kIsPair) {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              st_shared_v4(base + (((e + 4) ^ swizzle) << 4), expand_byte((hi >> (8 * e)) & 0xffu, negative));
          }
          fence_proxy_async();
        }
        __syncwarp();
        if (lane == 0 && alive) mbar_arrive(kIsPair && rank == 1 ? ready_local(s) : full(s));
        PROF_END(t_w2);
        word = next_word;
        value = next_value;
      }
    };
    if (kProfile && prof) t_total = clock64();
    // Stage n % kStages is free once the MMAs of k-block n - kStages are done.  The first kStages
    // k-blocks of an item reuse stages of the item before and can be written while that one is
    // still in TMEM.  With 256-row tiles the others wait for MMAs of their own item, which cannot
    // start before the item before has been drained -- so this warp takes its share of that
    // epilogue first instead of only waiting.
    const int member = 1 + (warp >> 2) % 4;
    int first = 0;  // count of k-blocks before the current item
    int previous = -1, taken = 0;
    for (; alive; ++taken) {
      const int q = take(taken, true);
      if (q < 0) break;
      const WorkItem item = work_item(p, q);
      const long long j0 = (long long)(item.tile % p.tiles_j) * kBN + rank * Shape::kBRows;
      const int origin = item.kb_begin - first;
      if (kTall) {
        run(first + (item.kb_count < kStages ? item.kb_count : kStages), j0, origin);
        if (previous >= 0 && alive) alive = drain(taken - 1, previous, member);
      }
      run(first + item.kb_count, j0, origin);
      first += item.kb_count;
      previous = q;
    }
    if (kTall && alive && previous >= 0) alive = drain(taken - 1, previous, member);
    if (kProfile && prof && threadIdx.x == 0) {
      p.profile[6] = clock64() - t_total; p.profile[7] = t_w0; p.profile[8] = t_w1; p.profile[9] = t_w2;
    }
  } else {
    // ---- epilogue warps ---------------------------------------------------------------
    if (kProfile && prof) t_total = clock64();
    for (int lt = 0;; ++lt) {
      const int q = take(lt, true);
      if (q < 0 || !drain(lt, q, 0)) break;
    }
    if (kProfile && prof && warp == kExpanderWarps && lane == 0) {
      p.profile[10] = clock64() - t_total; p.profile[11] = drain_counters[0]; p.profile[13] = drain_counters[1];
      p.profile[14] = drain_counters[3]; p.profile[15] = drain_counters[2];
    }
  }
#undef PROF_BEGIN
#undef PROF_END
#undef WAIT

  tc_fence_before();
  if (kIsPair) cluster_sync_all(); else __syncthreads();
  if (warp == kTmaWarp) {
    tc_fence_after();
    if (kIsPair) tmem_dealloc_pair(tmem_base, kTmemColumns);
    else tmem_dealloc(tmem_base, kTmemColumns);
  }
}

// ---- small helper kernels ---------------------------------------------------------------

// mult[0] = 2^e, mult[1] = 2^-e with max|cs| * 2^e in (2^13, 2^14]
__global__ void __launch_bounds__(1024) scale_exponent_kernel(const float* __restrict__ cs, long long count, float* mult) {
  __shared__ float shared[1024];
  float local = 0.0f;
  for (long long k = threadIdx.x; k < count; k += blockDim.x) local = fmaxf(local, fabsf(cs[k]));
  shared[threadIdx.x] = local;
  __syncthreads();
  for (int width = 512; width > 0; width >>= 1) {
    if ((int)threadIdx.x < width) shared[threadIdx.x] = fmaxf(shared[threadIdx.x], shared[threadIdx.x + width]);
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float largest = shared[0];
    int e = 0;
    if (largest > 0.0f && isfinite(largest)) {
      int exponent;
      frexpf(largest, &exponent);  // largest = f * 2^exponent, f in [0.5, 1)
      e = 14 - exponent;
      if (e > 100) e = 100;
      if (e < -100) e = -100;
    }
    mult[0] = ldexpf(1.0f, e);
    mult[1] = ldexpf(1.0f, -e);
  }
}

// Largest magnitude of a tensor, as the bit pattern of a non-negative float (so that an
// integer atomicMax orders it); slot must be zeroed first.
template <typename T>
__global__ void __launch_bounds__(256) amax_kernel(const T* __restrict__ a, long long count, unsigned* slot) {
  float local = 0.0f;
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < count; e += (long long)gridDim.x * blockDim.x)
    local = fmaxf(local, fabsf(DType<T>::load(a + e)));
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) local = fmaxf(local, __shfl_xor_sync(0xffffffffu, local, offset));
  if ((threadIdx.x & 31) == 0 && local > 0.0f) atomicMax(slot, __float_as_uint(local));
}

// a_mult[0] = 2^a, a_mult[1] = 2^-a with largest * 2^a in (2^13, 2^14]
__global__ void finish_amax_kernel(const unsigned* slot, float* a_mult) {
  const float largest = __uint_as_float(*slot);
  int a = 0;
  if (largest > 0.0f && isfinite(largest)) {
    int exponent;
    frexpf(largest, &exponent);
    a = 14 - exponent;
    if (a > 120) a = 120;
    if (a < -120) a = -120;
  }
  a_mult[0] = ldexpf(1.0f, a);
  a_mult[1] = ldexpf(1.0f, -a);
}

// bf16 -> fp16(x * 2^a), same layout
__global__ void __launch_bounds__(256)
rescale_to_half_kernel(const __nv_bfloat16* __restrict__ source, long long count, __half* __restrict__ out,
                       const float* __restrict__ a_mult) {
  const float m = a_mult[0];
  const long long vectors = count >> 3;
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < vectors; v += (long long)gridDim.x * blockDim.x) {
    const uint4 raw = reinterpret_cast<const uint4*>(source)[v];
    const __nv_bfloat16* in = reinterpret_cast<const __nv_bfloat16*>(&raw);
    uint4 packed;
    __half* o = reinterpret_cast<__half*>(&packed);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = __float2half_rn(__bfloat162float(in[e]) * m);
    reinterpret_cast<uint4*>(out)[v] = packed;
  }
  if (blockIdx.x == 0)
    for (long long e = (vectors << 3) + threadIdx.x; e < count; e += blockDim.x)
      out[e] = __float2half_rn(__bfloat162float(source[e]) * m);
}

// fp32 -> three 16-bit planes (hi, mid, lo) laid out along the contraction dimension.
//   row-major A [I, K]  -> planes [I, 3 * K]          (stack_rows = 0)
//   evidence dY [K, I]  -> planes [3 * Kpad, I], zero rows between K and Kpad
// A contraction scale, when there is one, is folded in here with one fp32 multiply per
// element (what the reference's CPU kernel does), so the expanded operand stays +-1.
// The contraction index is the column of a row-major A and the row of the stacked form.
template <typename TP>
__global__ void __launch_bounds__(256)
split_planes_kernel(const float* __restrict__ source, long long rows, long long columns,
                    TP* __restrict__ planes, long long padded_rows, int stack_rows,
                    const float* __restrict__ cs) {
  const long long total = (stack_rows ? padded_rows : rows) * columns;
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const long long r = e / columns, c = e - r * columns;
    float x = (r < rows) ? source[r * columns + c] : 0.0f;
    if (cs && r < rows) x = x * cs[stack_rows ? r : c];
    TP hi, mid, lo;
    DType<TP>::store(&hi, x);
    const float r1 = x - DType<TP>::load(&hi);
    DType<TP>::store(&mid, r1);
    DType<TP>::store(&lo, r1 - DType<TP>::load(&mid));
    if (stack_rows) {
      planes[(0 * padded_rows + r) * columns + c] = hi;
      planes[(1 * padded_rows + r) * columns + c] = mid;
      planes[(2 * padded_rows + r) * columns + c] = lo;
    } else {
      planes[r * (3 * columns) + c] = hi;
      planes[r * (3 * columns) + columns + c] = mid;
      planes[r * (3 * columns) + 2 * columns + c] = lo;
    }
  }
}

__global__ void __launch_bounds__(256)
finish_inner_kernel(const float* __restrict__ partial, int slices, long long I, float* __restrict__ out) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= I) return;
  float total = 0.0f;
  for (int s = 0; s < slices; ++s) total += partial[(long long)s * I + i];
  out[i] = total;
}

// Second half of a split tile: adds the slices of the contraction in ascending order and applies
// the epilogue of drain_tile.  One warp per output row, eight columns per lane.
template <typename TO>
__global__ void __launch_bounds__(256) split_finish_kernel(const TcParams p, int tile_rows, int members) {
  const int t = blockIdx.x;
  const int r = blockIdx.y * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int tile = p.split_begin + t;
  const int tile_j = tile % p.tiles_j;
  const long long i = (long long)(tile / p.tiles_j) * tile_rows + r;
  if (r >= tile_rows || i >= p.I) return;
  const long long j = (long long)tile_j * kBN + lane * 8;
  float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
  for (int slice = 0; slice < p.slices; ++slice) {
    const float4* source = reinterpret_cast<const float4*>(
        p.partial + ((long long)(t * p.slices + slice) * tile_rows + r) * kBN + lane * 8);
    const float4 lo = source[0], hi = source[1];
    acc[0] += lo.x; acc[1] += lo.y; acc[2] += lo.z; acc[3] += lo.w;
    acc[4] += hi.x; acc[5] += hi.y; acc[6] += hi.z; acc[7] += hi.w;
  }
  const float unscale = ((p.cs && p.mult) ? p.mult[1] : 1.0f) * (p.a_mult ? p.a_mult[1] : 1.0f);
  const float add = p.row_add ? p.row_add[i] : 0.0f;
  const float row_mul = p.row_scale ? p.row_scale[i] : 1.0f;
  float inner = 0.0f;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const long long column = j + e;
    if (column >= p.J) break;
    float value = acc[e] * unscale;
    if (p.out_scale) value *= p.out_scale[column];
    if (p.out_bias) value += p.out_bias[column];
    value += add;
    if (p.inner_bits) {
      const unsigned bit = (p.inner_bits[i * p.inner_pitch + (column >> 3)] >> (column & 7)) & 1u;
      inner += apply_sign(value, bit);
    }
    DType<TO>::store(static_cast<TO*>(p.out) + i * p.J + column, value * row_mul);
  }
  if (p.inner_partial) {
    inner = warp_sum(inner);
    if (lane == 0) {
      p.inner_partial[((long long)tile_j * members) * p.I + i] = inner;
      for (int member = 1; member < members; ++member)
        p.inner_partial[((long long)tile_j * members + member) * p.I + i] = 0.0f;
    }
  }
}

// ---- host side ------------------------------------------------------------------------

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
  static EncodeTiled cached = nullptr;
  if (cached) return cached;
  void* entry = nullptr;
  cudaDriverEntryPointQueryResult query;
  cudaError_t error = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &query);
  if (error != cudaSuccess || query != cudaDriverEntryPointSuccess || !entry) {
    set_last_cuda_error(error == cudaSuccess ? cudaErrorUnknown : error, "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
    return nullptr;
  }
  cached = reinterpret_cast<EncodeTiled>(entry);
  return cached;
}

// 2-D map over a row-major [outer, inner] 16-bit matrix, box {box_inner, box_outer}, 128B swizzle.
int make_map(CUtensorMap* map, const void* base, bool is_half, long long inner, long long outer,
             int box_inner, int box_outer) {
  EncodeTiled encode = encode_tiled();
  if (!encode) return QSTE_ERR_CUDA;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)inner * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t element_strides[2] = {1, 1};
  CUresult result = encode(map, is_half ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                           const_cast<void*>(base), dims, strides, box, element_strides,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (result != CUDA_SUCCESS) {
    set_last_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
    return QSTE_ERR_CUDA;
  }
  return QSTE_OK;
}

// How one problem is cut into work items (see TcParams).
struct TcPlan {
  int mode;        // TcMode
  int item_rows;   // rows of C per tile
  int tiles_i, tiles_j, split_begin, slices, items, grid;
  size_t partial_bytes;
};

int pair_capacity();

TcPlan tc_plan(long long I, long long J, int kblocks_total) {
  static const bool never_tall = getenv("QSTE_B200_TC_SHORT") != nullptr;    // for A/B timing
  static const bool never_pair = getenv("QSTE_B200_TC_NOPAIR") != nullptr;
  static const bool never_split = getenv("QSTE_B200_TC_NOSPLIT") != nullptr;
  // the persistent GEMMs leave this many SMs alone, for a collective that runs beside them on
  // another stream (its blocks cannot be placed while every SM holds a GEMM block); a per-thread
  // setting, so the workspace query and the call that follows it in one thread see one value
  const int reserved = reserved_sms();
  TcPlan plan;
  int sms = sm_count();
  if (reserved > 0 && reserved < sms - 8) sms -= reserved;
  plan.tiles_j = (int)ceil_div(J, kBN);
  // 256-row tiles whenever the output has more than 128 rows, they still fill the device, and
  // the contraction is long enough to pay for an epilogue that does not overlap the next tile;
  // pairs of CTAs on 512-row tiles when those still fill every pair
  plan.mode = kModeShort;
  // (QSTE_B200_TC_TALL_ANY lifts the length condition: a test switch, it makes items of one or
  // two k-blocks, where the producer of work items runs a whole ring ahead of the slowest reader)
  static const bool tall_any = getenv("QSTE_B200_TC_TALL_ANY") != nullptr;
  if (!never_tall && I > kBM && ceil_div(I, 2 * kBM) * plan.tiles_j >= sms && (kblocks_total >= 8 || tall_any)) plan.mode = kModeTall;
  int workers = sms;
  if (plan.mode == kModeTall && !never_pair) {
    int pairs = pair_capacity();
    if (pairs > sms / 2) pairs = sms / 2;
    if (pairs > 0 && ceil_div(I, 4 * kBM) * plan.tiles_j >= pairs) {
      plan.mode = kModePair;
      workers = pairs;
    }
  }
  plan.item_rows = plan.mode == kModePair ? 4 * kBM : (plan.mode == kModeTall ? 2 * kBM : kBM);
  plan.tiles_i = (int)ceil_div(I, plan.item_rows);
  const long long tiles = (long long)plan.tiles_i * plan.tiles_j;
  plan.split_begin = (int)tiles;
  plan.slices = 1;
  // The tiles of the last, partly filled round of CTAs -- all tiles, when there are fewer than
  // SMs -- are cut along the contraction so that the round keeps every SM busy for a fraction
  // of a tile's time instead of a few SMs for all of it.  At least four k-blocks per slice
  // (eight with 256-row tiles).
  const long long rest = tiles % workers;
  if (!never_split && rest > 0) {
    long long slices = workers / rest;
    const int shortest = plan.mode == kModeShort ? 4 : 8;
    if (slices > kblocks_total / shortest) slices = kblocks_total / shortest;
    if (slices >= 2) {
      plan.split_begin = (int)(tiles - rest);
      plan.slices = (int)slices;
    }
  }
  const long long split_tiles = tiles - plan.split_begin;
  plan.items = (int)(plan.split_begin + split_tiles * plan.slices);
  const int busy = plan.items < workers ? plan.items : workers;
  plan.grid = plan.mode == kModePair ? 2 * busy : busy;
  plan.partial_bytes = (size_t)split_tiles * plan.slices * plan.item_rows * kBN * sizeof(float);
  return plan;
}

struct TcLayout {
  size_t mult, inner_partial, partial, row_vectors, planes, total;
  long long padded_k;
};

TcLayout tc_layout(int kind, long long I, long long J, long long K, int dtype) {
  TcLayout l;
  size_t at = 0;
  l.mult = at; at += 256;
  const long long tiles_j = ceil_div(J, kBN);
  l.inner_partial = at; at = align_up(at + (size_t)(TcShape<kModeTall>::kMembers * tiles_j * I) * sizeof(float), 256);
  const int planes_of_a = dtype == QSTE_F32 ? 3 : 1;
  l.partial = at; at = align_up(at + tc_plan(I, J, planes_of_a * (int)ceil_div(K, kBK)).partial_bytes, 256);
  l.padded_k = ceil_div(K, kBK) * kBK;
  // 2^-a[m] and contraction scale * 2^-a[m] of a gradient re-encoded row by row
  l.row_vectors = at; at = align_up(at + (size_t)2 * (I > K ? I : K) * sizeof(float), 256);
  l.planes = at;
  if (dtype == QSTE_F32) {
    const size_t elements = (kind == TC_EVIDENCE) ? (size_t)3 * l.padded_k * I : (size_t)3 * I * K;
    at = align_up(at + elements * 2, 256);
  } else if (dtype == QSTE_BF16 && kind != TC_FORWARD) {
    at = align_up(at + (size_t)I * K * 2, 256);  // fp16 re-encoding of a bf16 gradient
  }
  l.total = at;
  return l;
}

template <typename TO, bool kProfile, int kMode>
int launch_tc_shape(const CUtensorMap& map, const TcParams& params, int grid, cudaStream_t stream) {
  auto kernel = packed_gemm_tc_kernel<TO, kProfile, kMode>;
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 64 || !configured[device]) {
    cudaError_t error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)TcShape<kMode>::kSmemBytes);
    if (error != cudaSuccess) {
      set_last_cuda_error(error, "cudaFuncSetAttribute(packed_gemm_tc)");
      return QSTE_ERR_CUDA;
    }
    if (device >= 0 && device < 64) configured[device] = true;
  }
  // persistent: at most one CTA per SM
  if (kMode == kModePair) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)grid, 1, 1);
    config.blockDim = dim3(kThreads, 1, 1);
    config.dynamicSmemBytes = TcShape<kMode>::kSmemBytes;
    config.stream = stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = 2;
    attribute.val.clusterDim.y = 1;
    attribute.val.clusterDim.z = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    const cudaError_t error = cudaLaunchKernelEx(&config, kernel, map, params);
    note_launches(1);
    if (error != cudaSuccess) {
      set_last_cuda_error(error, "cudaLaunchKernelEx(packed_gemm_tc, pairs)");
      return QSTE_ERR_CUDA;
    }
    return launch_status("packed_gemm_tc");
  }
  kernel<<<(unsigned)grid, kThreads, TcShape<kMode>::kSmemBytes, stream>>>(map, params);
  note_launches(1);
  return launch_status("packed_gemm_tc");
}

template <typename TO, bool kProfile>
int launch_tc_mode(const CUtensorMap& map, const TcParams& params, const TcPlan& plan, cudaStream_t stream) {
  switch (plan.mode) {
    case kModePair: return launch_tc_shape<TO, kProfile, kModePair>(map, params, plan.grid, stream);
    case kModeTall: return launch_tc_shape<TO, kProfile, kModeTall>(map, params, plan.grid, stream);
    default: return launch_tc_shape<TO, kProfile, kModeShort>(map, params, plan.grid, stream);
  }
}

template <typename TO>
int launch_tc(const CUtensorMap& map, const TcParams& params, const TcPlan& plan, cudaStream_t stream) {
  static const bool profile = getenv("QSTE_B200_TC_PROFILE") != nullptr;
  const int status = profile ? launch_tc_mode<TO, true>(map, params, plan, stream)
                             : launch_tc_mode<TO, false>(map, params, plan, stream);
  if (status != QSTE_OK || plan.slices < 2) return status;
  const int members = plan.mode == kModeShort ? TcShape<kModeShort>::kMembers : TcShape<kModeTall>::kMembers;
  const dim3 grid((unsigned)(plan.items - plan.split_begin) / plan.slices, (unsigned)(plan.item_rows / 8));
  split_finish_kernel<TO><<<grid, 256, 0, stream>>>(params, plan.item_rows, members);
  note_launches(1);
  return launch_status("split_finish");
}

// How many two-CTA clusters of the pair kernel can be resident at once (0: pairs unusable).
int pair_capacity() {
  static int cached[64];
  static bool known[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
  if (known[device]) return cached[device];
  auto kernel = packed_gemm_tc_kernel<__nv_bfloat16, false, kModePair>;
  int clusters = 0;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)TcShape<kModePair>::kSmemBytes) == cudaSuccess) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * (unsigned)sm_count(), 1, 1);
    config.blockDim = dim3(kThreads, 1, 1);
    config.dynamicSmemBytes = TcShape<kModePair>::kSmemBytes;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = 2;
    attribute.val.clusterDim.y = 1;
    attribute.val.clusterDim.z = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess) clusters = 0;
  }
  (void)cudaGetLastError();
  cached[device] = clusters;
  known[device] = true;
  return clusters;
}

}  // namespace

size_t tc_workspace(int kind, int64_t I, int64_t J, int64_t K, int dtype) {
  if (I <= 0 || J <= 0 || K <= 0) return 0;
  return tc_layout(kind, I, J, K, dtype).total;
}

size_t tc_workspace_prepared(int kind, int64_t I, int64_t J, int64_t K) {
  if (I <= 0 || J <= 0 || K <= 0) return 0;
  return tc_layout(kind, I, J, K, QSTE_F16).total;  // fp16 needs no copy of A
}

int tc_prepare_half(const void* a_bf16, int64_t count, const unsigned* amax_slot, float* a_mult,
                    void* out_half, cudaStream_t stream) {
  finish_amax_kernel<<<1, 1, 0, stream>>>(amax_slot, a_mult);
  long long grid = ceil_div(count / 8 + 1, 256);
  const long long cap = (long long)sm_count() * 16;
  if (grid > cap) grid = cap;
  rescale_to_half_kernel<<<(unsigned)grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(a_bf16), count,
                                                            static_cast<__half*>(out_half), a_mult);
  note_launches(2);
  return launch_status("tc_prepare_half");
}

bool tc_supported(int kind, int64_t I, int64_t J, int64_t K, int dtype, const void* a, const void* bits,
                  const void* out, int out_dtype) {
  if (I <= 0 || J <= 0 || K <= 0) return false;
  if (dtype_size(dtype) == 0 || dtype_size(out_dtype) == 0) return false;
  if (check_arch() != QSTE_OK) return false;
  if (!aligned(a, 16) || !aligned(out, 16) || !aligned(bits, 8)) return false;
  if (I > (1ll << 30) || J > (1ll << 30) || K > (1ll << 30)) return false;
  if (ceil_div(I, kBM) * ceil_div(J, kBN) > 0x7fffffffll) return false;
  if (J % 8 != 0) return false;                       // vector stores, row pitch of C
  if (kind == TC_FORWARD) {
    if (K % 64 != 0) return false;                    // whole 8-byte groups of bits per k-block
  } else {
    if (J % 64 != 0) return false;                    // the packed dimension is J
    if (kind == TC_TRANSPOSE && K % 8 != 0) return false;  // TMA row pitch of A
    if (kind == TC_EVIDENCE && I % 8 != 0) return false;
    if (dtype == QSTE_F32 && kind == TC_TRANSPOSE && K % 64 != 0) return false;  // plane boundaries
  }
  return true;
}

int tc_run(const TcProblem& problem, cudaStream_t stream) {
  const int kind = problem.kind;
  const long long I = problem.I, J = problem.J, K = problem.K;
  const TcLayout layout = tc_layout(kind, I, J, K, problem.a_dtype);
  char* workspace = problem.workspace;
  float* mult = reinterpret_cast<float*>(workspace + layout.mult);
  const int planes = problem.a_dtype == QSTE_F32 ? 3 : 1;

  // A operand after the optional pre-pass (fp32 split, bf16 -> fp16 re-encoding)
  // fp32: the scale is folded into the split planes, the kernel then runs unscaled
  const bool scaled = problem.contraction_scale != nullptr && problem.a_dtype != QSTE_F32;
  const bool prepared = problem.a_prepared != nullptr && problem.a_dtype == QSTE_BF16;
  const bool to_half = scaled && problem.a_dtype == QSTE_BF16 && !prepared;  // one 16-bit format for A and B
  float* a_mult = mult + 2;
  unsigned* amax_slot = reinterpret_cast<unsigned*>(mult + 4);
  const void* a = problem.a;
  const long long a_elements = I * K;
  auto capped_grid = [&](long long items) {
    long long grid = ceil_div(items, 256);
    const long long cap = (long long)sm_count() * 16;
    return (unsigned)(grid > cap ? cap : (grid < 1 ? 1 : grid));
  };
  // A bf16 gradient whose rows are contiguous in the contraction (dX) or are the contraction
  // (evidence) is re-encoded in one pass with one power of two per row; the power comes back
  // out through the epilogue's row scale (dX) or rides the contraction scale (evidence).
  const long long a_rows = kind == TC_EVIDENCE ? K : I, a_length = kind == TC_EVIDENCE ? I : K;
  const bool by_rows = to_half && kind != TC_FORWARD && (kind == TC_EVIDENCE || problem.row_scale == nullptr) &&
                       prepare_rows_supported(a_rows, a_length, problem.a);
  float* row_unscale = reinterpret_cast<float*>(workspace + layout.row_vectors);
  float* row_cs = row_unscale + (I > K ? I : K);
  if (by_rows) {
    const int status_of_prepass = prepare_rows(problem.a, nullptr, kind == TC_EVIDENCE ? problem.contraction_scale : nullptr,
                                     a_rows, a_length, workspace + layout.planes, row_unscale, row_cs, nullptr, nullptr,
                                     nullptr, stream);
    if (status_of_prepass != QSTE_OK) return status_of_prepass;
  } else if (to_half) {
    cudaError_t error = cudaMemsetAsync(amax_slot, 0, sizeof(unsigned), stream);
    if (error != cudaSuccess) { set_last_cuda_error(error, "cudaMemsetAsync"); return QSTE_ERR_CUDA; }
    amax_kernel<__nv_bfloat16><<<capped_grid(a_elements), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(problem.a), a_elements, amax_slot);
    finish_amax_kernel<<<1, 1, 0, stream>>>(amax_slot, a_mult);
    note_launches(2);
  }
  const float* contraction_scale = (by_rows && kind == TC_EVIDENCE) ? row_cs : problem.contraction_scale;
  if (planes == 3) {
    const bool stack = kind == TC_EVIDENCE;
    const long long rows = stack ? K : I, columns = stack ? I : K;
    const long long total = (stack ? layout.padded_k : rows) * columns;
    split_planes_kernel<__nv_bfloat16><<<capped_grid(total), 256, 0, stream>>>(
        static_cast<const float*>(problem.a), rows, columns, reinterpret_cast<__nv_bfloat16*>(workspace + layout.planes),
        layout.padded_k, stack ? 1 : 0, problem.contraction_scale);
    note_launches(1);
    a = workspace + layout.planes;
  } else if (by_rows) {
    a = workspace + layout.planes;
  } else if (to_half) {
    rescale_to_half_kernel<<<capped_grid(a_elements / 8 + 1), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(problem.a), a_elements, reinterpret_cast<__half*>(workspace + layout.planes), a_mult);
    note_launches(1);
    a = workspace + layout.planes;
  }
  if (prepared) a = problem.a_prepared;
  const bool a_is_half = problem.a_dtype == QSTE_F16 || to_half || prepared;
  CUtensorMap map;
  int status;
  if (kind == TC_EVIDENCE) {
    const long long outer = planes == 3 ? 3 * layout.padded_k : K;
    status = make_map(&map, a, a_is_half, I, outer, 64, kBK);
  } else {
    status = make_map(&map, a, a_is_half, (long long)planes * K, I, kBK, kBM);
  }
  if (status != QSTE_OK) return status;

  if (scaled) {
    scale_exponent_kernel<<<1, 1024, 0, stream>>>(contraction_scale, K, mult);
    note_launches(1);
  }

  TcParams params = {};
  params.bits = problem.bits;
  params.bit_pitch = problem.bit_pitch;
  params.cs = scaled ? contraction_scale : nullptr;
  params.mult = scaled ? mult : nullptr;
  params.a_mult = prepared ? problem.a_prepared_mult : ((to_half && !by_rows) ? a_mult : nullptr);
  params.out_scale = problem.out_scale;
  params.out_bias = problem.out_bias;
  params.row_add = problem.row_add;
  params.row_scale = (by_rows && kind == TC_TRANSPOSE) ? row_unscale : problem.row_scale;
  params.inner_bits = problem.inner_bits;
  params.inner_pitch = (J + 7) / 8;
  params.inner_partial = problem.inner_bits ? reinterpret_cast<float*>(workspace + layout.inner_partial) : nullptr;
  params.out = problem.out;
  params.out_dtype = problem.out_dtype;
  params.I = I; params.J = J; params.K = K;
  params.kblocks_b = (int)ceil_div(K, kBK);
  params.kblocks_total = planes * params.kblocks_b;
  const TcPlan plan = tc_plan(I, J, params.kblocks_total);
  params.tiles_i = plan.tiles_i;
  params.tiles_j = plan.tiles_j;
  params.split_begin = plan.split_begin;
  params.slices = plan.slices;
  params.items = plan.items;
  params.partial = reinterpret_cast<float*>(workspace + layout.partial);
  // two words of the workspace header (bytes 192..199), zero between launches
  static const bool static_schedule = getenv("QSTE_B200_TC_STATIC") != nullptr;
  params.schedule = (problem.diagnostics && !static_schedule && plan.items > plan.grid / (plan.mode == kModePair ? 2 : 1))
                        ? reinterpret_cast<unsigned*>(problem.diagnostics + 24) : nullptr;
  params.kind = kind;
  params.ab_is_half = a_is_half ? 1 : 0;
  params.diagnostics = problem.diagnostics;
  static const int profile_cta = getenv("QSTE_B200_TC_PROFILE_CTA") ? atoi(getenv("QSTE_B200_TC_PROFILE_CTA")) : 0;
  params.profile_cta = profile_cta;
  params.profile = problem.diagnostics ? problem.diagnostics + 8 : nullptr;  // workspace header bytes 64..191
  switch (problem.out_dtype) {
    case QSTE_F32: status = launch_tc<float>(map, params, plan, stream); break;
    case QSTE_F16: status = launch_tc<__half>(map, params, plan, stream); break;
    case QSTE_BF16: status = launch_tc<__nv_bfloat16>(map, params, plan, stream); break;
    default: return QSTE_ERR_DTYPE;
  }
  if (status != QSTE_OK) return status;
  if (problem.inner_bits && problem.inner_out) {
    const int members = plan.mode == kModeShort ? TcShape<kModeShort>::kMembers : TcShape<kModeTall>::kMembers;
    finish_inner_kernel<<<(unsigned)ceil_div(I, 256), 256, 0, stream>>>(params.inner_partial, params.tiles_j * members,
                                                                        I, problem.inner_out);
    note_launches(1);
    status = launch_status("finish_inner");
  }
  return status;
}

}  // namespace qste
