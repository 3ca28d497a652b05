// PTX wrappers shared by the tcgen05 kernels (sm_100a): mbarriers with bounded waits, TMA
// loads, tensor-memory allocation, tcgen05.mma / commit / ld / st, shared-memory matrix
// descriptors, and the sign-bit expansion.  Header-only; every function is inlined.
#pragma once

#include <cuda.h>
#include <stdint.h>

#include "common.cuh"

namespace qste {
namespace {

// polls before a bounded wait gives up (about a second of wall time with the back-off below)
constexpr uint32_t kSpinLimit = 1u << 22;

// ---- PTX wrappers ---------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
// Non-blocking probe of a phase (the MMA thread issues it one k-block early so that its
// latency overlaps the issue of the current MMAs).  kCluster: the barrier also receives
// arrivals from the other CTA of a pair, so the wait acquires at cluster scope.
template <bool kCluster>
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t done;
  if (kCluster)
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  else
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
// Bounded wait.  Returns false (and raises the abort flag) when it gives up.
// `site`: the source line of the wait; the first wait to give up leaves it, with its block and
// thread, in word 25 of the diagnostics header (bytes 200..207 of the workspace).
template <bool kCluster = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          unsigned long long* diagnostics, unsigned site = 0) {
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    if (kCluster ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity)) return true;
    if (spin > 64) {
      __nanosleep(spin > 4096 ? 256 : 32);
      if (*abort_flag) return false;
    }
  }
  *abort_flag = 1;
  if (diagnostics) {
    atomicAdd(diagnostics, 1ull);
    atomicCAS(diagnostics + 25, 0ull,
              ((unsigned long long)site << 32) | ((unsigned long long)(blockIdx.x & 0xffffu) << 16) | threadIdx.x);
  }
  return false;
}

// ---- what the two-CTA mode adds ----
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the barrier at the same offset in CTA `rank` of the cluster.  Default semantics
// (release at CTA scope): with .release.cluster the instruction held its thread for ~1100
// cycles.  What it orders here was written to this SM's own shared memory or tensor memory and
// was already complete when the arriving thread observed a CTA-scope barrier or wait.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar, uint32_t rank) {
  asm volatile(
      "{\n\t.reg .b32 remote;\n\t"
      "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
      "mbarrier.arrive.shared::cluster.b64 _, [remote];\n\t}"
      ::"r"(bar), "r"(rank) : "memory");
}
// the same with release semantics at cluster scope: orders this thread's earlier remote store
__device__ __forceinline__ void mbar_arrive_remote_release(uint32_t bar, uint32_t rank) {
  asm volatile(
      "{\n\t.reg .b32 remote;\n\t"
      "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
      "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [remote];\n\t}"
      ::"r"(bar), "r"(rank) : "memory");
}
__device__ __forceinline__ void st_shared_remote_u32(uint32_t address, uint32_t rank, uint32_t value) {
  asm volatile(
      "{\n\t.reg .b32 remote;\n\t"
      "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
      "st.shared::cluster.u32 [remote], %2;\n\t}"
      ::"r"(address), "r"(rank), "r"(value) : "memory");
}
// A-tile load of one CTA of a pair; the completion bytes go to the barrier of the even CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem), "l"(map), "r"(bar & 0xFEFFFFFFu), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_slot, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(columns) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrive (when the MMAs issued so far complete) on the barrier at this offset in BOTH CTAs
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((unsigned short)3) : "memory");
}

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(uint32_t smem, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(columns) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_load32(uint32_t address, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(address) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(r[e]);
}

// Shared-memory matrix descriptor, 128-byte swizzle (layout type 2), descriptor version 1.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_address, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t desc = 0;
  desc |= (uint64_t)((smem_address & 0x3ffff) >> 4);
  desc |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  desc |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  desc |= (uint64_t)1 << 46;
  desc |= (uint64_t)2 << 61;
  return desc;
}

// Eight sign bits -> eight 16-bit values: a set bit flips the sign of `negative`
// (a pair of identical negative 16-bit patterns).
__device__ __forceinline__ uint4 expand_byte(uint32_t byte, uint32_t negative) {
  const uint32_t z = byte * 0x8001u;  // bit b of the byte now also sits at bit b + 15
  uint4 v;
  v.x = ((z << 15) & 0x80008000u) ^ negative;
  v.y = ((z << 13) & 0x80008000u) ^ negative;
  v.z = ((z << 11) & 0x80008000u) ^ negative;
  v.w = ((z << 9) & 0x80008000u) ^ negative;
  return v;
}

__device__ __forceinline__ void st_shared_v4(uint32_t address, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(address), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}


// 32 bytes from one lane in one instruction: a row-per-lane store then writes whole 32-byte
// sectors, instead of two half-sector writes that L2 has to merge
__device__ __forceinline__ void st_global_v8(void* destination, const uint32_t* w) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(destination), "r"(w[0]), "r"(w[1]),
               "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}

// One lane writes 32 consecutive outputs of its row.  `wide_ok`: the row start is 32-byte
// aligned; `vector_ok`: 16-byte aligned.  Constant indices only: a dynamic index would move
// v[] to local memory.
template <typename TO>
__device__ __forceinline__ void store_row32(TO* destination, const float* v, bool vector_ok, bool wide_ok, int valid) {
  if (vector_ok && valid == 32) {
    constexpr int kWords = 32 * (int)sizeof(TO) / 4;
    uint32_t words[kWords];
    if constexpr (sizeof(TO) == 4) {
#pragma unroll
      for (int e = 0; e < 32; ++e) words[e] = __float_as_uint(v[e]);
    } else {
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        TO lo, hi;
        DType<TO>::store(&lo, v[2 * e]);
        DType<TO>::store(&hi, v[2 * e + 1]);
        words[e] = (uint32_t)(*reinterpret_cast<unsigned short*>(&lo)) |
                   ((uint32_t)(*reinterpret_cast<unsigned short*>(&hi)) << 16);
      }
    }
    if (wide_ok) {
#pragma unroll
      for (int e = 0; e < kWords / 8; ++e) st_global_v8(reinterpret_cast<uint32_t*>(destination) + 8 * e, words + 8 * e);
    } else {
#pragma unroll
      for (int e = 0; e < kWords / 4; ++e)
        reinterpret_cast<uint4*>(destination)[e] = make_uint4(words[4 * e], words[4 * e + 1], words[4 * e + 2], words[4 * e + 3]);
    }
  } else {
#pragma unroll
    for (int e = 0; e < 32; ++e)
      if (e < valid) DType<TO>::store(destination + e, v[e]);
  }
}


}  // namespace
}  // namespace qste
