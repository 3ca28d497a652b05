// Thread-block cluster helpers shared by the small-batch forward kernels (sm_100a).
#pragma once

#include <stdint.h>

namespace qste {

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}

// every thread of every CTA of the cluster; orders shared-memory writes before it against reads after it
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// the float at `local`'s offset in the shared memory of CTA `rank` of this cluster
__device__ __forceinline__ float ld_cluster_f32(const float* local, uint32_t rank) {
  const uint32_t address = (uint32_t)__cvta_generic_to_shared(local);
  float value;
  asm volatile(
      "{\n\t.reg .b32 remote;\n\t"
      "mapa.shared::cluster.u32 remote, %1, %2;\n\t"
      "ld.shared::cluster.f32 %0, [remote];\n\t}"
      : "=f"(value) : "r"(address), "r"(rank) : "memory");
  return value;
}

// slice `rank` of `slices` covers units [begin, end) of the contraction, as evenly as they divide
__device__ __forceinline__ void slice_units(int units, int slices, int rank, int& begin, int& end) {
  begin = (int)((long long)units * rank / slices);
  end = (int)((long long)units * (rank + 1) / slices);
}

}  // namespace qste
