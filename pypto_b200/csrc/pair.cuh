// Device helpers for kernels that run on a PAIR of SMs (a cluster of two CTAs driving one tcgen05 instruction
// stream with .cta_group::2): cluster rank and barrier, addresses in the partner's shared memory, loads whose
// completion bytes go to the leader's mbarrier, pair-wide commits and tensor-memory allocation.
// No load here is multicast: each CTA fetches its own bytes.
#pragma once
#include "common.cuh"

namespace pto {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
// Arrival on a barrier of the partner CTA with the default (CTA-scope release) semantics: for signalling that data
// in THIS CTA's shared memory is ready for this CTA's half of a pair-wide tcgen05 operation.  The cluster-scope
// release below costs a few thousand cycles per arrival under load.
__device__ __forceinline__ void mbar_arrive_peer(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load of one box into THIS CTA's shared memory whose completion bytes go to a barrier of either CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y, uint32_t mbar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(mbar_cluster)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  const uint32_t z = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8, %9, %10, %11, %12}, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(z), "r"(z), "r"(z), "r"(z), "r"(z), "r"(z), "r"(z), "r"(z)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in BOTH CTAs once every MMA issued so far has completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(mask)
               : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// Order of the output tiles of a persistent GEMM: groups of `group` tile rows, and within a group column after
// column.  The CTAs (or pairs) work on neighbouring tile numbers at the same time, so what they read together is a
// block of about `group` tile rows by (CTAs / group) tile columns instead of one tile row by all CTAs' columns: each
// line of either operand is fetched by many CTAs close together in time and far fewer bytes come from DRAM.
__device__ __forceinline__ void grouped_tile_coords(int tile, int group, int row_tiles, int col_tiles, int& rt, int& ct) {
  const int per_group = group * col_tiles;
  const int g = tile / per_group, r = tile - g * per_group;
  const int rows = min(group, row_tiles - g * group);
  ct = r / rows;
  rt = g * group + (r - ct * rows);
}

}  // namespace pto
