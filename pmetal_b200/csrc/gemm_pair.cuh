// Device helpers for kernels that run as CTA pairs (tcgen05 cta_group::2): cluster identity, remote barrier
// signalling, pair-wide TMEM allocation, MMA issue and commit.
#pragma once
#include "gemm_common.cuh"

namespace pm {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t num_clusters_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local_addr` (a shared::cta address) in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load into this CTA's shared memory; completion bytes are counted on `bar_cluster_addr`,
// which may be a barrier of the partner CTA. No multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
      "[%2];" ::"r"(dst_smem),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_local(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar_addr, int c0,
                                                  int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          dst_smem),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_addr), "r"(c0), "r"(c1)
      : "memory");
}
template <bool kLocal>
__device__ __forceinline__ void load_operand_pair_t(uint32_t dst, const CUtensorMap* map, uint32_t bar, int mn_major,
                                                    int rows, int row0, int k0) {
  if (!mn_major) {
    if (kLocal) tma_load_2d_local(dst, map, bar, k0, row0); else tma_load_2d_pair(dst, map, bar, k0, row0);
  } else {
    for (int j = 0; j < rows / 64; ++j) {
      if (kLocal) tma_load_2d_local(dst + j * 8192, map, bar, row0 + 64 * j, k0);
      else tma_load_2d_pair(dst + j * 8192, map, bar, row0 + 64 * j, k0);
    }
  }
}
__device__ __forceinline__ void load_operand_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int mn_major,
                                                  int rows, int row0, int k0, int local) {
  if (local) load_operand_pair_t<true>(dst, map, bar, mn_major, rows, row0, k0);
  else load_operand_pair_t<false>(dst, map, bar, mn_major, rows, row0, k0);
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded wait on a barrier that the partner CTA arrives on
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                  int* g_status, int code) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  unsigned long long t0 = 0;     // the global timer is read only after many failed polls (see mbar_wait)
  uint32_t spins = 0;
  while (!mbar_try_wait_cluster(bar, parity)) {
    if ((++spins & 255u) == 0u && spins >= 2048u) {
      if (*abort_flag) return false;
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        if (g_status) atomicCAS(g_status, 0, code);
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on a barrier (given by its shared::cluster address) when all MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}
// One commit that arrives on the barrier at the same shared-memory offset in both CTAs of the pair
// (a barrier signal, not a data copy).
__device__ __forceinline__ void umma_commit_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(mask)
      : "memory");
}
// kind::f16, bf16 x bf16 -> fp32, M = 256 across the pair
__device__ __forceinline__ uint32_t make_idesc_bf16_m256(uint32_t n, uint32_t a_mn, uint32_t b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (a_mn << 15) | (b_mn << 16) | ((n >> 3) << 17) | ((256u >> 4) << 24);
}

constexpr int kPairBN = 256;        // tile width across the pair
constexpr int kHalfBN = 128;        // B rows staged per CTA
constexpr int kPairStageBytes = kBM * kBK * 2 + kHalfBN * kBK * 2;   // 32 KB per CTA per stage

}  // namespace pm
