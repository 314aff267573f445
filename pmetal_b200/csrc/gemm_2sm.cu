// bf16 GEMM on CTA pairs: tcgen05.mma.cta_group::2 computes a 256 x 256 output tile across two SMs.
//
// Same math and operand options as gemm_tcgen05.cu:
//   D[M,N] = alpha * ( A[M,K] * B[N,K]^T + A2[M,K2] * B2[N,K2]^T ) (+ R[M,N])
// but launched as clusters of two CTAs. CTA r of a pair stages A rows [m0+128r, +128) and B rows
// [n0+128r, +128) of each 64-wide K block in its own shared memory; one thread of the leader CTA
// (cluster rank 0) issues the MMAs, which read both CTAs' shared memory and write 128 x 256 fp32
// accumulators into each CTA's TMEM. Per SM this moves 32 KB of operands per K block instead of the
// 48 KB a single CTA needs for 128 x 256, which is what lifts the kernel off the L2->SM bandwidth limit.
// No operand is multicast: every CTA fetches its own half with plain tiled TMA loads whose completion
// is counted on the leader's "full" barrier.
//
// Cross-CTA signalling:
//   full[s]   (leader)      <- TMA bytes of both CTAs + the leader producer's expect_tx arrive
//   empty[s]  (each CTA)    <- tcgen05.commit from the leader, once to its own and once to the peer's barrier
//   tfull[b]  (each CTA)    <- tcgen05.commit from the leader after the last K block (own + peer)
//   tempty[b] (leader)      <- 4 epilogue warps of each CTA (remote mbarrier.arrive from the peer)
// All waits are bounded (see common.cuh); the pair leaves through a cluster barrier so neither CTA
// exits while its partner can still touch its shared memory.
#include "gemm_pair.cuh"
#include "pmetal_b200.h"

namespace pm {

__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_2sm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_b2,
                     const GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int a_bytes = kBM * kBK * 2;
  const int kps = p.kps;                                   // K blocks (of 64) held by one pipeline stage
  const int stage_bytes = kps * kPairStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + p.stages * stage_bytes);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* tfull_bar = empty_bar + kMaxStages;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;           // [2]
  uint64_t* pfull_bar = tempty_bar + 2;           // [kMaxStages] leader only: "the partner's half has landed"
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pfull_bar + kMaxStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();        // 0 = leader
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < p.stages; ++i) {
      mbar_init(&full_bar[i], 1);     // leader producer's expect_tx arrive; bytes from both CTAs
      mbar_init(&empty_bar[i], 1);    // one tcgen05.commit
      mbar_init(&pfull_bar[i], 1);    // one remote arrive from the partner's forwarder
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);    // one tcgen05.commit
      mbar_init(&tempty_bar[i], 8);   // 4 epilogue warps of each CTA (used on the leader only)
    }
    *abort_flag = 0;
    mbar_init_fence();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    if (p.nk2) {
      tma_prefetch_desc(&map_a2);
      tma_prefetch_desc(&map_b2);
    }
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers are initialised before any remote signal
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int m_tiles = (p.M + 2 * kBM - 1) / (2 * kBM);
  const int n_tiles = (p.N + kPairBN - 1) / kPairBN;
  const int total = m_tiles * n_tiles * p.splits;
  const int nk = p.nk1 + p.nk2;
  const int per_split = (nk + p.splits - 1) / p.splits;
  const int first = static_cast<int>(cluster_id_x());
  const int stride = static_cast<int>(num_clusters_x());

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (one per CTA)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int w = first; w < total && ok; w += stride) {
        const int split = w % p.splits, tile = w / p.splits;
        const int nb = tile % n_tiles, mb = tile / n_tiles;
        const int kb0 = split * per_split, kb1 = min(nk, kb0 + per_split);
        const int m0 = mb * 2 * kBM + static_cast<int>(rank) * kBM;
        const int n_tile0 = nb * kPairBN;
        const int n0 = n_tile0 + static_cast<int>(rank) * kHalfBN;
        int a2_off = 0, b_off = 0;
        if (p.seg_mode == 1) a2_off = seg_of(p, n_tile0) * p.seg_r;
        if (p.seg_mode == 2) b_off = seg_of(p, mb * 2 * kBM) * p.seg_r;
        for (int kb = kb0; kb < kb1; kb += kps, ++it) {
          const int s = it % p.stages;
          const uint32_t ph = (it / p.stages) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, kTimeoutProducer)) { ok = false; break; }
          const int nsub = min(kps, kb1 - kb);
          uint32_t fb;
          if (p.fwd_full) {   // every CTA counts its own bytes on its own barrier
            fb = smem_u32(&full_bar[s]);
            mbar_expect_tx(&full_bar[s], nsub * kPairStageBytes);
          } else {            // both CTAs' bytes are counted on the leader's barrier
            fb = map_to_cta(smem_u32(&full_bar[s]), 0);
            if (leader) mbar_expect_tx(&full_bar[s], 2 * nsub * kPairStageBytes);
          }
          for (int j = 0; j < nsub; ++j) {
            const uint32_t sa = smem_u32(smem + s * stage_bytes + j * kPairStageBytes);
            const uint32_t sb = sa + a_bytes;
            const int kbj = kb + j;
            if (kbj < p.nk1) {
              load_operand_pair(sa, &map_a, fb, p.a_mn, kBM, m0, kbj * kBK, p.fwd_full);
              load_operand_pair(sb, &map_b, fb, p.b_mn, kHalfBN, n0 + b_off, kbj * kBK, p.fwd_full);
            } else {
              const int k0 = (kbj - p.nk1) * kBK;
              load_operand_pair(sa, &map_a2, fb, p.a2_mn, kBM, m0, k0 + a2_off, p.fwd_full);
              load_operand_pair(sb, &map_b2, fb, p.b2_mn, kHalfBN, n0, k0, p.fwd_full);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ partner CTA: forward "stage landed"
    if (lane == 0 && !leader && p.fwd_full) {
      uint32_t it = 0;
      bool ok = true;
      for (int w = first; w < total && ok; w += stride) {
        const int split = w % p.splits;
        const int kb0 = split * per_split, kb1 = min(nk, kb0 + per_split);
        for (int kb = kb0; kb < kb1; kb += kps, ++it) {
          const int s = it % p.stages;
          const uint32_t ph = (it / p.stages) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
          mbar_arrive_cluster(map_to_cta(smem_u32(&pfull_bar[s]), 0));
        }
      }
    }
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int w = first; w < total && ok; w += stride) {
        const int split = w % p.splits;
        const int kb0 = split * per_split, kb1 = min(nk, kb0 + per_split);
        if (kb0 >= kb1) continue;
        const int buf = acc_it & 1;
        const uint32_t aph = (acc_it >> 1) & 1;
        if (!mbar_wait_cluster(&tempty_bar[buf], aph ^ 1, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * kPairBN;
        uint32_t accumulate = 0;
        for (int kb = kb0; kb < kb1; kb += kps, ++it) {
          const int s = it % p.stages;
          const uint32_t ph = (it / p.stages) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
          if (p.fwd_full && !mbar_wait_cluster(&pfull_bar[s], ph, abort_flag, p.status, kTimeoutMma)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const int nsub = min(kps, kb1 - kb);
          for (int js = 0; js < nsub; ++js) {
            const uint32_t sa = smem_u32(smem + s * stage_bytes + js * kPairStageBytes);
            const uint32_t sb = sa + a_bytes;
            const int kbj = kb + js;
            int amn, bmn, nmma;
            if (kbj < p.nk1) {
              amn = p.a_mn; bmn = p.b_mn; nmma = 4;
            } else {
              amn = p.a2_mn; bmn = p.b2_mn;
              const int rem = p.K2 - (kbj - p.nk1) * kBK;
              nmma = min(4, (rem + 15) / 16);
            }
            const uint32_t idesc = make_idesc_bf16_m256(kPairBN, amn, bmn);
            const uint64_t da = make_smem_desc(sa, amn ? 8192u : 16u, 1024u);
            const uint64_t db = make_smem_desc(sb, bmn ? 8192u : 16u, 1024u);
            const uint32_t astep = amn ? 128u : 2u;
            const uint32_t bstep = bmn ? 128u : 2u;
            for (int j = 0; j < nmma; ++j) {
              umma_f16_pair(d_tmem, da + static_cast<uint64_t>(astep * j), db + static_cast<uint64_t>(bstep * j),
                            idesc, accumulate);
              accumulate = 1;
            }
          }
          // the stage is free in both CTAs once these MMAs have read it
          if (p.commit_both) {
            umma_commit_both(&empty_bar[s]);
          } else {
            umma_commit_pair(map_to_cta(smem_u32(&empty_bar[s]), 0));
            umma_commit_pair(map_to_cta(smem_u32(&empty_bar[s]), 1));
          }
        }
        if (ok) {
          if (p.commit_both) {
            umma_commit_both(&tfull_bar[buf]);
          } else {
            umma_commit_pair(map_to_cta(smem_u32(&tfull_bar[buf]), 0));
            umma_commit_pair(map_to_cta(smem_u32(&tfull_bar[buf]), 1));
          }
        }
        ++acc_it;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5 of each CTA)
    const int q = warp & 3;
    uint32_t acc_it = 0;
    bool ok = true;
    for (int w = first; w < total && ok; w += stride) {
      const int split = w % p.splits, tile = w / p.splits;
      const int kb0 = split * per_split, kb1 = min(nk, kb0 + per_split);
      if (kb0 >= kb1) continue;
      const int nb = tile % n_tiles, mb = tile / n_tiles;
      const int buf = acc_it & 1;
      const uint32_t aph = (acc_it >> 1) & 1;
      if (!mbar_wait(&tfull_bar[buf], aph, abort_flag, p.status, kTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after();
      const int row = mb * 2 * kBM + static_cast<int>(rank) * kBM + q * 32 + lane;
      const bool row_ok = row < p.M;
      for (int c = 0; c < kPairBN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + buf * kPairBN + c * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
        tmem_ld_wait();
        const int col0 = nb * kPairBN + c * 32;
        if (!row_ok || col0 >= p.n_store) continue;
        epilogue_store_chunk(p, r, row, col0);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[buf]), 0));
      ++acc_it;
    }
  }

  // ------------------------------------------------------------------ tail
  __syncwarp();
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the partner is done with this CTA's shared memory, barriers and TMEM
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

}  // namespace pm

using namespace pm;

// Same contract as pm_gemm_bf16 with the tile fixed at 256 x 256 per CTA pair.
extern "C" int pm_gemm_bf16_2sm(const void* A, int a_mn, int lda, int a_rows, const void* B, int b_mn, int ldb,
                                int b_rows, const void* A2, int a2_mn, int lda2, int a2_k, const void* B2, int b2_mn,
                                int ldb2, int b2_rows, void* D, int out_mode, int ldd, const void* R, int ldr, int M,
                                int N, int K, int K2, int n_store, float alpha, int splits, int seg_mode,
                                const int* seg_end, int seg_r, int max_ctas, int* status,
                                cudaStream_t stream) {
  if (splits < 1 || (splits > 1 && (out_mode < 2 || out_mode > 3))) return -12;   // split-K needs the atomic modes
  if (M <= 0 || N <= 0 || K <= 0) return -13;
  if (out_mode == 0 && ((ldd % 8) || (reinterpret_cast<uintptr_t>(D) & 15))) return -14;
  if (R && ((ldr % 8) || (reinterpret_cast<uintptr_t>(R) & 15))) return -15;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.K2 = K2; p.bn = kPairBN;
  p.a_mn = a_mn; p.b_mn = b_mn; p.a2_mn = a2_mn; p.b2_mn = b2_mn;
  p.nk1 = (K + kBK - 1) / kBK;
  p.nk2 = K2 > 0 ? (K2 + kBK - 1) / kBK : 0;
  p.splits = splits;
  p.out_mode = out_mode; p.ldd = ldd; p.ldr = ldr; p.n_store = n_store > 0 ? n_store : N;
  p.alpha = alpha; p.D = D; p.R = R;
  p.seg_mode = seg_mode; p.seg_r = seg_r;
  for (int i = 0; i < 4; ++i) p.seg_end[i] = (seg_mode && seg_end) ? seg_end[i] : 0x7fffffff;
  p.status = status;
  p.kps = 2;
  p.commit_both = 0;
  p.fwd_full = 0;
  int stages = (227 * 1024 - 2048) / (p.kps * kPairStageBytes);
  if (stages > kMaxStages) stages = kMaxStages;
  p.stages = stages;
  p.tmem_cols = 512;

  CUtensorMap ma, mb, ma2, mb2;
  int rc;
  if ((rc = operand_map(&ma, A, a_mn, a_rows, K, lda, kBM))) return rc * 10 - 1;
  if ((rc = operand_map(&mb, B, b_mn, b_rows, K, ldb, kHalfBN))) return rc * 10 - 2;
  if (K2 > 0) {
    if ((rc = operand_map(&ma2, A2, a2_mn, a_rows, a2_k, lda2, kBM))) return rc * 10 - 3;
    if ((rc = operand_map(&mb2, B2, b2_mn, b2_rows, K2, ldb2, kHalfBN))) return rc * 10 - 4;
  } else {
    ma2 = ma; mb2 = mb;
  }
  const size_t smem = static_cast<size_t>(stages) * p.kps * kPairStageBytes + 1024 + 512;
  static DeviceOnce configured;
  if (configured.pending()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_2sm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured.mark();
  }
  const int m_tiles = (M + 2 * kBM - 1) / (2 * kBM), n_tiles = (N + kPairBN - 1) / kPairBN;
  int pairs = m_tiles * n_tiles * splits;
  int cap = (max_ctas > 0 ? max_ctas : num_sms()) / 2;
  if (pairs > cap) pairs = cap;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_bf16_2sm_kernel, ma, mb, ma2, mb2, p);
  return static_cast<int>(e);
}
