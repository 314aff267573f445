// Persistent bf16 GEMM on 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM),
// operands staged by TMA through a multi-stage mbarrier pipeline.
//
//   D[M,N] = alpha * ( A[M,K] * B[N,K]^T  +  A2[M,K2] * B2[N,K2]^T )  (+ R[M,N])
//
// The second product is the low-rank LoRA term folded into the same accumulator as extra
// K-blocks, so y = x W^T + (s x A^T) B^T costs one pass over the output
// (cf. the reference's fused_lora_forward, crates/pmetal-metal/src/kernels/metal/fused_lora.metal:128).
// Each operand can be K-major or MN-major in global memory (the transposed products
// dA = dT^T x and dB = dY^T T of the LoRA backward read token-major tensors directly).
//
// Roles inside a 192-thread CTA: warp 0 = TMA producer, warp 1 = MMA issuer and TMEM
// owner, warps 2..5 = epilogue (TMEM -> registers -> global). Two accumulator buffers
// in TMEM let the epilogue of tile i overlap the MMAs of tile i+1.
#include "gemm_common.cuh"
#include "pmetal_b200.h"

namespace pm {

__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_b2,
                         const GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // carve: [stages][A 16 KB][B bn*128 B] | barriers
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int a_bytes = kBM * kBK * 2;
  const int b_bytes = p.bn * kBK * 2;
  const int stage_bytes = a_bytes + b_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + p.stages * stage_bytes);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* tfull_bar = empty_bar + kMaxStages;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;           // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < p.stages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 4);
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
    tmem_alloc(tmem_slot, p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int m_tiles = (p.M + kBM - 1) / kBM;
  const int n_tiles = (p.N + p.bn - 1) / p.bn;
  const int total = m_tiles * n_tiles * p.splits;
  const int nk = p.nk1 + p.nk2;
  const int per_split = (nk + p.splits - 1) / p.splits;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
        const int split = w % p.splits, tile = w / p.splits;
        const int nb = tile % n_tiles, mb = tile / n_tiles;
        const int kb0 = split * per_split, kb1 = min(nk, kb0 + per_split);
        const int m0 = mb * kBM, n0 = nb * p.bn;
        int a2_off = 0, b_off = 0;
        if (p.seg_mode == 1) a2_off = seg_of(p, n0) * p.seg_r;
        if (p.seg_mode == 2) b_off = seg_of(p, m0) * p.seg_r;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % p.stages;
          const uint32_t ph = (it / p.stages) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, kTimeoutProducer)) { ok = false; break; }
          uint8_t* sa = smem + s * stage_bytes;
          uint8_t* sb = sa + a_bytes;
          mbar_expect_tx(&full_bar[s], a_bytes + b_bytes);
          if (kb < p.nk1) {
            load_operand(sa, &map_a, &full_bar[s], p.a_mn, kBM, m0, kb * kBK);
            // seg_mode 3: B is [K, seg_r] (MN-major, one narrow block of columns shared by every segment of K); the
            // tile is fetched seg * seg_r columns to the left of its origin, so the rows of segment `seg` land in
            // output columns [seg * seg_r, (seg + 1) * seg_r) and everything else reads as zero (out-of-range fill)
            const int b_k_off = (p.seg_mode == 3) ? -seg_of(p, kb * kBK) * p.seg_r : 0;
            load_operand(sb, &map_b, &full_bar[s], p.b_mn, p.bn, n0 + b_off + b_k_off, kb * kBK);
          } else {
            const int k0 = (kb - p.nk1) * kBK;
            load_operand(sa, &map_a2, &full_bar[s], p.a2_mn, kBM, m0, k0 + a2_off);
            load_operand(sb, &map_b2, &full_bar[s], p.b2_mn, p.bn, n0, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
        const int split = w % p.splits;
        const int kb0 = split * per_split, kb1 = min(nk, kb0 + per_split);
        if (kb0 >= kb1) continue;
        const int buf = acc_it & 1;
        const uint32_t aph = (acc_it >> 1) & 1;
        if (!mbar_wait(&tempty_bar[buf], aph ^ 1, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * p.bn;
        uint32_t accumulate = 0;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % p.stages;
          const uint32_t ph = (it / p.stages) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * stage_bytes);
          const uint32_t sb = sa + a_bytes;
          int amn, bmn, nmma;
          if (kb < p.nk1) {
            amn = p.a_mn; bmn = p.b_mn; nmma = 4;
          } else {
            amn = p.a2_mn; bmn = p.b2_mn;
            const int rem = p.K2 - (kb - p.nk1) * kBK;
            nmma = min(4, (rem + 15) / 16);
          }
          const uint32_t idesc = make_idesc_bf16(p.bn, amn, bmn);
          const uint64_t da = make_smem_desc(sa, amn ? 8192u : 16u, 1024u);
          const uint64_t db = make_smem_desc(sb, bmn ? 8192u : 16u, 1024u);
          const uint32_t astep = amn ? 128u : 2u;   // 16 K elements: 2048 B (MN-major) or 32 B (K-major), >> 4
          const uint32_t bstep = bmn ? 128u : 2u;
          for (int j = 0; j < nmma; ++j) {
            umma_f16(d_tmem, da + static_cast<uint64_t>(astep * j), db + static_cast<uint64_t>(bstep * j), idesc,
                     accumulate);
            accumulate = 1;
          }
          umma_commit(&empty_bar[s]);   // frees the stage once these MMAs have read it
        }
        if (ok) umma_commit(&tfull_bar[buf]);
        ++acc_it;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;   // TMEM lane quarter this warp may access
    uint32_t acc_it = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
      const int split = w % p.splits, tile = w / p.splits;
      const int kb0 = split * per_split, kb1 = min(nk, kb0 + per_split);
      if (kb0 >= kb1) continue;
      const int nb = tile % n_tiles, mb = tile / n_tiles;
      const int buf = acc_it & 1;
      const uint32_t aph = (acc_it >> 1) & 1;
      if (!mbar_wait(&tfull_bar[buf], aph, abort_flag, p.status, kTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after();
      const int row = mb * kBM + q * 32 + lane;
      const bool row_ok = row < p.M;
      if (p.out_mode == 6) {
        // park this split's partial rows, then count the arrival of this warp's quarter of the tile; the warp that
        // completes the count owns the reduction of that quarter
        float* mine = p.ws + ((static_cast<size_t>(tile) * p.splits + split) * kBM + q * 32 + lane) * p.bn;
        for (int c = 0; c < p.bn / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + buf * p.bn + c * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
          tmem_ld_wait();
          if (row_ok && nb * p.bn + c * 32 < p.n_store) {
#pragma unroll
            for (int v = 0; v < 8; ++v)
              __stcg(reinterpret_cast<float4*>(mine + c * 32) + v,
                     make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]), __uint_as_float(r[4 * v + 2]),
                                 __uint_as_float(r[4 * v + 3])));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[buf]);
        ++acc_it;
        __threadfence();
        __syncwarp();
        unsigned seen = 0;
        if (lane == 0) seen = atomicAdd(p.ws_cnt + tile * 4 + q, 1u);
        seen = __shfl_sync(0xffffffffu, seen, 0);
        if (seen != static_cast<unsigned>(p.splits - 1)) continue;
        __threadfence();
        if (row_ok) {
          const float* base = p.ws + (static_cast<size_t>(tile) * p.splits * kBM + q * 32 + lane) * p.bn;
          for (int c = 0; c < p.bn / 32; ++c) {
            const int col0 = nb * p.bn + c * 32;
            if (col0 >= p.n_store) break;
            float acc[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) acc[e] = 0.f;
            for (int s2 = 0; s2 < p.splits; ++s2) {        // fixed order: the result does not depend on who came last
              const float4* src = reinterpret_cast<const float4*>(base + static_cast<size_t>(s2) * kBM * p.bn + c * 32);
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                const float4 x = __ldcg(src + v);
                acc[4 * v] += x.x; acc[4 * v + 1] += x.y; acc[4 * v + 2] += x.z; acc[4 * v + 3] += x.w;
              }
            }
            uint32_t r[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(acc[e]);
            epilogue_store_chunk(p, r, row, col0);
          }
        }
        __syncwarp();
        if (lane == 0) p.ws_cnt[tile * 4 + q] = 0u;       // ready for the next launch on this stream
        continue;
      }
      for (int c = 0; c < p.bn / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + buf * p.bn + c * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
        tmem_ld_wait();
        const int col0 = nb * p.bn + c * 32;
        if (!row_ok || col0 >= p.n_store) continue;
        epilogue_store_chunk(p, r, row, col0);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      ++acc_it;
    }
  }

  // ------------------------------------------------------------------ tail: release TMEM
  __syncwarp();
  if (*abort_flag) {
    // give TMA copies still in flight time to land before the CTA's shared memory is released
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

}  // namespace pm

using namespace pm;

// Returns 0 on success, negative on argument / descriptor errors, or the CUDA error code.
//   a_rows/b_rows: extent of the operand along M / N as seen by the tensor map (rows beyond it read as zero).
extern "C" int pm_gemm_bf16(const void* A, int a_mn, int lda, int a_rows, const void* B, int b_mn, int ldb, int b_rows,
                            const void* A2, int a2_mn, int lda2, int a2_k, const void* B2, int b2_mn, int ldb2,
                            int b2_rows, void* D, int out_mode, int ldd, const void* R, int ldr, int M, int N, int K,
                            int K2, int n_store, float alpha, int bn, int splits, int seg_mode, const int* seg_end,
                            int seg_r, int max_ctas, float* ws, long long ws_floats, unsigned* ws_cnt,
                            long long ws_cnt_len, int* status, cudaStream_t stream) {
  if (bn != 32 && bn != 64 && bn != 128 && bn != 256) return -10;
  if ((b_mn || (K2 > 0 && b2_mn)) && (bn % 64)) return -11;
  // split-K needs the atomic modes, or mode 6 with its workspace (every split must own at least one K block)
  if (splits < 1 || (splits > 1 && out_mode != 2 && out_mode != 3 && out_mode != 6)) return -12;
  if (out_mode == 6) {
    const long long tiles = static_cast<long long>((M + kBM - 1) / kBM) * ((N + bn - 1) / bn);
    const int nk_all = (K + kBK - 1) / kBK + (K2 > 0 ? (K2 + kBK - 1) / kBK : 0);
    const int per = (nk_all + splits - 1) / splits;
    if (!ws || !ws_cnt || tiles * splits * kBM * bn > ws_floats || tiles * 4 > ws_cnt_len) return -17;
    if (static_cast<long long>(splits - 1) * per >= nk_all) return -18;
  }
  if (M <= 0 || N <= 0 || K <= 0) return -13;
  if ((out_mode == 0 || out_mode == 6) && ((ldd % 8) || (reinterpret_cast<uintptr_t>(D) & 15))) return -14;
  if (R && ((ldr % 8) || (reinterpret_cast<uintptr_t>(R) & 15))) return -15;
  // seg_mode 3 shifts a TMA load by seg * seg_r elements: the shift must keep the 16-byte alignment of the copy
  if (seg_mode == 3 && (!b_mn || (seg_r % 8) || N > bn || splits != 1)) return -16;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.K2 = K2; p.bn = bn;
  p.a_mn = a_mn; p.b_mn = b_mn; p.a2_mn = a2_mn; p.b2_mn = b2_mn;
  p.nk1 = (K + kBK - 1) / kBK;
  p.nk2 = K2 > 0 ? (K2 + kBK - 1) / kBK : 0;
  p.splits = splits;
  p.out_mode = out_mode; p.ldd = ldd; p.ldr = ldr; p.n_store = n_store > 0 ? n_store : N;
  p.alpha = alpha; p.D = D; p.R = R;
  p.seg_mode = seg_mode; p.seg_r = seg_r;
  for (int i = 0; i < 4; ++i) p.seg_end[i] = (seg_mode && seg_end) ? seg_end[i] : 0x7fffffff;
  p.status = status;
  p.ws = ws; p.ws_cnt = ws_cnt;
  const int stage_bytes = kBM * kBK * 2 + bn * kBK * 2;
  int stages = (227 * 1024 - 2048) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  int cols = 32;
  while (cols < 2 * bn) cols *= 2;
  p.tmem_cols = cols;
  // Narrow tiles stream one big operand and do little arithmetic: two CTAs per SM (half the ring each) keep two
  // independent TMA pipelines busy per SM. PMETAL_GEMM_OCC=1 switches it off; PMETAL_GEMM_STAGES caps the ring depth.
  static int env_occ = -1, env_stages = -1;
  if (env_occ < 0) {
    const char* e = getenv("PMETAL_GEMM_OCC");
    env_occ = e ? atoi(e) : 2;
    const char* s2 = getenv("PMETAL_GEMM_STAGES");
    env_stages = s2 ? atoi(s2) : 0;
  }
  int occ = 1;
  if (env_occ >= 2 && bn <= 64 && cols <= 256) {
    occ = 2;
    const int half = (113 * 1024 - 2048) / stage_bytes;
    if (stages > half) stages = half;
  }
  if (env_stages > 0 && stages > env_stages) stages = env_stages;
  if (stages < 2) return -19;
  p.stages = stages;

  CUtensorMap ma, mb, ma2, mb2;
  int rc;
  if ((rc = operand_map(&ma, A, a_mn, a_rows, K, lda, kBM))) return rc * 10 - 1;
  if ((rc = operand_map(&mb, B, b_mn, b_rows, K, ldb, bn))) return rc * 10 - 2;
  if (K2 > 0) {
    if ((rc = operand_map(&ma2, A2, a2_mn, a_rows, a2_k, lda2, kBM))) return rc * 10 - 3;
    if ((rc = operand_map(&mb2, B2, b2_mn, b2_rows, K2, ldb2, bn))) return rc * 10 - 4;
  } else {
    ma2 = ma; mb2 = mb;
  }
  const size_t smem = static_cast<size_t>(stages) * stage_bytes + 1024 /*align*/ + 256 /*barriers*/;
  static DeviceOnce configured;
  if (configured.pending()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(227 * 1024));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured.mark();
  }
  const int m_tiles = (M + kBM - 1) / kBM, n_tiles = (N + bn - 1) / bn;
  int grid = m_tiles * n_tiles * splits;
  int cap = max_ctas > 0 ? max_ctas : num_sms() * occ;
  if (grid > cap) grid = cap;
  gemm_bf16_tcgen05_kernel<<<grid, kThreads, smem, stream>>>(ma, mb, ma2, mb2, p);
  return static_cast<int>(cudaGetLastError());
}
