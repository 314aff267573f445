// Varlen causal flash attention backward on tcgen05 tensor cores (head_dim 128, GQA): dQ kernel and dK/dV kernel.
//
// Both kernels recompute P = exp2(S*scale*log2e - lse*log2e) from Q, K and the saved log-sum-exp, form
// dS = P * (dP - delta) * scale with dP = dO V^T and delta = rowsum(dO * O), and are deterministic
// (no atomics):
//   dQ kernel : one CTA per (128-query tile, head); loops over key tiles; dQ += dS K accumulates in TMEM.
//   dKV kernel: one CTA per (128-key tile, kv head); loops over the query heads of the GQA group and the
//               query tiles that can see these keys; works on the transposed tiles S^T = K Q^T and
//               dP^T = V dO^T so that a thread owns one key row; dV += P^T dO and dK += dS^T Q accumulate
//               in TMEM.
// A [128][128] bf16 tile in shared memory (two 128B-swizzled [128][64] boxes) is read by tcgen05.mma either
// as a K-major operand (its rows are the M/N index) or as an MN-major operand (its rows are the reduction
// index), which is how the same Q, dO, K tiles serve both products of each kernel without a transpose.
//
// Both kernels run 320 threads: warp 0 = TMA producer, warp 1 = MMA issuer, warps 2..5 and 6..9 = two compute groups.
// The element-wise work has no row reductions (log-sum-exp and delta are inputs), so the two groups split the 128 columns of every
// row: group g handles the 32-column chunks 2g and 2g+1 of S / dP and of the output tiles. A group reads its 64
// columns of S (and dP) with back-to-back tcgen05.ld instructions and one wait, and releases the TMEM buffer as soon
// as the values are in registers, so the tensor cores start on the next tile while this one is still being formed.
#include "attention_tc.cuh"
#include "pmetal_b200.h"

namespace pm {

enum {
  kDqBarQdO = 0, kDqBarKvFull = 1 /*2*/, kDqBarKvFree = 3 /*2*/, kDqBarSpFull = 5, kDqBarSpFree = 6, kDqBarDsReady = 7,
  kDqBarDsFree = 8, kDqBarDqFull = 9, kDqBarCount = 10
};

// dS for this group's 64 columns of one query row (dQ kernel): p = exp2(s*a + b); ds = p * (dp - delta) * scale, packed
// as bf16 into pk[32]. sv / dv hold the row's S and dP values (chunks c0 and c0 + 1).
template <bool kMask>
__device__ __forceinline__ void dq_ds_pack(const uint32_t (&sv)[64], const uint32_t (&dv)[64], float a, float b,
                                           float delta, float scale, int lo, int span, int c0, uint32_t (&pk)[32]) {
#pragma unroll
  for (int e = 0; e < 64; e += 2) {
    float d2[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      float pv = fast_exp2(fmaf(__uint_as_float(sv[e + u]), a, b));
      if (kMask) pv = (span >= 0 && static_cast<unsigned>(c0 * 32 + e + u - lo) <= static_cast<unsigned>(span)) ? pv : 0.f;
      d2[u] = pv * (__uint_as_float(dv[e + u]) - delta) * scale;
    }
    pk[e >> 1] = pack_bf16x2(d2[0], d2[1]);
  }
}

// two back-to-back 32-column TMEM loads into one 64-entry array (no wait)
__device__ __forceinline__ void tmem_ld_64(uint32_t taddr, uint32_t (&v)[64]) {
  tmem_ld_32x32b_x32(taddr, *reinterpret_cast<uint32_t (*)[32]>(&v[0]));
  tmem_ld_32x32b_x32(taddr + 32, *reinterpret_cast<uint32_t (*)[32]>(&v[32]));
}

// TMEM columns: [0,128) S   [128,256) dP   [256,384) dQ accumulator
__global__ void __launch_bounds__(kFaThreads2, 1)
attn_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                      const FaParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = smem + kFaTileBytes;
  uint8_t* sK = smem + 2 * kFaTileBytes;   // 2 buffers
  uint8_t* sV = smem + 4 * kFaTileBytes;   // 2 buffers
  uint8_t* sdS = smem + 6 * kFaTileBytes;
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + 7 * kFaTileBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + kDqBarCount);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y;
  const int hk = h / (p.hq / p.hkv);
  const int q0 = qt * kFaTile;

  if (threadIdx.x == 0) {
    mbar_init(&bar[kDqBarQdO], 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar[kDqBarKvFull + i], 1);
      mbar_init(&bar[kDqBarKvFree + i], 1);
    }
    mbar_init(&bar[kDqBarSpFull], 1);
    mbar_init(&bar[kDqBarSpFree], 8);
    mbar_init(&bar[kDqBarDsReady], 8);
    mbar_init(&bar[kDqBarDsFree], 1);
    mbar_init(&bar[kDqBarDqFull], 1);
    *abort_flag = 0;
    mbar_init_fence();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
    tma_prefetch_desc(&map_do);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int kv_lo = (p.seq_start[q0] / kFaTile) * kFaTile;
  const int kv_hi = min(q0 + kFaTile, p.T);
  const int n_tiles = (kv_hi - kv_lo + kFaTile - 1) / kFaTile;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&bar[kDqBarQdO], 2 * kFaTileBytes);
      tma_load_2d(sQ, &map_q, &bar[kDqBarQdO], h * 128, q0);
      tma_load_2d(sQ + kFaBox, &map_q, &bar[kDqBarQdO], h * 128 + 64, q0);
      tma_load_2d(sdO, &map_do, &bar[kDqBarQdO], h * 128, q0);
      tma_load_2d(sdO + kFaBox, &map_do, &bar[kDqBarQdO], h * 128 + 64, q0);
      for (int j = 0; j < n_tiles; ++j) {
        const int b = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&bar[kDqBarKvFree + b], ph ^ 1, abort_flag, p.status, kTimeoutProducer)) break;
        const int j0 = kv_lo + j * kFaTile;
        mbar_expect_tx(&bar[kDqBarKvFull + b], 2 * kFaTileBytes);
        tma_load_2d(sK + b * kFaTileBytes, &map_k, &bar[kDqBarKvFull + b], hk * 128, j0);
        tma_load_2d(sK + b * kFaTileBytes + kFaBox, &map_k, &bar[kDqBarKvFull + b], hk * 128 + 64, j0);
        tma_load_2d(sV + b * kFaTileBytes, &map_v, &bar[kDqBarKvFull + b], hk * 128, j0);
        tma_load_2d(sV + b * kFaTileBytes + kFaBox, &map_v, &bar[kDqBarKvFull + b], hk * 128 + 64, j0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t id_kk = make_idesc_bf16(128, 0, 0);
      const uint32_t id_kmn = make_idesc_bf16(128, 0, 1);
      const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sdO), ds_addr = smem_u32(sdS);
      bool ok = mbar_wait(&bar[kDqBarQdO], 0, abort_flag, p.status, kTimeoutMma);
      auto issue_s_dp = [&](int j) -> bool {
        const int b = j & 1;
        if (!mbar_wait(&bar[kDqBarKvFull + b], (j >> 1) & 1, abort_flag, p.status, kTimeoutMma)) return false;
        if (!mbar_wait(&bar[kDqBarSpFree], (j & 1) ^ 1, abort_flag, p.status, kTimeoutMma)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + b * kFaTileBytes), v_addr = smem_u32(sV + b * kFaTileBytes);
#pragma unroll
        for (int s = 0; s < 8; ++s)
          umma_f16(tmem_base, desc_kmajor(q_addr, s), desc_kmajor(k_addr, s), id_kk, s > 0);
#pragma unroll
        for (int s = 0; s < 8; ++s)
          umma_f16(tmem_base + 128, desc_kmajor(do_addr, s), desc_kmajor(v_addr, s), id_kk, s > 0);
        umma_commit(&bar[kDqBarSpFull]);
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_s_dp(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int b = j & 1;
        if (j + 1 < n_tiles) ok = issue_s_dp(j + 1);
        if (!ok) break;
        if (!mbar_wait(&bar[kDqBarDsReady], j & 1, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + b * kFaTileBytes);
#pragma unroll
        for (int s = 0; s < 8; ++s)   // dQ += dS[q][keys] * K[keys][d]: K tile read as an MN-major operand
          umma_f16(tmem_base + 256, desc_kmajor(ds_addr, s), desc_mnmajor(k_addr, s), id_kmn, (j > 0) || (s > 0));
        umma_commit(&bar[kDqBarDsFree]);
        umma_commit(&bar[kDqBarKvFree + b]);
      }
      if (ok) umma_commit(&bar[kDqBarDqFull]);
    }
  } else {
    const int qd = warp & 3;
    const int c0 = (warp >= 6) ? 2 : 0;        // first of the two 32-column chunks this warp group owns
    const int r = qd * 32 + lane;
    const int i = q0 + r;
    const int ic = min(i, p.T - 1);
    const int st = p.seq_start[ic];
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const float sl2 = p.scale * kFaLog2e;
    const float lse2 = p.lse[static_cast<long long>(h) * p.T + ic] * kFaLog2e;
    const float dl = p.delta[static_cast<long long>(h) * p.T + ic];
    const int st_max = p.seq_start[min(q0 + kFaTile - 1, p.T - 1)];
    const uint32_t ds_addr = smem_u32(sdS);
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int j0 = kv_lo + j * kFaTile;
      if (!mbar_wait(&bar[kDqBarSpFull], j & 1, abort_flag, p.status, kTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after();
      uint32_t pk[32];
      {
        uint32_t sv[64], dv[64];
        tmem_ld_64(tmem_base + lane_off + c0 * 32, sv);
        tmem_ld_64(tmem_base + lane_off + 128 + c0 * 32, dv);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar[kDqBarSpFree]);    // S and dP are in registers: the next pair of MMAs may start
        const int lo = max(st - j0, 0);
        const int span = (i < p.T) ? (min(i - j0, kFaTile - 1) - lo) : -1;
        const bool need_mask = (j0 + kFaTile - 1 > q0) || (j0 < st_max) || (q0 + kFaTile > p.T);
        if (need_mask) dq_ds_pack<true>(sv, dv, sl2, -lse2, dl, p.scale, lo, span, c0, pk);
        else dq_ds_pack<false>(sv, dv, sl2, -lse2, dl, p.scale, 0, 0, c0, pk);
      }
      // the previous tile's dS must have been consumed by its MMA before it is overwritten
      if (j > 0 && !mbar_wait(&bar[kDqBarDsFree], (j - 1) & 1, abort_flag, p.status, kTimeoutEpilogue)) {
        ok = false;
        break;
      }
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t ck[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) ck[e] = pk[cc * 16 + e];
        store_row_chunk_sw128(ds_addr, r, c0 + cc, ck);
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[kDqBarDsReady]);
    }
    if (ok && n_tiles > 0 && mbar_wait(&bar[kDqBarDqFull], 0, abort_flag, p.status, kTimeoutEpilogue)) {
      tc_fence_after();
      __nv_bfloat16* drow = p.out + static_cast<long long>(ic) * p.o_stride + static_cast<long long>(h) * 128;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = c0 + cc;
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_base + 256 + c * 32 + lane_off, v);
        tmem_ld_wait();
        if (i < p.T) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[g * 8]), __uint_as_float(v[g * 8 + 1]));
            o.y = pack_bf16x2(__uint_as_float(v[g * 8 + 2]), __uint_as_float(v[g * 8 + 3]));
            o.z = pack_bf16x2(__uint_as_float(v[g * 8 + 4]), __uint_as_float(v[g * 8 + 5]));
            o.w = pack_bf16x2(__uint_as_float(v[g * 8 + 6]), __uint_as_float(v[g * 8 + 7]));
            *reinterpret_cast<uint4*>(drow + c * 32 + g * 8) = o;
          }
        }
      }
    }
  }

  __syncwarp();
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}


enum {
  kKvBarKv = 0, kKvBarQdoFull = 1 /*2*/, kKvBarQdoFree = 3 /*2*/, kKvBarSFull = 5, kKvBarSFree = 6, kKvBarDpFull = 7,
  kKvBarDpFree = 8, kKvBarPReady = 9, kKvBarPFree = 10, kKvBarDsReady = 11, kKvBarDsFree = 12, kKvBarAccFull = 13,
  kKvBarCount = 14
};

// P for this group's 64 columns of one query row (dK/dV kernel): p = exp2(s*a + b) (masked), packed bf16 into pk[32].
template <bool kMask>
__device__ __forceinline__ void kv_p_row(uint32_t taddr, float a, float b, int lo, int span, int c0, uint32_t (&pk)[32]) {
  uint32_t sv[64];
  tmem_ld_64(taddr + c0 * 32, sv);
  tmem_ld_wait();
#pragma unroll
  for (int e = 0; e < 64; e += 2) {
    float p2[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      float pv = fast_exp2(fmaf(__uint_as_float(sv[e + u]), a, b));
      if (kMask) pv = (span >= 0 && static_cast<unsigned>(c0 * 32 + e + u - lo) <= static_cast<unsigned>(span)) ? pv : 0.f;
      p2[u] = pv;
    }
    pk[e >> 1] = pack_bf16x2(p2[0], p2[1]);
  }
}

// One CTA per (key tile, kv head). For every query tile that can see the key tile, and every query head of the
// group: S = Q K^T and dP = dO V^T (rows = queries, as in the dQ kernel), P and dS are formed per query row, and
// the same [query][key] smem tile is then read as an MN-major A operand: dV += P^T dO, dK += dS^T Q.
// S and dP have separate full/free barriers so that S of the next pair is computed while dS of this one is formed.
// TMEM columns: [0,128) S   [128,256) dP   [256,384) dV accumulator   [384,512) dK accumulator
__global__ void __launch_bounds__(kFaThreads2, 1)
attn_bwd_dkv_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                       const FaParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + kFaTileBytes;
  uint8_t* sQ = smem + 2 * kFaTileBytes;    // 2 buffers
  uint8_t* sdO = smem + 4 * kFaTileBytes;   // 2 buffers
  uint8_t* sX = smem + 6 * kFaTileBytes;    // P[query][key], then dS[query][key]
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + 7 * kFaTileBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + kKvBarCount);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jt = blockIdx.x, hk = blockIdx.y;
  const int rep = p.hq / p.hkv;
  const int j0 = jt * kFaTile;
  const int j_last = min(j0 + kFaTile, p.T) - 1;

  if (threadIdx.x == 0) {
    mbar_init(&bar[kKvBarKv], 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar[kKvBarQdoFull + i], 1);
      mbar_init(&bar[kKvBarQdoFree + i], 1);
    }
    mbar_init(&bar[kKvBarSFull], 1);
    mbar_init(&bar[kKvBarSFree], 8);
    mbar_init(&bar[kKvBarDpFull], 1);
    mbar_init(&bar[kKvBarDpFree], 8);
    mbar_init(&bar[kKvBarPReady], 8);
    mbar_init(&bar[kKvBarPFree], 1);
    mbar_init(&bar[kKvBarDsReady], 8);
    mbar_init(&bar[kKvBarDsFree], 1);
    mbar_init(&bar[kKvBarAccFull], 1);
    *abort_flag = 0;
    mbar_init_fence();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
    tma_prefetch_desc(&map_do);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // query tiles m0 = j0, j0+128, ... while the tile's first row belongs to a document that began at or
  // before the last key of this tile
  int n_q_tiles = 0;
  for (bool done = false; !done;) {
    const int m0 = j0 + (n_q_tiles + lane) * kFaTile;
    bool okt = m0 < p.T;
    if (okt) okt = p.seq_start[m0] <= j_last;
    const unsigned bm = __ballot_sync(0xffffffffu, okt);
    const int cnt = (bm == 0xffffffffu) ? 32 : (__ffs(~bm) - 1);
    n_q_tiles += cnt;
    done = cnt < 32;
  }
  const int total = n_q_tiles * rep;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&bar[kKvBarKv], 2 * kFaTileBytes);
      tma_load_2d(sK, &map_k, &bar[kKvBarKv], hk * 128, j0);
      tma_load_2d(sK + kFaBox, &map_k, &bar[kKvBarKv], hk * 128 + 64, j0);
      tma_load_2d(sV, &map_v, &bar[kKvBarKv], hk * 128, j0);
      tma_load_2d(sV + kFaBox, &map_v, &bar[kKvBarKv], hk * 128 + 64, j0);
      for (int w = 0; w < total; ++w) {
        const int b = w & 1;
        if (!mbar_wait(&bar[kKvBarQdoFree + b], ((w >> 1) & 1) ^ 1, abort_flag, p.status, kTimeoutProducer)) break;
        const int hh = hk * rep + w / n_q_tiles;
        const int m0 = j0 + (w % n_q_tiles) * kFaTile;
        mbar_expect_tx(&bar[kKvBarQdoFull + b], 2 * kFaTileBytes);
        tma_load_2d(sQ + b * kFaTileBytes, &map_q, &bar[kKvBarQdoFull + b], hh * 128, m0);
        tma_load_2d(sQ + b * kFaTileBytes + kFaBox, &map_q, &bar[kKvBarQdoFull + b], hh * 128 + 64, m0);
        tma_load_2d(sdO + b * kFaTileBytes, &map_do, &bar[kKvBarQdoFull + b], hh * 128, m0);
        tma_load_2d(sdO + b * kFaTileBytes + kFaBox, &map_do, &bar[kKvBarQdoFull + b], hh * 128 + 64, m0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t id_kk = make_idesc_bf16(128, 0, 0);
      const uint32_t id_mm = make_idesc_bf16(128, 1, 1);
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), x_addr = smem_u32(sX);
      bool ok = mbar_wait(&bar[kKvBarKv], 0, abort_flag, p.status, kTimeoutMma);
      auto issue_s = [&](int w) -> bool {
        const int b = w & 1;
        if (!mbar_wait(&bar[kKvBarQdoFull + b], (w >> 1) & 1, abort_flag, p.status, kTimeoutMma)) return false;
        if (!mbar_wait(&bar[kKvBarSFree], (w & 1) ^ 1, abort_flag, p.status, kTimeoutMma)) return false;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQ + b * kFaTileBytes);
#pragma unroll
        for (int s = 0; s < 8; ++s)   // S = Q K^T
          umma_f16(tmem_base, desc_kmajor(q_addr, s), desc_kmajor(k_addr, s), id_kk, s > 0);
        umma_commit(&bar[kKvBarSFull]);
        return true;
      };
      auto issue_dp = [&](int w) -> bool {   // the Q/dO buffer of w was already seen full by issue_s(w)
        const int b = w & 1;
        if (!mbar_wait(&bar[kKvBarDpFree], (w & 1) ^ 1, abort_flag, p.status, kTimeoutMma)) return false;
        tc_fence_after();
        const uint32_t do_addr = smem_u32(sdO + b * kFaTileBytes);
#pragma unroll
        for (int s = 0; s < 8; ++s)   // dP = dO V^T
          umma_f16(tmem_base + 128, desc_kmajor(do_addr, s), desc_kmajor(v_addr, s), id_kk, s > 0);
        umma_commit(&bar[kKvBarDpFull]);
        return true;
      };
      if (ok && total > 0) ok = issue_s(0) && issue_dp(0);
      for (int w = 0; w < total && ok; ++w) {
        const int b = w & 1;
        const uint32_t q_addr = smem_u32(sQ + b * kFaTileBytes), do_addr = smem_u32(sdO + b * kFaTileBytes);
        if (!mbar_wait(&bar[kKvBarPReady], w & 1, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int s = 0; s < 8; ++s)   // dV[key][d] += P[q][key]^T dO[q][d]: both operands MN-major
          umma_f16(tmem_base + 256, desc_mnmajor(x_addr, s), desc_mnmajor(do_addr, s), id_mm, (w > 0) || (s > 0));
        umma_commit(&bar[kKvBarPFree]);
        if (w + 1 < total) ok = issue_s(w + 1);
        if (!ok) break;
        if (!mbar_wait(&bar[kKvBarDsReady], w & 1, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int s = 0; s < 8; ++s)   // dK[key][d] += dS[q][key]^T Q[q][d]
          umma_f16(tmem_base + 384, desc_mnmajor(x_addr, s), desc_mnmajor(q_addr, s), id_mm, (w > 0) || (s > 0));
        umma_commit(&bar[kKvBarDsFree]);
        umma_commit(&bar[kKvBarQdoFree + b]);
        if (w + 1 < total) ok = issue_dp(w + 1);
      }
      if (ok) umma_commit(&bar[kKvBarAccFull]);
    }
  } else {
    const int qd = warp & 3;
    const int grp = (warp >= 6) ? 1 : 0;   // warp group: owns column chunks 2*grp, 2*grp+1; writes dV (0) or dK (1)
    const int c0 = 2 * grp;
    const int r = qd * 32 + lane;          // query row within the tile; key row in the epilogue
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const float sl2 = p.scale * kFaLog2e;
    const uint32_t x_addr = smem_u32(sX);
    bool ok = true;
    for (int w = 0; w < total && ok; ++w) {
      const int hh = hk * rep + w / n_q_tiles;
      const int m0 = j0 + (w % n_q_tiles) * kFaTile;
      const int i = m0 + r, ic = min(i, p.T - 1);
      // per-row values of this pair; the loads are in flight while the S barrier is waited on
      const int st = p.seq_start[ic];
      const int st_max = p.seq_start[min(m0 + kFaTile - 1, p.T - 1)];
      const float lse2 = p.lse[static_cast<long long>(hh) * p.T + ic] * kFaLog2e;
      const float dl = p.delta[static_cast<long long>(hh) * p.T + ic];
      const int lo = max(st - j0, 0);
      const int span = (i < p.T) ? (min(i - j0, kFaTile - 1) - lo) : -1;
      const bool need_mask = (j0 + kFaTile - 1 > m0) || (j0 < st_max) || (m0 + kFaTile > p.T);

      if (!mbar_wait(&bar[kKvBarSFull], w & 1, abort_flag, p.status, kTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after();
      uint32_t pk[32];
      if (need_mask) kv_p_row<true>(tmem_base + lane_off, sl2, -lse2, lo, span, c0, pk);
      else kv_p_row<false>(tmem_base + lane_off, sl2, -lse2, 0, 0, c0, pk);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[kKvBarSFree]);
      // the previous pair's dK MMA must be done with the shared P/dS tile
      if (w > 0 && !mbar_wait(&bar[kKvBarDsFree], (w - 1) & 1, abort_flag, p.status, kTimeoutEpilogue)) {
        ok = false;
        break;
      }
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t ck[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) ck[e] = pk[cc * 16 + e];
        store_row_chunk_sw128(x_addr, r, c0 + cc, ck);
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[kKvBarPReady]);

      if (!mbar_wait(&bar[kKvBarDpFull], w & 1, abort_flag, p.status, kTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after();
      {                                    // dS = P * (dP - delta) * scale, in place over the packed P row
        uint32_t dv[64];
        tmem_ld_64(tmem_base + 128 + c0 * 32 + lane_off, dv);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar[kKvBarDpFree]);
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const uint32_t pp = pk[e];
          const float p0 = __uint_as_float(pp << 16), p1 = __uint_as_float(pp & 0xffff0000u);
          pk[e] = pack_bf16x2(p0 * (__uint_as_float(dv[2 * e]) - dl) * p.scale,
                              p1 * (__uint_as_float(dv[2 * e + 1]) - dl) * p.scale);
        }
      }
      if (!mbar_wait(&bar[kKvBarPFree], w & 1, abort_flag, p.status, kTimeoutEpilogue)) { ok = false; break; }
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t ck[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) ck[e] = pk[cc * 16 + e];
        store_row_chunk_sw128(x_addr, r, c0 + cc, ck);
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[kKvBarDsReady]);
    }
    if (ok && total > 0 && mbar_wait(&bar[kKvBarAccFull], 0, abort_flag, p.status, kTimeoutEpilogue)) {
      tc_fence_after();
      const int jrow = j0 + r;
      const int jc = min(jrow, p.T - 1);
      __nv_bfloat16* krow = p.out + static_cast<long long>(jc) * p.o_stride + static_cast<long long>(hk) * 128;
      __nv_bfloat16* vrow = p.out2 + static_cast<long long>(jc) * p.o2_stride + static_cast<long long>(hk) * 128;
      {
        const int half = grp;              // group 0 drains the dV accumulator, group 1 the dK accumulator
        __nv_bfloat16* dst = half ? krow : vrow;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_base + 256 + half * 128 + c * 32 + lane_off, v);
          tmem_ld_wait();
          if (jrow < p.T) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(v[g * 8]), __uint_as_float(v[g * 8 + 1]));
              o.y = pack_bf16x2(__uint_as_float(v[g * 8 + 2]), __uint_as_float(v[g * 8 + 3]));
              o.z = pack_bf16x2(__uint_as_float(v[g * 8 + 4]), __uint_as_float(v[g * 8 + 5]));
              o.w = pack_bf16x2(__uint_as_float(v[g * 8 + 6]), __uint_as_float(v[g * 8 + 7]));
              *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = o;
            }
          }
        }
      }
    }
  }

  __syncwarp();
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace pm

using namespace pm;

// dout, q: [T, hq*128] (token strides o_stride / q_stride); k, v: [T, hkv*128] (v may be a strided view).
// dq:[T,hq,128], dk:[T,hkv,128], dv:[T,hkv,128] (strided). lse, delta: [hq][T].
extern "C" int pm_attn_bwd_tc(const void* dout, long long do_stride, const void* q, long long q_stride, const void* k,
                              long long k_stride, const void* v, long long v_stride, const float* lse,
                              const float* delta, void* dq, long long dq_stride, void* dk, long long dk_stride, void* dv,
                              long long dv_stride, const int* seq_start, int T, int hq, int hkv, float scale, int* status,
                              cudaStream_t st) {
  if (hq % hkv || T <= 0) return -1;
  if ((q_stride | k_stride | v_stride | do_stride | dq_stride | dk_stride | dv_stride) % 8) return -2;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(dout) | reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) |
       reinterpret_cast<uintptr_t>(dv)) & 15)
    return -3;
  CUtensorMap mq, mk, mv, mdo;
  int rc;
  if ((rc = make_map(&mq, q, static_cast<uint64_t>(hq) * 128, T, q_stride, 64, kFaTile))) return rc;
  if ((rc = make_map(&mk, k, static_cast<uint64_t>(hkv) * 128, T, k_stride, 64, kFaTile))) return rc;
  if ((rc = make_map(&mv, v, static_cast<uint64_t>(hkv) * 128, T, v_stride, 64, kFaTile))) return rc;
  if ((rc = make_map(&mdo, dout, static_cast<uint64_t>(hq) * 128, T, do_stride, 64, kFaTile))) return rc;
  FaParams p{};
  p.lse = const_cast<float*>(lse); p.delta = delta; p.seq_start = seq_start;
  p.T = T; p.hq = hq; p.hkv = hkv; p.scale = scale; p.status = status;
  const int smem = 227 * 1024;
  static DeviceOnce once;
  if (once.pending()) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_dq_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaFuncSetAttribute(attn_bwd_dkv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    once.mark();
  }
  const int tiles = (T + kFaTile - 1) / kFaTile;
  p.out = static_cast<__nv_bfloat16*>(dq);
  p.o_stride = dq_stride;
  attn_bwd_dq_tc_kernel<<<dim3(tiles, hq), kFaThreads2, smem, st>>>(mq, mk, mv, mdo, p);
  int e = static_cast<int>(cudaGetLastError());
  if (e) return e;
  p.out = static_cast<__nv_bfloat16*>(dk);
  p.o_stride = dk_stride;
  p.out2 = static_cast<__nv_bfloat16*>(dv);
  p.o2_stride = dv_stride;
  attn_bwd_dkv_tc_kernel<<<dim3(tiles, hkv), kFaThreads2, smem, st>>>(mq, mk, mv, mdo, p);
  return static_cast<int>(cudaGetLastError());
}
