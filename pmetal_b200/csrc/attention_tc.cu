// Varlen causal flash attention forward on tcgen05 tensor cores (head_dim 128, GQA).
//
// One CTA per (128-query tile, head). Q, K and V tiles arrive by TMA into 128-byte-swizzled shared
// memory; S = Q K^T and O_j = P V are tcgen05.mma instructions with fp32 accumulators in TMEM:
//
//   TMEM columns   [0,128) S buffer 0   [128,256) S buffer 1   [256,384) O buffer 0   [384,512) O buffer 1
//
// Warp roles: warp 0 TMA producer, warp 1 MMA issuer (owns TMEM), warps 2..5 softmax. A softmax thread
// owns one query row (TMEM lane), so row max and row sum need no shuffles. Per key tile it reads the row
// of S from TMEM twice (max pass, exp pass), writes P as bf16 into shared memory in the layout the
// P·V MMA reads, and folds the previous tile's O_j into its register accumulator with the online-softmax
// correction. QK^T of tile j+1 is issued before the softmax of tile j finishes, so tensor cores and the
// exp pipeline overlap. Same masking rule as attention.cu: key j is visible to query i iff
// seq_start[i] <= j <= i.
#include "attention_tc.cuh"
#include "pmetal_b200.h"

namespace pm {

// barrier indices inside the shared barrier array
enum {
  kBarQ = 0, kBarK = 1 /*2*/, kBarV = 3 /*2*/, kBarKvFree = 5 /*2*/, kBarSFull = 7 /*2*/, kBarSFree = 9 /*2*/,
  kBarP = 11, kBarOFull = 12 /*2*/, kBarOFree = 14 /*2*/, kBarCount = 16
};

// Row maximum of 128 fp32 TMEM columns of this thread's lane; with kMask only columns in [lo, lo+span] count.
template <bool kMask>
__device__ __forceinline__ float row_max(uint32_t taddr, int lo, int span) {
  float mx = -INFINITY;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t v[32];
    tmem_ld_32x32b_x32(taddr + c * 32, v);
    tmem_ld_wait();
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      float x = __uint_as_float(v[e]);
      if (kMask) x = (static_cast<unsigned>(c * 32 + e - lo) <= static_cast<unsigned>(span) && span >= 0) ? x : -INFINITY;
      mx = fmaxf(mx, x);
    }
  }
  return mx;
}

// p = exp2(s * a + b) for the 128 columns of this row, written as bf16 into the swizzled P tile; returns the row sum.
template <bool kMask>
__device__ __forceinline__ float exp_rows(uint32_t taddr, uint32_t tile_addr, int r, float a, float b, int lo,
                                          int span) {
  float rs = 0.f;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t v[32];
    tmem_ld_32x32b_x32(taddr + c * 32, v);
    tmem_ld_wait();
    uint32_t pk[16];
#pragma unroll
    for (int e = 0; e < 32; e += 2) {
      float p0 = fast_exp2(fmaf(__uint_as_float(v[e]), a, b));
      float p1 = fast_exp2(fmaf(__uint_as_float(v[e + 1]), a, b));
      if (kMask) {
        const bool any = span >= 0;
        p0 = (any && static_cast<unsigned>(c * 32 + e - lo) <= static_cast<unsigned>(span)) ? p0 : 0.f;
        p1 = (any && static_cast<unsigned>(c * 32 + e + 1 - lo) <= static_cast<unsigned>(span)) ? p1 : 0.f;
      }
      rs += p0 + p1;
      pk[e >> 1] = pack_bf16x2(p0, p1);
    }
    store_row_chunk_sw128(tile_addr, r, c, pk);
  }
  return rs;
}

__global__ void __launch_bounds__(kFaThreads, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const FaParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                          // 32 KB
  uint8_t* sK = smem + kFaTileBytes;           // 2 x 32 KB
  uint8_t* sV = smem + 3 * kFaTileBytes;       // 2 x 32 KB
  uint8_t* sP = smem + 5 * kFaTileBytes;       // 32 KB
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + 6 * kFaTileBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + kBarCount);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;   // late (long) tiles first
  const int h = blockIdx.y;
  const int hk = h / (p.hq / p.hkv);
  const int q0 = qt * kFaTile;

  if (threadIdx.x == 0) {
    mbar_init(&bar[kBarQ], 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar[kBarK + i], 1);
      mbar_init(&bar[kBarV + i], 1);
      mbar_init(&bar[kBarKvFree + i], 1);
      mbar_init(&bar[kBarSFull + i], 1);
      mbar_init(&bar[kBarSFree + i], 4);
      mbar_init(&bar[kBarOFull + i], 1);
      mbar_init(&bar[kBarOFree + i], 4);
    }
    mbar_init(&bar[kBarP], 4);
    *abort_flag = 0;
    mbar_init_fence();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // key range of this query tile: from the document start of its first row up to its last row
  int kv_lo = (p.seq_start[q0] / kFaTile) * kFaTile;
  const int kv_hi = max(min(q0 + kFaTile + p.shift, p.Tk), 0);
  const int n_tiles = max((kv_hi - kv_lo + kFaTile - 1) / kFaTile, 0);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(&bar[kBarQ], kFaTileBytes);
      tma_load_2d(sQ, &map_q, &bar[kBarQ], h * 128, q0);
      tma_load_2d(sQ + kFaBox, &map_q, &bar[kBarQ], h * 128 + 64, q0);
      for (int j = 0; j < n_tiles; ++j) {
        const int b = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&bar[kBarKvFree + b], ph ^ 1, abort_flag, p.status, kTimeoutProducer)) break;
        const int j0 = kv_lo + j * kFaTile;
        mbar_expect_tx(&bar[kBarK + b], kFaTileBytes);
        tma_load_2d(sK + b * kFaTileBytes, &map_k, &bar[kBarK + b], hk * 128, j0);
        tma_load_2d(sK + b * kFaTileBytes + kFaBox, &map_k, &bar[kBarK + b], hk * 128 + 64, j0);
        mbar_expect_tx(&bar[kBarV + b], kFaTileBytes);
        tma_load_2d(sV + b * kFaTileBytes, &map_v, &bar[kBarV + b], hk * 128, j0);
        tma_load_2d(sV + b * kFaTileBytes + kFaBox, &map_v, &bar[kBarV + b], hk * 128 + 64, j0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_qk = make_idesc_bf16(128, 0, 0);   // A = Q (K-major), B = K (K-major)
      const uint32_t idesc_pv = make_idesc_bf16(128, 0, 1);   // A = P (K-major), B = V (MN-major: rows are keys)
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      bool ok = mbar_wait(&bar[kBarQ], 0, abort_flag, p.status, kTimeoutMma);
      auto issue_qk = [&](int j) -> bool {
        const int b = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&bar[kBarK + b], ph, abort_flag, p.status, kTimeoutMma)) return false;
        if (!mbar_wait(&bar[kBarSFree + b], ph ^ 1, abort_flag, p.status, kTimeoutMma)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + b * kFaTileBytes);
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          const uint32_t off = (s >> 2) * kFaBox + (s & 3) * 32;
          umma_f16(tmem_base + b * 128, make_smem_desc(q_addr + off, 16u, 1024u),
                   make_smem_desc(k_addr + off, 16u, 1024u), idesc_qk, s > 0);
        }
        umma_commit(&bar[kBarSFull + b]);
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_qk(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int b = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (j + 1 < n_tiles) ok = issue_qk(j + 1);   // overlaps the softmax of tile j
        if (!ok) break;
        if (!mbar_wait(&bar[kBarV + b], ph, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
        if (!mbar_wait(&bar[kBarP], j & 1, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
        if (!mbar_wait(&bar[kBarOFree + b], ph ^ 1, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + b * kFaTileBytes);
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          // A: P[128 q][128 keys], K-major in two 64-key boxes; B: V[128 keys][128 d], MN-major: 16 keys = 2048 B,
          // the two 64-wide d chunks are the two boxes (LBO = 16 KB)
          umma_f16(tmem_base + 256 + b * 128,
                   make_smem_desc(p_addr + (s >> 2) * kFaBox + (s & 3) * 32, 16u, 1024u),
                   make_smem_desc(v_addr + s * 2048, static_cast<uint32_t>(kFaBox), 1024u), idesc_pv, s > 0);
        }
        umma_commit(&bar[kBarOFull + b]);    // O_j ready; also: P and this K/V stage have been consumed
        umma_commit(&bar[kBarKvFree + b]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax (one thread per query row)
    const int qd = warp & 3;
    const int r = qd * 32 + lane;
    const int i = q0 + r;
    const int ic = min(i, p.T - 1);
    const int st = p.seq_start[ic];
    const int st_max = p.seq_start[min(q0 + kFaTile - 1, p.T - 1)];
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const float sl2 = p.scale * kFaLog2e;
    float o_reg[128];
#pragma unroll
    for (int c = 0; c < 128; ++c) o_reg[c] = 0.f;
    float m_run = -INFINITY, l_run = 0.f, corr_prev = 1.f;
    const uint32_t sP_addr = smem_u32(sP);
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int b = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      const int j0 = kv_lo + j * kFaTile;
      const bool need_mask = (j0 + kFaTile - 1 > q0 + p.shift) || (j0 < st_max) || (j0 + kFaTile > p.Tk);
      if (!mbar_wait(&bar[kBarSFull + b], ph, abort_flag, p.status, kTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after();
      // valid key columns of this row inside the tile: [lo, lo + span]; span < 0 means none
      const int lo = max(st - j0, 0);
      const int span = min(min(i + p.shift, p.Tk - 1) - j0, kFaTile - 1) - lo;
      // pass 1: row maximum
      const float mx = need_mask ? row_max<true>(tmem_base + b * 128 + lane_off, lo, span)
                                 : row_max<false>(tmem_base + b * 128 + lane_off, 0, 0);
      const float m_new = fmaxf(m_run, mx * sl2);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_use);
      m_run = m_new;
      // P of the previous tile must have been consumed before it is overwritten
      if (j > 0 && !mbar_wait(&bar[kBarOFull + (b ^ 1)], ((j - 1) >> 1) & 1, abort_flag, p.status, kTimeoutEpilogue)) {
        ok = false;
        break;
      }
      // pass 2: p = exp2(s * scale - m), row sum, bf16 P into shared memory (128B-swizzled, two 64-key boxes)
      const float rs = need_mask ? exp_rows<true>(tmem_base + b * 128 + lane_off, sP_addr, r, sl2, -m_use, lo, span)
                                 : exp_rows<false>(tmem_base + b * 128 + lane_off, sP_addr, r, sl2, -m_use, 0, 0);
      l_run = l_run * corr + rs;
      fence_async_smem();        // generic-proxy writes of P -> visible to the tensor-core (async) proxy
      tc_fence_before();         // this thread's TMEM reads of S are complete
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bar[kBarP]);
        mbar_arrive(&bar[kBarSFree + b]);
      }
      // fold the previous tile's O into the running accumulator (its MMA finished: waited above)
      if (j > 0) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_base + 256 + (b ^ 1) * 128 + c * 32 + lane_off, v);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) o_reg[c * 32 + e] = o_reg[c * 32 + e] * corr_prev + __uint_as_float(v[e]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar[kBarOFree + (b ^ 1)]);
      }
      corr_prev = corr;
    }
    if (ok && n_tiles > 0) {
      const int jl = n_tiles - 1, b = jl & 1;
      if (mbar_wait(&bar[kBarOFull + b], (jl >> 1) & 1, abort_flag, p.status, kTimeoutEpilogue)) {
        tc_fence_after();
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        __nv_bfloat16* orow = p.out + static_cast<long long>(ic) * p.o_stride + static_cast<long long>(h) * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_base + 256 + b * 128 + c * 32 + lane_off, v);
          tmem_ld_wait();
          if (i < p.T) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 o;
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e)
                f[e] = (o_reg[c * 32 + g * 8 + e] * corr_prev + __uint_as_float(v[g * 8 + e])) * inv;
              o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
              o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
              *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = o;
            }
          }
        }
        if (i < p.T) p.lse[static_cast<long long>(h) * p.T + i] = (m_run + log2f(l_run)) / kFaLog2e;
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


// ============================================================================================== persistent kernel
// Same tiling, 320 threads: warp 0 TMA, warp 1 MMA, warps 2..5 = softmax group 0, warps 6..9 = softmax group 1.
//
// Work items are (128-query tile, head) pairs, longest first; CTA c takes items c, c + gridDim.x, ... and keeps its
// tensor memory, barriers and pipelines alive across them, so the loads and the first Q K^T products of the next
// item run while the softmax groups finish the current one.
//
// Inside an item the key tiles alternate between the two groups. A group owns an S buffer, a P tile and an O buffer
// together with its own running (max, sum): the kernel computes two independent online-softmax partials over disjoint
// key subsets and merges them at the end of the item. O_b accumulates in TMEM across the group's tiles (the P·V MMA adds
// to it); a thread rescales its row of O in TMEM only when the running maximum grew by more than 2^8, so the common
// case costs two TMEM reads of S per key tile (maximum, then exponentials) and none of O.
//
//   TMEM columns   [0,128) S0   [128,256) S1   [256,384) O0   [384,512) O1
//   shared memory  Q | KV ring: K0 K1 V0 V1 | P0 P1   (7 x 32 KB)
enum {
  kB2QFull = 0, kB2QFree = 1, kB2K = 2 /*2*/, kB2V = 4 /*2*/, kB2KvFree = 6 /*2*/, kB2SFull = 8 /*2*/,
  kB2SFree = 10 /*2*/, kB2P = 12 /*2*/, kB2OFull = 14 /*2*/, kB2OFree = 16 /*2*/, kB2Count = 18
};
constexpr float kFaRescaleGap = 8.f;   // log2 units: P stays below 2^8 while the stale maximum is kept

__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// barrier among the 256 softmax threads only (the TMA and MMA warps never join it)
__device__ __forceinline__ void softmax_groups_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// item w of the launch -> (query tile, head); long query tiles (late in the stream) come first
struct FaItem {
  int q0, h, hk, kv_lo, n_tiles;
};
__device__ __forceinline__ FaItem fa_item(const FaParams& p, int w, int n_qt) {
  FaItem it;
  const int qt = n_qt - 1 - w / p.hq;
  it.h = w % p.hq;
  it.hk = it.h / (p.hq / p.hkv);
  it.q0 = qt * kFaTile;
  it.kv_lo = (p.seq_start[it.q0] / kFaTile) * kFaTile;
  const int kv_hi = max(min(it.q0 + kFaTile + p.shift, p.Tk), 0);
  it.n_tiles = max((kv_hi - it.kv_lo + kFaTile - 1) / kFaTile, 0);
  return it;
}

// k-th item of this CTA: rounds of gridDim.x items, walked forwards and backwards in turn, so that with items sorted
// by decreasing length every CTA gets a similar total
__device__ __forceinline__ int fa_work(int k) {
  const int g = static_cast<int>(gridDim.x), c = static_cast<int>(blockIdx.x);
  return k * g + ((k & 1) ? g - 1 - c : c);
}

__global__ void __launch_bounds__(kFaThreads2, 1)
attn_fwd_tc2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const FaParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                          // 32 KB
  uint8_t* sK = smem + kFaTileBytes;           // 2 x 32 KB
  uint8_t* sV = smem + 3 * kFaTileBytes;       // 2 x 32 KB
  uint8_t* sP = smem + 5 * kFaTileBytes;       // 2 x 32 KB (one per softmax group)
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + 7 * kFaTileBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + kB2Count);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.T + kFaTile - 1) / kFaTile;
  const int total = n_qt * p.hq;

  if (threadIdx.x == 0) {
    mbar_init(&bar[kB2QFull], 1);
    mbar_init(&bar[kB2QFree], 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar[kB2K + i], 1);
      mbar_init(&bar[kB2V + i], 1);
      mbar_init(&bar[kB2KvFree + i], 1);
      mbar_init(&bar[kB2SFull + i], 1);
      mbar_init(&bar[kB2SFree + i], 4);
      mbar_init(&bar[kB2P + i], 4);
      mbar_init(&bar[kB2OFull + i], 1);
      mbar_init(&bar[kB2OFree + i], 8);
    }
    *abort_flag = 0;
    mbar_init_fence();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t g = 0;        // key tiles loaded so far: ring stage g & 1
      bool ok = true;
      int k = 0;
      for (int w = fa_work(0); w < total && ok; w = fa_work(++k)) {
        const FaItem it = fa_item(p, w, n_qt);
        // Q is single-buffered: the previous item's last Q K^T must have read it
        if (!mbar_wait(&bar[kB2QFree], (k & 1) ^ 1, abort_flag, p.status, kTimeoutProducer)) break;
        mbar_expect_tx(&bar[kB2QFull], kFaTileBytes);
        tma_load_2d(sQ, &map_q, &bar[kB2QFull], it.h * 128, it.q0);
        tma_load_2d(sQ + kFaBox, &map_q, &bar[kB2QFull], it.h * 128 + 64, it.q0);
        for (int j = 0; j < it.n_tiles; ++j, ++g) {
          const int s = g & 1;
          if (!mbar_wait(&bar[kB2KvFree + s], ((g >> 1) & 1) ^ 1, abort_flag, p.status, kTimeoutProducer)) { ok = false; break; }
          const int j0 = it.kv_lo + j * kFaTile;
          mbar_expect_tx(&bar[kB2K + s], kFaTileBytes);
          tma_load_2d(sK + s * kFaTileBytes, &map_k, &bar[kB2K + s], it.hk * 128, j0);
          tma_load_2d(sK + s * kFaTileBytes + kFaBox, &map_k, &bar[kB2K + s], it.hk * 128 + 64, j0);
          mbar_expect_tx(&bar[kB2V + s], kFaTileBytes);
          tma_load_2d(sV + s * kFaTileBytes, &map_v, &bar[kB2V + s], it.hk * 128, j0);
          tma_load_2d(sV + s * kFaTileBytes + kFaBox, &map_v, &bar[kB2V + s], it.hk * 128 + 64, j0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_qk = make_idesc_bf16(128, 0, 0);   // A = Q (K-major), B = K (K-major)
      const uint32_t idesc_pv = make_idesc_bf16(128, 0, 1);   // A = P (K-major), B = V (MN-major: rows are keys)
      const uint32_t q_addr = smem_u32(sQ);
      uint32_t g0 = 0;                 // key tiles of earlier items
      uint32_t cnt[2] = {0, 0};        // tiles issued so far on S/O buffer b (phases of SFree, P)
      bool ok = true;
      int k = 0;
      for (int w = fa_work(0); w < total && ok; w = fa_work(++k)) {
        const FaItem it = fa_item(p, w, n_qt);
        const int flip = k & 1;        // the group that takes tile 0 alternates from item to item
        if (!mbar_wait(&bar[kB2QFull], k & 1, abort_flag, p.status, kTimeoutMma)) break;
        uint32_t qk_cnt[2] = {cnt[0], cnt[1]};
        auto issue_qk = [&](int j) -> bool {
          const int b = (j + flip) & 1;
          const uint32_t g = g0 + j;
          const int s = g & 1;
          if (!mbar_wait(&bar[kB2K + s], (g >> 1) & 1, abort_flag, p.status, kTimeoutMma)) return false;
          if (!mbar_wait(&bar[kB2SFree + b], (qk_cnt[b] & 1) ^ 1, abort_flag, p.status, kTimeoutMma)) return false;
          ++qk_cnt[b];
          tc_fence_after();
          const uint32_t k_addr = smem_u32(sK + s * kFaTileBytes);
#pragma unroll
          for (int x = 0; x < 8; ++x)
            umma_f16(tmem_base + b * 128, desc_kmajor(q_addr, x), desc_kmajor(k_addr, x), idesc_qk, x > 0);
          umma_commit(&bar[kB2SFull + b]);
          if (j == it.n_tiles - 1) umma_commit(&bar[kB2QFree]);   // Q may be replaced by the next item's tile
          return true;
        };
        if (it.n_tiles == 0) umma_commit(&bar[kB2QFree]);
        if (it.n_tiles > 0) ok = issue_qk(0);
        for (int j = 0; j < it.n_tiles && ok; ++j) {
          const int b = (j + flip) & 1;
          const uint32_t g = g0 + j;
          const int s = g & 1;
          if (j + 1 < it.n_tiles) ok = issue_qk(j + 1);   // overlaps the softmax of tile j
          if (!ok) break;
          if (!mbar_wait(&bar[kB2V + s], (g >> 1) & 1, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
          if (!mbar_wait(&bar[kB2P + b], cnt[b] & 1, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
          // first P·V of the item on this buffer overwrites it: the previous item's output must have been read
          if (j < 2 && !mbar_wait(&bar[kB2OFree + b], (k & 1) ^ 1, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
          ++cnt[b];
          tc_fence_after();
          const uint32_t v_addr = smem_u32(sV + s * kFaTileBytes), p_addr = smem_u32(sP + b * kFaTileBytes);
#pragma unroll
          for (int x = 0; x < 8; ++x)   // O_b (+)= P_b[128 q][128 keys] V[128 keys][128 d]
            umma_f16(tmem_base + 256 + b * 128, desc_kmajor(p_addr, x), desc_mnmajor(v_addr, x), idesc_pv,
                     (j >= 2) || (x > 0));
          umma_commit(&bar[kB2OFull + b]);    // O_b updated; P_b and this K/V stage have been consumed
          umma_commit(&bar[kB2KvFree + s]);
        }
        g0 += it.n_tiles;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax groups (one thread per query row)
    const int grp = (warp >= 6) ? 1 : 0;
    const int qd = warp & 3;
    const int r = qd * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const float sl2 = p.scale * kFaLog2e;
    const uint32_t s_tmem = tmem_base + grp * 128 + lane_off;
    const uint32_t o_tmem = tmem_base + 256 + grp * 128 + lane_off;
    const uint32_t o_other = tmem_base + 256 + (grp ^ 1) * 128 + lane_off;
    const uint32_t sP_addr = smem_u32(sP + grp * kFaTileBytes);
    float* xch = reinterpret_cast<float*>(sP + grp * kFaTileBytes);          // this group's P tile, free after its last P·V
    const float* xo = reinterpret_cast<const float*>(sP + (grp ^ 1) * kFaTileBytes);
    uint32_t cnt = 0;      // tiles this group has processed so far (phases of SFull, OFull)
    bool ok = true;
    int k = 0;
    // the item description and this row's document start are fetched one item ahead of their use
    FaItem it_next = {};
    int st_next = 0, st_max_next = 0;
    if (fa_work(0) < total) {
      it_next = fa_item(p, fa_work(0), n_qt);
      st_next = p.seq_start[min(it_next.q0 + r, p.T - 1)];
      st_max_next = p.seq_start[min(it_next.q0 + kFaTile - 1, p.T - 1)];
    }
    for (int w = fa_work(0); w < total; w = fa_work(++k)) {
      const FaItem it = it_next;
      const int st = st_next, st_max = st_max_next;
      if (fa_work(k + 1) < total) {
        it_next = fa_item(p, fa_work(k + 1), n_qt);
        st_next = p.seq_start[min(it_next.q0 + r, p.T - 1)];
        st_max_next = p.seq_start[min(it_next.q0 + kFaTile - 1, p.T - 1)];
      }
      const int flip = k & 1;
      const int i = it.q0 + r;
      const int ic = min(i, p.T - 1);
      float m_run = -INFINITY, l_run = 0.f;
      int kk = 0;          // index of the tile among this group's tiles of the item
      for (int j = grp ^ flip; j < it.n_tiles && ok; j += 2, ++kk, ++cnt) {
        const int j0 = it.kv_lo + j * kFaTile;
        const bool need_mask = (j0 + kFaTile - 1 > it.q0 + p.shift) || (j0 < st_max) || (j0 + kFaTile > p.Tk);
        if (!mbar_wait(&bar[kB2SFull + grp], cnt & 1, abort_flag, p.status, kTimeoutEpilogue)) { ok = false; break; }
        tc_fence_after();
        // valid key columns of this row inside the tile: [lo, lo + span]; span < 0 means none
        const int lo = max(st - j0, 0);
        const int span = min(min(i + p.shift, p.Tk - 1) - j0, kFaTile - 1) - lo;
        // pass 1 over S_b: row maximum
        const float mx = need_mask ? row_max<true>(s_tmem, lo, span) : row_max<false>(s_tmem, 0, 0);
        const float m_cand = fmaxf(m_run, mx * sl2);
        // the previous tile's P·V must be complete: it read P_b and wrote O_b
        if (kk > 0 && !mbar_wait(&bar[kB2OFull + grp], (cnt - 1) & 1, abort_flag, p.status, kTimeoutEpilogue)) {
          ok = false;
          break;
        }
        const bool grow = (m_run != -INFINITY) && (m_cand > m_run + kFaRescaleGap);
        if (m_run == -INFINITY) m_run = m_cand;          // nothing accumulated for this row yet (its O row is exactly 0)
        if (kk > 0 && __any_sync(0xffffffffu, grow)) {
          tc_fence_after();
          const float corr = grow ? fast_exp2(m_run - m_cand) : 1.f;
          if (grow) { m_run = m_cand; l_run *= corr; }
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(o_tmem + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * corr);
            tmem_st_32x32b_x32(o_tmem + c * 32, o);
          }
          tmem_st_wait();
        }
        const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
        // pass 2 over S_b: p = exp2(s * scale - m), row sum, bf16 P into this group's shared-memory tile
        const float rs = need_mask ? exp_rows<true>(s_tmem, sP_addr, r, sl2, -m_use, lo, span)
                                   : exp_rows<false>(s_tmem, sP_addr, r, sl2, -m_use, 0, 0);
        l_run += rs;
        fence_async_smem();        // generic-proxy writes of P -> visible to the tensor-core (async) proxy
        tc_fence_before();         // TMEM reads / writes of this thread are ordered before the MMA that follows the arrive
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bar[kB2P + grp]);
          mbar_arrive(&bar[kB2SFree + grp]);   // S_b has been read twice: the next Q K^T on this buffer may overwrite it
        }
      }
      // ---- merge the two groups' partials and write the output
      if (ok && kk > 0 && !mbar_wait(&bar[kB2OFull + grp], (cnt - 1) & 1, abort_flag, p.status, kTimeoutEpilogue)) ok = false;
      if (kk > 0 && ok) {
        xch[r] = m_run;
        xch[128 + r] = l_run;
      }
      tc_fence_before();
      softmax_groups_sync();       // every softmax thread reaches this point, also after an abandoned wait
      tc_fence_after();
      const int n_other = (it.n_tiles + 1 - ((grp ^ 1) ^ flip)) / 2;     // tiles of the other group in this item
      if (ok && !*abort_flag && it.n_tiles > 0) {
        const float m_o = n_other > 0 ? xo[r] : -INFINITY;
        const float l_o = n_other > 0 ? xo[128 + r] : 0.f;
        const float m_me = kk > 0 ? m_run : -INFINITY;
        const float m = fmaxf(m_me, m_o);
        const float a_me = (m_me == -INFINITY) ? 0.f : fast_exp2(m_me - m);
        const float a_o = (m_o == -INFINITY) ? 0.f : fast_exp2(m_o - m);
        const float l = l_run * a_me + l_o * a_o;
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const float w_me = a_me * inv, w_o = a_o * inv;
        __nv_bfloat16* orow = p.out + static_cast<long long>(ic) * p.o_stride + static_cast<long long>(it.h) * 128;
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int c = 2 * grp + cc;          // group g writes output columns [64 g, 64 g + 64)
          uint32_t a[32], bq[32];
          tmem_ld_32x32b_x32(o_tmem + c * 32, a);
          tmem_ld_32x32b_x32(o_other + c * 32, bq);
          tmem_ld_wait();
          if (i < p.T) {
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) {
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const float x = (w_me != 0.f) ? __uint_as_float(a[gq * 8 + e]) * w_me : 0.f;
                const float y = (w_o != 0.f) ? __uint_as_float(bq[gq * 8 + e]) * w_o : 0.f;
                f[e] = x + y;
              }
              uint4 o;
              o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
              o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
              *reinterpret_cast<uint4*>(orow + c * 32 + gq * 8) = o;
            }
          }
        }
        if (grp == 0 && i < p.T) p.lse[static_cast<long long>(it.h) * p.T + i] = (m + log2f(l)) / kFaLog2e;
      }
      // both O buffers and both exchange areas are free again
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bar[kB2OFree]);
        mbar_arrive(&bar[kB2OFree + 1]);
      }
      softmax_groups_sync();
      if (!ok || *abort_flag) break;
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

// q:[T, hq*128 (+...)] with token stride q_stride, k/v:[Tk, ...] likewise (v may be a strided view). out:[T,hq,128],
// lse:[hq,T]. Key j is visible to query i iff seq_start[i] <= j <= i + shift.
static int attn_fwd_tc_launch(int variant, const void* q, long long q_stride, const void* k, long long k_stride,
                              const void* v, long long v_stride, void* out, long long o_stride, float* lse,
                              const int* seq_start, int T, int Tk, int shift, int hq, int hkv, float scale, int* status,
                              cudaStream_t st) {
  if (hq % hkv || T <= 0 || Tk <= 0) return -1;
  if ((q_stride | k_stride | v_stride | o_stride) % 8) return -2;
  CUtensorMap mq, mk, mv;
  int rc;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) return -3;
  if ((rc = make_map(&mq, q, static_cast<uint64_t>(hq) * 128, T, q_stride, 64, kFaTile))) return rc;
  if ((rc = make_map(&mk, k, static_cast<uint64_t>(hkv) * 128, Tk, k_stride, 64, kFaTile))) return rc;
  if ((rc = make_map(&mv, v, static_cast<uint64_t>(hkv) * 128, Tk, v_stride, 64, kFaTile))) return rc;
  FaParams p{};
  p.out = static_cast<__nv_bfloat16*>(out);
  p.o_stride = o_stride; p.lse = lse; p.seq_start = seq_start;
  p.T = T; p.hq = hq; p.hkv = hkv; p.scale = scale; p.status = status;
  p.Tk = Tk; p.shift = shift;
  const int smem = 6 * kFaTileBytes + 1024 + 256;
  const int smem2 = 7 * kFaTileBytes + 1024 + 256;
  static DeviceOnce once;
  if (once.pending()) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaFuncSetAttribute(attn_fwd_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2);
    if (e != cudaSuccess) return static_cast<int>(e);
    once.mark();
  }
  dim3 grid((T + kFaTile - 1) / kFaTile, hq);
  if (variant == 1) {
    attn_fwd_tc_kernel<<<grid, kFaThreads, smem, st>>>(mq, mk, mv, p);
  } else {
    const int items = static_cast<int>(grid.x) * hq;      // persistent: one CTA per SM walks the item list
    attn_fwd_tc2_kernel<<<items < num_sms() ? items : num_sms(), kFaThreads2, smem2, st>>>(mq, mk, mv, p);
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int pm_attn_fwd_tc_rect(const void* q, long long q_stride, const void* k, long long k_stride, const void* v,
                                   long long v_stride, void* out, long long o_stride, float* lse, const int* seq_start,
                                   int T, int Tk, int shift, int hq, int hkv, float scale, int* status,
                                   cudaStream_t st) {
  return attn_fwd_tc_launch(2, q, q_stride, k, k_stride, v, v_stride, out, o_stride, lse, seq_start, T, Tk, shift, hq,
                            hkv, scale, status, st);
}

// Single-softmax-group variant of the same kernel (kept selectable for comparison measurements).
extern "C" int pm_attn_fwd_tc_rect_v1(const void* q, long long q_stride, const void* k, long long k_stride,
                                      const void* v, long long v_stride, void* out, long long o_stride, float* lse,
                                      const int* seq_start, int T, int Tk, int shift, int hq, int hkv, float scale,
                                      int* status, cudaStream_t st) {
  return attn_fwd_tc_launch(1, q, q_stride, k, k_stride, v, v_stride, out, o_stride, lse, seq_start, T, Tk, shift, hq,
                            hkv, scale, status, st);
}

extern "C" int pm_attn_fwd_tc(const void* q, long long q_stride, const void* k, long long k_stride, const void* v,
                              long long v_stride, void* out, long long o_stride, float* lse, const int* seq_start, int T,
                              int hq, int hkv, float scale, int* status, cudaStream_t st) {
  return pm_attn_fwd_tc_rect(q, q_stride, k, k_stride, v, v_stride, out, o_stride, lse, seq_start, T, T, 0, hq, hkv, scale,
                             status, st);
}
