// Grouped GEMMs over expert-sorted token rows (mixture-of-experts training): forward, input gradient and weight
// gradient on tcgen05 tensor cores (cf. the reference's grouped_gemm_forward / grouped_gemm_backward_dx /
// grouped_gemm_backward_dw, crates/pmetal-metal/src/kernels/metal/grouped_gemm.metal:125-465).
//
// Token rows are sorted by expert into a padded layout: expert e owns rows [off[e], off[e+1]) of the row buffers, every
// off[e] is a multiple of 128 and the padding rows are zero. A 128-row tile therefore belongs to exactly one expert and
// a 64-row reduction block never mixes two experts, so the kernels need no row masks; `off` stays on the device (the
// number of tiles that hold rows is read by the kernel), which keeps the launch sequence free of host round trips.
//
//   mode 0  Y[r, :]   = X[r, :] W_e^T          X [R, K],  W stacked [E*N, K] (K-major),        Y  [R, N]
//   mode 1  dX[r, :]  = dY[r, :] W_e           dY [R, N], W stacked [E*N, K] read MN-major,    dX [R, K]
//   mode 2  dW_e      = dY_e^T X_e (fp32)      dY [R, N] and X [R, K] both read MN-major,      dW [E, N, K]
//
// Same CTA layout as gemm_tcgen05.cu: warp 0 TMA producer, warp 1 MMA issuer (TMEM double-buffered), warps 2..5
// epilogue; persistent over the tile list; every wait is bounded.
#include "gemm_common.cuh"
#include "pmetal_b200.h"

namespace pm {

struct GroupedParams {
  int mode;
  int E;
  int rows_cap;      // row capacity of the sorted buffers (multiple of 128)
  int N, K;          // per-expert weight shape [N, K]
  int bn;            // tile width
  int stages, tmem_cols;
  const int* off;    // [E + 1] padded row offsets (device)
  void* D;
  int ldd;
  int accumulate;    // mode 2: add to D instead of overwriting
  float alpha;
  int* status;
};

struct GroupTile {
  int valid;         // 0: nothing to do for this work item
  int a_row, a_k0;   // A operand: mn coordinate, first reduction coordinate
  int b_row, b_k0;
  int nk;            // 64-wide reduction blocks
  int out_row, out_col;
  long long out_base;   // element offset of the expert's output (mode 2)
};

// expert that owns sorted row `row` (off is non-decreasing; row < off[E])
__device__ __forceinline__ int expert_of_row(const int* off, int E, int row) {
  int lo = 0, hi = E;              // invariant: off[lo] <= row < off[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(off + mid) <= row) lo = mid; else hi = mid;
  }
  return lo;
}

__device__ __forceinline__ GroupTile group_tile(const GroupedParams& p, int w) {
  GroupTile t;
  t.valid = 0;
  t.out_base = 0;
  if (p.mode < 2) {
    const int out_cols = p.mode == 0 ? p.N : p.K;
    const int red = p.mode == 0 ? p.K : p.N;
    const int n_tiles = (out_cols + p.bn - 1) / p.bn;
    const int mb = w / n_tiles, nb = w % n_tiles;
    const int m0 = mb * kBM;
    t.out_row = m0; t.out_col = nb * p.bn;
    if (m0 >= __ldg(p.off + p.E)) return t;       // past the last expert: the epilogue clears these rows
    const int e = expert_of_row(p.off, p.E, m0);
    t.valid = 1;
    t.a_row = m0; t.a_k0 = 0;
    t.nk = (red + kBK - 1) / kBK;
    if (p.mode == 0) { t.b_row = e * p.N + nb * p.bn; t.b_k0 = 0; }       // rows of the stacked weight
    else { t.b_row = nb * p.bn; t.b_k0 = e * p.N; }                        // MN-major: columns, then the expert's rows
  } else {
    const int m_tiles = (p.N + kBM - 1) / kBM, n_tiles = (p.K + p.bn - 1) / p.bn;
    const int per = m_tiles * n_tiles;
    const int e = w / per, r = w % per;
    const int mb = r / n_tiles, nb = r % n_tiles;
    const int lo = __ldg(p.off + e), hi = __ldg(p.off + e + 1);
    if (hi <= lo) return t;
    t.valid = 1;
    t.a_row = mb * kBM; t.a_k0 = lo;
    t.b_row = nb * p.bn; t.b_k0 = lo;
    t.nk = (hi - lo + kBK - 1) / kBK;
    t.out_row = mb * kBM; t.out_col = nb * p.bn;
    t.out_base = static_cast<long long>(e) * p.N * p.ldd;
  }
  return t;
}

__device__ __forceinline__ int group_total(const GroupedParams& p) {
  if (p.mode < 2) return (p.rows_cap / kBM) * (((p.mode == 0 ? p.N : p.K) + p.bn - 1) / p.bn);
  return p.E * ((p.N + kBM - 1) / kBM) * ((p.K + p.bn - 1) / p.bn);
}

__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GroupedParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
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
  // operand majors: mode 0 both K-major; mode 1 A K-major, B MN-major; mode 2 both MN-major
  const int a_mn = p.mode == 2, b_mn = p.mode >= 1;

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
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total = group_total(p);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
        const GroupTile t = group_tile(p, w);
        if (!t.valid) continue;
        for (int kb = 0; kb < t.nk; ++kb, ++it) {
          const int s = it % p.stages;
          const uint32_t ph = (it / p.stages) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, kTimeoutProducer)) { ok = false; break; }
          uint8_t* sa = smem + s * stage_bytes;
          uint8_t* sb = sa + a_bytes;
          mbar_expect_tx(&full_bar[s], a_bytes + b_bytes);
          load_operand(sa, &map_a, &full_bar[s], a_mn, kBM, t.a_row, t.a_k0 + kb * kBK);
          load_operand(sb, &map_b, &full_bar[s], b_mn, p.bn, t.b_row, t.b_k0 + kb * kBK);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      const uint32_t idesc = make_idesc_bf16(p.bn, a_mn, b_mn);
      const uint32_t astep = a_mn ? 128u : 2u, bstep = b_mn ? 128u : 2u;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
        const GroupTile t = group_tile(p, w);
        if (!t.valid) continue;
        const int buf = acc_it & 1;
        const uint32_t aph = (acc_it >> 1) & 1;
        if (!mbar_wait(&tempty_bar[buf], aph ^ 1, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * p.bn;
        const int red = p.mode == 0 ? p.K : p.N;      // modes 0/1: the last block may be partial (zero-filled by TMA)
        uint32_t accumulate = 0;
        for (int kb = 0; kb < t.nk; ++kb, ++it) {
          const int s = it % p.stages;
          const uint32_t ph = (it / p.stages) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * stage_bytes);
          const uint32_t sb = sa + a_bytes;
          int nmma = 4;
          if (p.mode < 2) nmma = min(4, (red - kb * kBK + 15) / 16);
          const uint64_t da = make_smem_desc(sa, a_mn ? 8192u : 16u, 1024u);
          const uint64_t db = make_smem_desc(sb, b_mn ? 8192u : 16u, 1024u);
          for (int j = 0; j < nmma; ++j) {
            umma_f16(d_tmem, da + static_cast<uint64_t>(astep * j), db + static_cast<uint64_t>(bstep * j), idesc,
                     accumulate);
            accumulate = 1;
          }
          umma_commit(&empty_bar[s]);
        }
        if (ok) umma_commit(&tfull_bar[buf]);
        ++acc_it;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;
    uint32_t acc_it = 0;
    bool ok = true;
    const int out_rows = p.mode == 2 ? p.N : p.rows_cap;
    const int out_cols = p.mode == 0 ? p.N : p.K;
    for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
      const GroupTile t = group_tile(p, w);
      if (!t.valid) {
        if (p.mode < 2) {      // rows past the last expert's slab hold nothing: write zeros so the buffer is defined
          const int row = t.out_row + q * 32 + lane;
          if (row < out_rows) {
            __nv_bfloat16* drow = static_cast<__nv_bfloat16*>(p.D) + static_cast<size_t>(row) * p.ldd;
            for (int c = t.out_col; c < min(t.out_col + p.bn, out_cols); c += 8)
              *reinterpret_cast<uint4*>(drow + c) = make_uint4(0u, 0u, 0u, 0u);
          }
        }
        continue;
      }
      const int buf = acc_it & 1;
      const uint32_t aph = (acc_it >> 1) & 1;
      if (!mbar_wait(&tfull_bar[buf], aph, abort_flag, p.status, kTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after();
      const int row = t.out_row + q * 32 + lane;
      const bool row_ok = row < out_rows;
      for (int c = 0; c < p.bn / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + buf * p.bn + c * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
        tmem_ld_wait();
        const int col0 = t.out_col + c * 32;
        if (!row_ok || col0 >= out_cols) continue;
        if (p.mode < 2) {
          __nv_bfloat16* drow = static_cast<__nv_bfloat16*>(p.D) + static_cast<size_t>(row) * p.ldd + col0;
          if (col0 + 32 <= out_cols) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[v * 8]) * p.alpha, __uint_as_float(r[v * 8 + 1]) * p.alpha);
              o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]) * p.alpha, __uint_as_float(r[v * 8 + 3]) * p.alpha);
              o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]) * p.alpha, __uint_as_float(r[v * 8 + 5]) * p.alpha);
              o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]) * p.alpha, __uint_as_float(r[v * 8 + 7]) * p.alpha);
              *reinterpret_cast<uint4*>(drow + v * 8) = o;
            }
          } else {
            for (int e = 0; e < 32 && col0 + e < out_cols; ++e)
              drow[e] = __float2bfloat16(__uint_as_float(r[e]) * p.alpha);
          }
        } else {
          float* drow = static_cast<float*>(p.D) + t.out_base + static_cast<size_t>(row) * p.ldd + col0;
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            if (col0 + e < out_cols) {
              const float val = __uint_as_float(r[e]) * p.alpha;
              drow[e] = p.accumulate ? drow[e] + val : val;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      ++acc_it;
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
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

// ------------------------------------------------------------------------------------------------ few rows per expert
// Decode and verification steps give every expert a handful of rows, so a 128-row token tile would be nearly all
// padding and its MMAs would cost as much as a full tile. Here the operands trade places: the A tile is 128 rows of the
// expert's weight, the B tile is `bn` token rows (32, 64 or 128), and the accumulator holds Y^T (weight row in the TMEM
// lane, token in the column). The MMA cost then scales with the token count, the slabs need no padding (a B tile may run
// into the next expert's rows or past the buffer: those columns are never stored), and the kernel is a pure stream of the
// weights of the experts that have rows.
//   plain   Y[r, :] = X[r, :] W_e^T                           W stacked [E*N, K]
//   swiglu  Y[r, :] = silu(X[r, :] G_e^T) * (X[r, :] U_e^T)   W stacked [E*2N, K], rows [G_e (N rows); U_e (N rows)] per
//           expert; the A tile is 64 rows of G_e on top of the same 64 rows of U_e, and the two halves meet in shared
//           memory in the epilogue
struct SkinnyParams {
  int E, N, K, bn, swiglu;
  int stages, tmem_cols;
  const int* off;        // [E + 1] row offsets (no alignment)
  __nv_bfloat16* D;
  int ldd;
  float alpha;
  int* status;
};

__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                           const SkinnyParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
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
  uint64_t* xfull_bar = reinterpret_cast<uint64_t*>(tmem_slot + 2);      // exchange buffer filled (2 arrivals)
  uint64_t* xfree_bar = xfull_bar + 1;                                   // exchange buffer read (2 arrivals)
  float* xch = reinterpret_cast<float*>(smem + p.stages * stage_bytes + 256);      // [64][bn + 1] up-projection values

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
    mbar_init(xfull_bar, 2);
    mbar_init(xfree_bar, 2);
    *abort_flag = 0;
    mbar_init_fence();
    tma_prefetch_desc(&map_w);
    tma_prefetch_desc(&map_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int rows_per_tile = p.swiglu ? 64 : kBM;                 // output channels per work item
  const int n_tiles = (p.N + rows_per_tile - 1) / rows_per_tile;
  const int total = p.E * n_tiles;
  const int nk = (p.K + kBK - 1) / kBK;
  const int w_rows = p.swiglu ? 2 * p.N : p.N;                   // weight rows per expert

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
        const int e = w / n_tiles, nb = w % n_tiles;
        const int lo = __ldg(p.off + e), cnt = __ldg(p.off + e + 1) - lo;
        for (int t0 = 0; t0 < cnt && ok; t0 += p.bn) {
          for (int kb = 0; kb < nk; ++kb, ++it) {
            const int s = it % p.stages;
            const uint32_t ph = (it / p.stages) & 1;
            if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, kTimeoutProducer)) { ok = false; break; }
            uint8_t* sa = smem + s * stage_bytes;
            mbar_expect_tx(&full_bar[s], a_bytes + b_bytes);
            if (p.swiglu) {       // two 64-row boxes: gate rows, then the up rows of the same channels
              tma_load_2d(sa, &map_w, &full_bar[s], kb * kBK, e * w_rows + nb * 64);
              tma_load_2d(sa + 8192, &map_w, &full_bar[s], kb * kBK, e * w_rows + p.N + nb * 64);
            } else {
              tma_load_2d(sa, &map_w, &full_bar[s], kb * kBK, e * w_rows + nb * kBM);
            }
            tma_load_2d(sa + a_bytes, &map_x, &full_bar[s], kb * kBK, lo + t0);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      const uint32_t idesc = make_idesc_bf16(p.bn, 0, 0);
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
        const int e = w / n_tiles;
        const int cnt = __ldg(p.off + e + 1) - __ldg(p.off + e);
        for (int t0 = 0; t0 < cnt && ok; t0 += p.bn) {
          const int buf = acc_it & 1;
          const uint32_t aph = (acc_it >> 1) & 1;
          if (!mbar_wait(&tempty_bar[buf], aph ^ 1, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * p.bn;
          uint32_t accumulate = 0;
          for (int kb = 0; kb < nk; ++kb, ++it) {
            const int s = it % p.stages;
            const uint32_t ph = (it / p.stages) & 1;
            if (!mbar_wait(&full_bar[s], ph, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + s * stage_bytes);
            const int nmma = min(4, (p.K - kb * kBK + 15) / 16);
            const uint64_t da = make_smem_desc(sa, 16u, 1024u);
            const uint64_t db = make_smem_desc(sa + a_bytes, 16u, 1024u);
            for (int j = 0; j < nmma; ++j) {
              umma_f16(d_tmem, da + static_cast<uint64_t>(2u * j), db + static_cast<uint64_t>(2u * j), idesc, accumulate);
              accumulate = 1;
            }
            umma_commit(&empty_bar[s]);
          }
          if (ok) umma_commit(&tfull_bar[buf]);
          ++acc_it;
        }
      }
    }
  } else {
    const int q = warp & 3;          // TMEM lane quarter: lanes 32 q .. 32 q + 31
    uint32_t acc_it = 0;
    bool ok = true;
    const int ldx = p.bn + 1;
    for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
      const int e = w / n_tiles, nb = w % n_tiles;
      const int lo = __ldg(p.off + e), cnt = __ldg(p.off + e + 1) - lo;
      for (int t0 = 0; t0 < cnt && ok; t0 += p.bn) {
        const int buf = acc_it & 1;
        const uint32_t aph = (acc_it >> 1) & 1;
        if (!mbar_wait(&tfull_bar[buf], aph, abort_flag, p.status, kTimeoutEpilogue)) { ok = false; break; }
        tc_fence_after();
        const int live = min(p.bn, cnt - t0);                    // token columns that hold rows of this expert
        if (!p.swiglu) {
          const int n = nb * kBM + q * 32 + lane;
          for (int c = 0; c * 32 < live; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(tmem_base + buf * p.bn + c * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
            tmem_ld_wait();
            if (n < p.N) {
              __nv_bfloat16* d = p.D + static_cast<size_t>(lo + t0 + c * 32) * p.ldd + n;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (c * 32 + j < live) d[static_cast<size_t>(j) * p.ldd] = __float2bfloat16(__uint_as_float(r[j]) * p.alpha);
            }
          }
        } else {
          // lanes 0..63 hold the gate projection, lanes 64..127 the up projection of the same 64 channels: the two
          // warps of the upper half park their values in shared memory, the two of the lower half combine and store
          const bool upper = q >= 2;
          const int ch = (q & 1) * 32 + lane;                    // channel within the tile
          const int n = nb * 64 + ch;
          const uint32_t xph = acc_it & 1;
          if (upper) {
            if (!mbar_wait(xfree_bar, xph ^ 1, abort_flag, p.status, kTimeoutEpilogue)) { ok = false; break; }
            for (int c = 0; c * 32 < live; ++c) {
              uint32_t r[32];
              tmem_ld_32x32b_x32(tmem_base + buf * p.bn + c * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j) xch[ch * ldx + c * 32 + j] = __uint_as_float(r[j]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(xfull_bar);
          } else {
            bool have = false;
            for (int c = 0; c * 32 < live; ++c) {
              uint32_t r[32];
              tmem_ld_32x32b_x32(tmem_base + buf * p.bn + c * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
              tmem_ld_wait();
              if (!have) {
                if (!mbar_wait(xfull_bar, xph, abort_flag, p.status, kTimeoutEpilogue)) { ok = false; break; }
                have = true;
              }
              if (n < p.N) {
                __nv_bfloat16* d = p.D + static_cast<size_t>(lo + t0 + c * 32) * p.ldd + n;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  if (c * 32 + j < live) {
                    const float g = __uint_as_float(r[j]) * p.alpha, u = xch[ch * ldx + c * 32 + j] * p.alpha;
                    d[static_cast<size_t>(j) * p.ldd] = __float2bfloat16(g / (1.f + __expf(-g)) * u);
                  }
                }
              }
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(xfree_bar);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[buf]);
        ++acc_it;
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
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

}  // namespace pm

using namespace pm;

// a, b: the two operands of the mode (see the table at the top); both bf16, row strides lda / ldb in elements.
// off: int32 [E + 1] on the device, multiples of 128, off[E] <= rows_cap. D: bf16 [rows_cap, ldd] (modes 0, 1) or fp32
// [E, N, ldd] (mode 2; experts without rows are left untouched, so clear D first unless accumulating).
extern "C" int pm_grouped_gemm(int mode, const void* a, int lda, const void* b, int ldb, void* D, int ldd, const int* off,
                               int E, int rows_cap, int N, int K, float alpha, int accumulate, int* status,
                               cudaStream_t stream) {
  if (mode < 0 || mode > 2 || E < 1 || rows_cap <= 0 || (rows_cap % kBM) || N <= 0 || K <= 0) return -1;
  if ((N % 8) || (K % 8) || (ldd % 8 && mode < 2)) return -2;
  GroupedParams p{};
  p.mode = mode; p.E = E; p.rows_cap = rows_cap; p.N = N; p.K = K;
  p.off = off; p.D = D; p.ldd = ldd; p.accumulate = accumulate; p.alpha = alpha; p.status = status;
  const int out_cols = mode == 0 ? N : K;
  int bn = 256;
  while (bn > 64 && bn / 2 >= out_cols) bn /= 2;
  p.bn = bn;
  const int stage_bytes = kBM * kBK * 2 + bn * kBK * 2;
  int stages = (227 * 1024 - 2048) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  p.stages = stages;
  int cols = 32;
  while (cols < 2 * bn) cols *= 2;
  p.tmem_cols = cols;
  CUtensorMap ma, mb;
  int rc;
  if (mode == 0) {          // X [rows_cap, K] K-major; W [E*N, K] K-major
    if ((rc = operand_map(&ma, a, 0, rows_cap, K, lda, kBM))) return rc * 10 - 1;
    if ((rc = operand_map(&mb, b, 0, E * N, K, ldb, bn))) return rc * 10 - 2;
  } else if (mode == 1) {   // dY [rows_cap, N] K-major (reduction over N); W [E*N, K]: reduction rows, K contiguous
    if ((rc = operand_map(&ma, a, 0, rows_cap, N, lda, kBM))) return rc * 10 - 1;
    if ((rc = operand_map(&mb, b, 1, K, E * N, ldb, bn))) return rc * 10 - 2;
  } else {                  // dY [rows_cap, N] and X [rows_cap, K], both with the token index as the reduction
    if ((rc = operand_map(&ma, a, 1, N, rows_cap, lda, kBM))) return rc * 10 - 1;
    if ((rc = operand_map(&mb, b, 1, K, rows_cap, ldb, bn))) return rc * 10 - 2;
  }
  const size_t smem = static_cast<size_t>(stages) * stage_bytes + 1024 + 256;
  static DeviceOnce configured;
  if (configured.pending()) {
    cudaError_t e = cudaFuncSetAttribute(grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured.mark();
  }
  long long total = mode < 2 ? static_cast<long long>(rows_cap / kBM) * ((out_cols + bn - 1) / bn)
                             : static_cast<long long>(E) * ((N + kBM - 1) / kBM) * ((K + bn - 1) / bn);
  int grid = num_sms();
  if (total < grid) grid = static_cast<int>(total);
  grouped_gemm_kernel<<<grid, kThreads, smem, stream>>>(ma, mb, p);
  return static_cast<int>(cudaGetLastError());
}

// Few rows per expert (see the kernel): x [rows, K] expert-sorted with offsets off [E + 1] (any alignment), w stacked
// [E * N, K] (swiglu 0) or [E * 2N, K] with gate rows above up rows per expert (swiglu 1); y [rows, N] bf16.
// bn (32, 64, 128) is the token tile: experts with more rows take several passes over their weights.
extern "C" int pm_grouped_gemm_skinny(const void* x, int ldx, int rows, const void* w, int ldw, void* y, int ldy,
                                      const int* off, int E, int N, int K, int bn, int swiglu, float alpha, int* status,
                                      cudaStream_t stream) {
  if (E < 1 || rows <= 0 || N <= 0 || K <= 0 || (K % 8) || (ldx % 8) || (ldw % 8)) return -1;
  if (bn != 32 && bn != 64 && bn != 128) return -2;
  SkinnyParams p{};
  p.E = E; p.N = N; p.K = K; p.bn = bn; p.swiglu = swiglu ? 1 : 0;
  p.off = off; p.D = static_cast<__nv_bfloat16*>(y); p.ldd = ldy; p.alpha = alpha; p.status = status;
  const int stage_bytes = kBM * kBK * 2 + bn * kBK * 2;
  const int xch_bytes = swiglu ? 64 * (bn + 1) * 4 : 0;
  int stages = (227 * 1024 - 2048 - xch_bytes) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  p.stages = stages;
  int cols = 32;
  while (cols < 2 * bn) cols *= 2;
  p.tmem_cols = cols;
  CUtensorMap mw, mx;
  int rc;
  const long long w_rows = static_cast<long long>(E) * (swiglu ? 2 * N : N);
  if (w_rows > 0x7fffffff) return -3;
  if ((rc = operand_map(&mw, w, 0, static_cast<int>(w_rows), K, ldw, swiglu ? 64 : kBM))) return rc * 10 - 1;
  if ((rc = operand_map(&mx, x, 0, rows, K, ldx, bn))) return rc * 10 - 2;
  const size_t smem = static_cast<size_t>(stages) * stage_bytes + 1024 + 256 + xch_bytes;
  static DeviceOnce configured;
  if (configured.pending()) {
    cudaError_t e = cudaFuncSetAttribute(grouped_gemm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured.mark();
  }
  const long long total = static_cast<long long>(E) * ((N + (swiglu ? 64 : kBM) - 1) / (swiglu ? 64 : kBM));
  int grid = num_sms();
  if (total < grid) grid = static_cast<int>(total);
  grouped_gemm_skinny_kernel<<<grid, kThreads, smem, stream>>>(mw, mx, p);
  return static_cast<int>(cudaGetLastError());
}
