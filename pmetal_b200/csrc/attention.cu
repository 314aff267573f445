// Varlen (packed-sequence) causal flash attention, forward and backward, head_dim 128, GQA.
//
// The token stream is a concatenation of documents; `seq_start[t]` is the index of the first
// token of the document that token t belongs to. Query i may attend key j iff
// seq_start[i] <= j <= i (and i - j < window when a sliding window is set), i.e. a
// block-diagonal causal mask that is never materialised. The reference has a varlen forward
// only (flash_attention_varlen_forward_d128, crates/pmetal-metal/src/kernels/metal/
// flash_attention.metal:1093-1130) and falls back to a dense [T,T] mask for packed training;
// here forward, dQ and dK/dV all work from the boundaries.
//
// Tiles are 64 queries x 64 keys, 4 warps per CTA, mma.sync.m16n8k16 bf16 with fp32 accumulation,
// online softmax in base 2, K/V (or Q/dO) tiles double-buffered with cp.async, shared memory rows
// XOR-swizzled in 16-byte chunks. The backward is two kernels, both deterministic:
//   dQ  : one CTA per (query tile, head), loops over key tiles (recomputes S and dP)
//   dKV : one CTA per (key tile, kv head), loops over the query heads of the group and query tiles
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "host_util.cuh"

#include "pdl.cuh"
#include "pmetal_b200.h"

namespace pm {

constexpr int kD = 128;     // head dim
constexpr int kTile = 64;   // rows per tile (queries or keys)
constexpr int kAttnThreads = 128;
constexpr int kTileBytes = kTile * kD * 2;   // 16 KB
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// byte offset of element (row, col) in a swizzled [rows][128] bf16 tile
__device__ __forceinline__ uint32_t sw_off(int row, int col) {
  return static_cast<uint32_t>(row * 256 + ((((col >> 3) ^ (row & 7)) << 4) | ((col & 7) << 1)));
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Copy a [64][128] bf16 tile (rows row0.., clamped to < T) from a strided global tensor into swizzled smem.
__device__ __forceinline__ void load_tile(uint8_t* smem_tile, const __nv_bfloat16* base, long long row_stride, int row0,
                                          int T) {
  const uint32_t sbase = smem_addr(smem_tile);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int idx = threadIdx.x + i * kAttnThreads;   // 0..1023
    const int r = idx >> 4, c = idx & 15;
    int gr = row0 + r;
    gr = gr < T ? gr : T - 1;
    cp_async16(sbase + r * 256 + ((c ^ (r & 7)) << 4), base + static_cast<long long>(gr) * row_stride + c * 8);
  }
}

// A-operand fragments (16 rows x 16 k) of a row-major swizzled tile: rows r0.., k columns k0..
__device__ __forceinline__ void load_a_frag(uint32_t tile, int r0, int k0, int lane, uint32_t (&a)[4]) {
  const int row = r0 + (lane & 15), col = k0 + ((lane >> 4) << 3);
  ldsm_x4(tile + sw_off(row, col), a[0], a[1], a[2], a[3]);
}
// B-operand fragments for C = A * X^T where X is a row-major tile [n][k]: two n-tiles (n0, n0+8), k0..k0+15.
__device__ __forceinline__ void load_b_frag_nt(uint32_t tile, int n0, int k0, int lane, uint32_t (&b)[4]) {
  const int id = lane >> 3, r = lane & 7;
  const int row = n0 + ((id >> 1) << 3) + r, col = k0 + ((id & 1) << 3);
  ldsm_x4(tile + sw_off(row, col), b[0], b[1], b[2], b[3]);
}
// B-operand fragments for C = A * X where X is a row-major tile [k][n]: two n-tiles (n0, n0+8), k0..k0+15.
__device__ __forceinline__ void load_b_frag_nn(uint32_t tile, int k0, int n0, int lane, uint32_t (&b)[4]) {
  const int id = lane >> 3, r = lane & 7;
  const int row = k0 + ((id & 1) << 3) + r, col = n0 + ((id >> 1) << 3);
  ldsm_x4_t(tile + sw_off(row, col), b[0], b[1], b[2], b[3]);
}

struct AttnParams {
  const __nv_bfloat16 *q, *k, *v, *o, *dout;
  __nv_bfloat16 *out, *dq, *dk, *dv;
  long long q_stride, k_stride, v_stride, o_stride, dq_stride, dk_stride, dv_stride;   // per-token strides (elements)
  const int* seq_start;
  float* lse;          // [Hq][T], natural log
  const float* delta;  // [Hq][T]
  int T, hq, hkv;
  float scale;
  int window;
};

// ================================================================================= forward
__global__ void __launch_bounds__(kAttnThreads) attn_fwd_kernel(const AttnParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kTileBytes;               // 2 buffers
  uint8_t* sV = smem + 3 * kTileBytes;           // 2 buffers
  int* sStart = reinterpret_cast<int*>(smem + 5 * kTileBytes);

  const int qt = gridDim.x - 1 - blockIdx.x;     // longest (latest) tiles first
  const int h = blockIdx.y;
  const int hk = h / (p.hq / p.hkv);
  const int q0 = qt * kTile;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;

  if (threadIdx.x < kTile) {
    const int i = q0 + threadIdx.x;
    sStart[threadIdx.x] = p.seq_start[i < p.T ? i : p.T - 1];
  }
  const int first_start = p.seq_start[q0];
  int kv_lo = first_start;
  if (p.window > 0) kv_lo = max(kv_lo, q0 - p.window + 1);
  kv_lo = (kv_lo / kTile) * kTile;
  const int kv_hi = min(q0 + kTile, p.T);
  const int n_tiles = (kv_hi - kv_lo + kTile - 1) / kTile;

  const __nv_bfloat16* qb = p.q + static_cast<long long>(h) * kD;
  const __nv_bfloat16* kb = p.k + static_cast<long long>(hk) * kD;
  const __nv_bfloat16* vb = p.v + static_cast<long long>(hk) * kD;

  load_tile(sQ, qb, p.q_stride, q0, p.T);
  load_tile(sK, kb, p.k_stride, kv_lo, p.T);
  load_tile(sV, vb, p.v_stride, kv_lo, p.T);
  cp_async_commit();

  float o_acc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float sl2 = p.scale * kLog2e;
  const uint32_t q_tile = smem_addr(sQ);

  for (int it = 0; it < n_tiles; ++it) {
    const int buf = it & 1;
    const int j0 = kv_lo + it * kTile;
    if (it + 1 < n_tiles) {
      load_tile(sK + (buf ^ 1) * kTileBytes, kb, p.k_stride, j0 + kTile, p.T);
      load_tile(sV + (buf ^ 1) * kTileBytes, vb, p.v_stride, j0 + kTile, p.T);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t k_tile = smem_addr(sK + buf * kTileBytes);
    const uint32_t v_tile = smem_addr(sV + buf * kTileBytes);

    // S = Q K^T  (16 x 64 per warp)
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      uint32_t a[4];
      load_a_frag(q_tile, warp * 16, kk * 16, lane, a);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        load_b_frag_nt(k_tile, np * 16, kk * 16, lane, b);
        mma_bf16(s[2 * np], a[0], a[1], a[2], a[3], b[0], b[1]);
        mma_bf16(s[2 * np + 1], a[0], a[1], a[2], a[3], b[2], b[3]);
      }
    }
    // mask + online softmax. Thread holds rows r0 = warp*16+g and r0+8, columns nt*8 + 2*t4 + {0,1}.
    const int r_lo = warp * 16 + g;
    const int i_lo = q0 + r_lo, i_hi = i_lo + 8;
    const int st_lo = sStart[r_lo], st_hi = sStart[r_lo + 8];
    const bool need_mask = (j0 + kTile - 1 > q0) || (j0 < sStart[kTile - 1]) ||
                           (p.window > 0 && j0 < q0 + kTile - p.window);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[nt][e] * sl2;
        if (need_mask) {
          const int j = j0 + nt * 8 + 2 * t4 + (e & 1);
          const int i = (e < 2) ? i_lo : i_hi;
          const int st = (e < 2) ? st_lo : st_hi;
          bool ok = (j <= i) && (j >= st);
          if (p.window > 0) ok = ok && (i - j < p.window);
          if (!ok) v = -INFINITY;
        }
        s[nt][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
      corr[r] = (m_run[r] == -INFINITY) ? 0.f : exp2f(m_run[r] - m_use[r]);
      m_run[r] = m_new;
      l_run[r] *= corr[r];
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = exp2f(s[nt][e] - m_use[e >> 1]);
        s[nt][e] = pv;
        rs[e >> 1] += pv;
      }
    }
    l_run[0] += rs[0];
    l_run[1] += rs[1];
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      o_acc[nt][0] *= corr[0];
      o_acc[nt][1] *= corr[0];
      o_acc[nt][2] *= corr[1];
      o_acc[nt][3] *= corr[1];
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const uint32_t a0 = pack2(s[2 * kk][0], s[2 * kk][1]);
      const uint32_t a1 = pack2(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t a2 = pack2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      const uint32_t a3 = pack2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        uint32_t b[4];
        load_b_frag_nn(v_tile, kk * 16, np * 16, lane, b);
        mma_bf16(o_acc[2 * np], a0, a1, a2, a3, b[0], b[1]);
        mma_bf16(o_acc[2 * np + 1], a0, a1, a2, a3, b[2], b[3]);
      }
    }
    __syncthreads();   // all warps done with this K/V buffer before it is refilled
  }

  // finalise: divide by the row sum, write O and LSE
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  const int r_lo = warp * 16 + g;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int i = q0 + r_lo + r * 8;
    if (i >= p.T) continue;
    const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
    __nv_bfloat16* orow = p.out + static_cast<long long>(i) * p.o_stride + static_cast<long long>(h) * kD;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      *reinterpret_cast<uint32_t*>(orow + nt * 8 + 2 * t4) =
          pack2(o_acc[nt][2 * r] * inv, o_acc[nt][2 * r + 1] * inv);
    }
    if (t4 == 0) p.lse[static_cast<long long>(h) * p.T + i] = (m_run[r] + log2f(l_run[r])) / kLog2e;
  }
}

// ================================================================================= backward: dQ
// Same tiling as the forward. P = exp2(S*scale*log2e - lse*log2e); dP = dO V^T; dS = P (dP - delta) scale;
// dQ = sum_j dS K.
__global__ void __launch_bounds__(kAttnThreads) attn_bwd_dq_kernel(const AttnParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sdO = smem + kTileBytes;
  uint8_t* sK = smem + 2 * kTileBytes;   // 2 buffers
  uint8_t* sV = smem + 4 * kTileBytes;   // 2 buffers
  int* sStart = reinterpret_cast<int*>(smem + 6 * kTileBytes);

  const int qt = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y;
  const int hk = h / (p.hq / p.hkv);
  const int q0 = qt * kTile;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;

  if (threadIdx.x < kTile) {
    const int i = q0 + threadIdx.x;
    sStart[threadIdx.x] = p.seq_start[i < p.T ? i : p.T - 1];
  }
  int kv_lo = p.seq_start[q0];
  if (p.window > 0) kv_lo = max(kv_lo, q0 - p.window + 1);
  kv_lo = (kv_lo / kTile) * kTile;
  const int kv_hi = min(q0 + kTile, p.T);
  const int n_tiles = (kv_hi - kv_lo + kTile - 1) / kTile;

  const __nv_bfloat16* kb = p.k + static_cast<long long>(hk) * kD;
  const __nv_bfloat16* vb = p.v + static_cast<long long>(hk) * kD;
  load_tile(sQ, p.q + static_cast<long long>(h) * kD, p.q_stride, q0, p.T);
  load_tile(sdO, p.dout + static_cast<long long>(h) * kD, p.o_stride, q0, p.T);
  load_tile(sK, kb, p.k_stride, kv_lo, p.T);
  load_tile(sV, vb, p.v_stride, kv_lo, p.T);
  cp_async_commit();

  const int r_lo = warp * 16 + g;
  const int i_lo = q0 + r_lo, i_hi = i_lo + 8;
  const int ic_lo = min(i_lo, p.T - 1), ic_hi = min(i_hi, p.T - 1);
  const float lse2[2] = {p.lse[static_cast<long long>(h) * p.T + ic_lo] * kLog2e,
                         p.lse[static_cast<long long>(h) * p.T + ic_hi] * kLog2e};
  const float dl[2] = {p.delta[static_cast<long long>(h) * p.T + ic_lo],
                       p.delta[static_cast<long long>(h) * p.T + ic_hi]};
  const float sl2 = p.scale * kLog2e;

  float dq_acc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) dq_acc[i][j] = 0.f;
  const uint32_t q_tile = smem_addr(sQ), do_tile = smem_addr(sdO);

  for (int it = 0; it < n_tiles; ++it) {
    const int buf = it & 1;
    const int j0 = kv_lo + it * kTile;
    if (it + 1 < n_tiles) {
      load_tile(sK + (buf ^ 1) * kTileBytes, kb, p.k_stride, j0 + kTile, p.T);
      load_tile(sV + (buf ^ 1) * kTileBytes, vb, p.v_stride, j0 + kTile, p.T);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t k_tile = smem_addr(sK + buf * kTileBytes);
    const uint32_t v_tile = smem_addr(sV + buf * kTileBytes);

    float s[8][4], dp[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) { s[i][j] = 0.f; dp[i][j] = 0.f; }
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      uint32_t a[4], ad[4];
      load_a_frag(q_tile, warp * 16, kk * 16, lane, a);
      load_a_frag(do_tile, warp * 16, kk * 16, lane, ad);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        load_b_frag_nt(k_tile, np * 16, kk * 16, lane, b);
        mma_bf16(s[2 * np], a[0], a[1], a[2], a[3], b[0], b[1]);
        mma_bf16(s[2 * np + 1], a[0], a[1], a[2], a[3], b[2], b[3]);
        load_b_frag_nt(v_tile, np * 16, kk * 16, lane, b);
        mma_bf16(dp[2 * np], ad[0], ad[1], ad[2], ad[3], b[0], b[1]);
        mma_bf16(dp[2 * np + 1], ad[0], ad[1], ad[2], ad[3], b[2], b[3]);
      }
    }
    const int st_lo = sStart[r_lo], st_hi = sStart[r_lo + 8];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + nt * 8 + 2 * t4 + (e & 1);
        const int i = (e < 2) ? i_lo : i_hi;
        const int st = (e < 2) ? st_lo : st_hi;
        bool ok = (j <= i) && (j >= st) && (i < p.T);
        if (p.window > 0) ok = ok && (i - j < p.window);
        const float pv = ok ? exp2f(s[nt][e] * sl2 - lse2[e >> 1]) : 0.f;
        s[nt][e] = pv * (dp[nt][e] - dl[e >> 1]) * p.scale;   // dS
      }
    }
    // dQ += dS K
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const uint32_t a0 = pack2(s[2 * kk][0], s[2 * kk][1]);
      const uint32_t a1 = pack2(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t a2 = pack2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      const uint32_t a3 = pack2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        uint32_t b[4];
        load_b_frag_nn(k_tile, kk * 16, np * 16, lane, b);
        mma_bf16(dq_acc[2 * np], a0, a1, a2, a3, b[0], b[1]);
        mma_bf16(dq_acc[2 * np + 1], a0, a1, a2, a3, b[2], b[3]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int i = q0 + r_lo + r * 8;
    if (i >= p.T) continue;
    __nv_bfloat16* drow = p.dq + static_cast<long long>(i) * p.dq_stride + static_cast<long long>(h) * kD;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt)
      *reinterpret_cast<uint32_t*>(drow + nt * 8 + 2 * t4) = pack2(dq_acc[nt][2 * r], dq_acc[nt][2 * r + 1]);
  }
}

// ================================================================================= backward: dK, dV
// One CTA per (key tile, kv head). Works on the transposed score tile S^T = K Q^T so that each warp owns
// 16 key rows and accumulates dV += P^T dO and dK += dS^T Q in registers over every query tile that can
// see these keys and every query head of the GQA group.
__global__ void __launch_bounds__(kAttnThreads) attn_bwd_dkv_kernel(const AttnParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sK = smem;
  uint8_t* sV = smem + kTileBytes;
  uint8_t* sQ = smem + 2 * kTileBytes;    // 2 buffers
  uint8_t* sdO = smem + 4 * kTileBytes;   // 2 buffers
  float* sLse = reinterpret_cast<float*>(smem + 6 * kTileBytes);   // [2][64]
  float* sDelta = sLse + 2 * kTile;                                 // [2][64]
  int* sStart = reinterpret_cast<int*>(sDelta + 2 * kTile);         // [2][64]

  const int jt = blockIdx.x;
  const int hk = blockIdx.y;
  const int rep = p.hq / p.hkv;
  const int j0 = jt * kTile;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int j_last = min(j0 + kTile, p.T) - 1;

  // query tiles m0 = j0, j0+64, ... while the tile's first row belongs to a document that started at or
  // before the last key of this tile (later tiles cannot see these keys)
  int n_q_tiles = 0;
  for (bool done = false; !done;) {
    const int m0 = j0 + (n_q_tiles + lane) * kTile;
    bool ok = m0 < p.T;
    if (ok) ok = p.seq_start[m0] <= j_last && !(p.window > 0 && m0 - j_last >= p.window);
    const unsigned b = __ballot_sync(0xffffffffu, ok);
    const int cnt = (b == 0xffffffffu) ? 32 : (__ffs(~b) - 1);
    n_q_tiles += cnt;
    done = cnt < 32;
  }
  const int total = n_q_tiles * rep;

  load_tile(sK, p.k + static_cast<long long>(hk) * kD, p.k_stride, j0, p.T);
  load_tile(sV, p.v + static_cast<long long>(hk) * kD, p.v_stride, j0, p.T);

  auto issue = [&](int w, int buf) {
    const int hh = hk * rep + (w / n_q_tiles);
    const int m0 = j0 + (w % n_q_tiles) * kTile;
    load_tile(sQ + buf * kTileBytes, p.q + static_cast<long long>(hh) * kD, p.q_stride, m0, p.T);
    load_tile(sdO + buf * kTileBytes, p.dout + static_cast<long long>(hh) * kD, p.o_stride, m0, p.T);
    if (threadIdx.x < kTile) {
      const int i = min(m0 + static_cast<int>(threadIdx.x), p.T - 1);
      sLse[buf * kTile + threadIdx.x] = p.lse[static_cast<long long>(hh) * p.T + i] * kLog2e;
      sDelta[buf * kTile + threadIdx.x] = p.delta[static_cast<long long>(hh) * p.T + i];
      sStart[buf * kTile + threadIdx.x] = p.seq_start[i];
    }
  };
  if (total > 0) issue(0, 0);
  cp_async_commit();

  float dk_acc[16][4], dv_acc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) { dk_acc[i][j] = 0.f; dv_acc[i][j] = 0.f; }
  const float sl2 = p.scale * kLog2e;
  const uint32_t k_tile = smem_addr(sK), v_tile = smem_addr(sV);
  const int jr_lo = j0 + warp * 16 + g, jr_hi = jr_lo + 8;   // key rows owned by this thread

  for (int w = 0; w < total; ++w) {
    const int buf = w & 1;
    const int m0 = j0 + (w % n_q_tiles) * kTile;
    if (w + 1 < total) {
      issue(w + 1, buf ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t q_tile = smem_addr(sQ + buf * kTileBytes);
    const uint32_t do_tile = smem_addr(sdO + buf * kTileBytes);
    const float* lse2 = sLse + buf * kTile;
    const float* dl = sDelta + buf * kTile;
    const int* st = sStart + buf * kTile;

    // S^T = K Q^T and dP^T = V dO^T  (16 keys x 64 queries per warp)
    float s[8][4], dp[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) { s[i][j] = 0.f; dp[i][j] = 0.f; }
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      uint32_t a[4], av[4];
      load_a_frag(k_tile, warp * 16, kk * 16, lane, a);
      load_a_frag(v_tile, warp * 16, kk * 16, lane, av);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        load_b_frag_nt(q_tile, np * 16, kk * 16, lane, b);
        mma_bf16(s[2 * np], a[0], a[1], a[2], a[3], b[0], b[1]);
        mma_bf16(s[2 * np + 1], a[0], a[1], a[2], a[3], b[2], b[3]);
        load_b_frag_nt(do_tile, np * 16, kk * 16, lane, b);
        mma_bf16(dp[2 * np], av[0], av[1], av[2], av[3], b[0], b[1]);
        mma_bf16(dp[2 * np + 1], av[0], av[1], av[2], av[3], b[2], b[3]);
      }
    }
    // element (key row, query col): P^T and dS^T
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int c = nt * 8 + 2 * t4 + (e & 1);   // query index within tile
        const int i = m0 + c;
        const int j = (e < 2) ? jr_lo : jr_hi;
        bool ok = (j <= i) && (j >= st[c]) && (i < p.T);
        if (p.window > 0) ok = ok && (i - j < p.window);
        const float pv = ok ? exp2f(s[nt][e] * sl2 - lse2[c]) : 0.f;
        s[nt][e] = pv;                                           // P^T
        dp[nt][e] = pv * (dp[nt][e] - dl[c]) * p.scale;          // dS^T
      }
    }
    // dV += P^T dO ; dK += dS^T Q   (reduction over the 64 queries)
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const uint32_t pa0 = pack2(s[2 * kk][0], s[2 * kk][1]);
      const uint32_t pa1 = pack2(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t pa2 = pack2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      const uint32_t pa3 = pack2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
      const uint32_t sa0 = pack2(dp[2 * kk][0], dp[2 * kk][1]);
      const uint32_t sa1 = pack2(dp[2 * kk][2], dp[2 * kk][3]);
      const uint32_t sa2 = pack2(dp[2 * kk + 1][0], dp[2 * kk + 1][1]);
      const uint32_t sa3 = pack2(dp[2 * kk + 1][2], dp[2 * kk + 1][3]);
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        uint32_t b[4];
        load_b_frag_nn(do_tile, kk * 16, np * 16, lane, b);
        mma_bf16(dv_acc[2 * np], pa0, pa1, pa2, pa3, b[0], b[1]);
        mma_bf16(dv_acc[2 * np + 1], pa0, pa1, pa2, pa3, b[2], b[3]);
        load_b_frag_nn(q_tile, kk * 16, np * 16, lane, b);
        mma_bf16(dk_acc[2 * np], sa0, sa1, sa2, sa3, b[0], b[1]);
        mma_bf16(dk_acc[2 * np + 1], sa0, sa1, sa2, sa3, b[2], b[3]);
      }
    }
    __syncthreads();
  }
  if (total == 0) cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int j = j0 + warp * 16 + g + r * 8;
    if (j >= p.T) continue;
    __nv_bfloat16* krow = p.dk + static_cast<long long>(j) * p.dk_stride + static_cast<long long>(hk) * kD;
    __nv_bfloat16* vrow = p.dv + static_cast<long long>(j) * p.dv_stride + static_cast<long long>(hk) * kD;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      *reinterpret_cast<uint32_t*>(krow + nt * 8 + 2 * t4) = pack2(dk_acc[nt][2 * r], dk_acc[nt][2 * r + 1]);
      *reinterpret_cast<uint32_t*>(vrow + nt * 8 + 2 * t4) = pack2(dv_acc[nt][2 * r], dv_acc[nt][2 * r + 1]);
    }
  }
}

}  // namespace pm

using namespace pm;

static int set_smem(const void* fn, int bytes) {
  return static_cast<int>(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
}

// q:[T,hq,128] k:[T,hkv,128] v:[T,hkv,128] with per-token strides; out:[T,hq,128]; lse:[hq,T]
extern "C" int pm_attn_fwd(const void* q, long long q_stride, const void* k, long long k_stride, const void* v,
                           long long v_stride, void* out, long long o_stride, float* lse, const int* seq_start, int T,
                           int hq, int hkv, float scale, int window, cudaStream_t st) {
  if (hq % hkv || T <= 0) return -1;
  if ((q_stride | k_stride | v_stride | o_stride) % 8) return -2;
  AttnParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q); p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v); p.out = static_cast<__nv_bfloat16*>(out);
  p.q_stride = q_stride; p.k_stride = k_stride; p.v_stride = v_stride; p.o_stride = o_stride;
  p.seq_start = seq_start; p.lse = lse; p.T = T; p.hq = hq; p.hkv = hkv; p.scale = scale; p.window = window;
  const int smem = 5 * kTileBytes + 256;
  static DeviceOnce once;
  if (once.pending()) { int e = set_smem(reinterpret_cast<const void*>(attn_fwd_kernel), smem); if (e) return e; once.mark(); }
  dim3 grid((T + kTile - 1) / kTile, hq);
  attn_fwd_kernel<<<grid, kAttnThreads, smem, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

// dq:[T,hq,128] dk,dv:[T,hkv,128] (strided). delta:[hq,T] = rowsum(dO*O) computed beforehand.
extern "C" int pm_attn_bwd(const void* dout, const void* q, long long q_stride, const void* k, long long k_stride,
                           const void* v, long long v_stride, long long o_stride, const float* lse, const float* delta,
                           void* dq, long long dq_stride, void* dk, long long dk_stride, void* dv, long long dv_stride,
                           const int* seq_start, int T, int hq, int hkv, float scale, int window, cudaStream_t st) {
  if (hq % hkv || T <= 0) return -1;
  if ((q_stride | k_stride | v_stride | o_stride | dq_stride | dk_stride | dv_stride) % 8) return -2;
  AttnParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q); p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v); p.dout = static_cast<const __nv_bfloat16*>(dout);
  p.dq = static_cast<__nv_bfloat16*>(dq); p.dk = static_cast<__nv_bfloat16*>(dk); p.dv = static_cast<__nv_bfloat16*>(dv);
  p.q_stride = q_stride; p.k_stride = k_stride; p.v_stride = v_stride; p.o_stride = o_stride;
  p.dq_stride = dq_stride; p.dk_stride = dk_stride; p.dv_stride = dv_stride;
  p.seq_start = seq_start; p.lse = const_cast<float*>(lse); p.delta = delta;
  p.T = T; p.hq = hq; p.hkv = hkv; p.scale = scale; p.window = window;
  const int smem_dq = 6 * kTileBytes + 256;
  const int smem_dkv = 6 * kTileBytes + 6 * kTile * 4;
  static DeviceOnce once;
  if (once.pending()) {
    int e = set_smem(reinterpret_cast<const void*>(attn_bwd_dq_kernel), smem_dq);
    if (e) return e;
    e = set_smem(reinterpret_cast<const void*>(attn_bwd_dkv_kernel), smem_dkv);
    if (e) return e;
    once.mark();
  }
  dim3 gq((T + kTile - 1) / kTile, hq);
  attn_bwd_dq_kernel<<<gq, kAttnThreads, smem_dq, st>>>(p);
  int e = static_cast<int>(cudaGetLastError());
  if (e) return e;
  dim3 gk((T + kTile - 1) / kTile, hkv);
  attn_bwd_dkv_kernel<<<gk, kAttnThreads, smem_dkv, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

// ================================================================================= paged-KV decode / verify attention
// Attention of a few new query tokens per sequence against a block-paged KV cache (block = 64 tokens =
// one key tile). Used for single-token decode (q_len 1), speculative verification (q_len = k+1) and
// chunked prefill continuation. The rows of the 64-row query tile are the (query token, head-in-group)
// pairs of one (sequence, kv head): row = i * rep + g. Key position t is visible to query token i iff
// t <= seq_len - q_len + i. With n_split > 1 each CTA covers a slice of the key blocks and writes an
// unnormalised partial (o, m, l) to scratch; `paged_attn_combine_kernel` merges the slices.
// The reference has no paged attention kernel: its paged cache is gathered and concatenated into a dense
// tensor before every SDPA call (crates/pmetal-mlx/src/kv_cache/paged.rs:262-530).
namespace pm {

struct PagedParams {
  const __nv_bfloat16* q;        // [total_q, hq, 128]
  const __nv_bfloat16* k_cache;  // [num_blocks, 64, hkv, 128]
  const __nv_bfloat16* v_cache;
  __nv_bfloat16* out;            // [total_q, hq, 128]
  const int* block_table;        // [num_seqs, max_blocks]
  const int* seq_lens;           // [num_seqs] keys available (new tokens included)
  const int* q_start;            // [num_seqs] first query row of the sequence in q
  const int* q_lens;             // [num_seqs]
  float* part_o;                 // [n_split, total_q, hq, 128] (only when n_split > 1)
  float* part_ml;                // [n_split, total_q, hq, 2]
  int max_blocks, hq, hkv, n_split, total_q, q_tiles;
  float scale;
  int window;
  int sink;                      // with a window: the first `sink` keys stay visible (attention-sink cache)
  // int8 cache (kQ8): k_cache / v_cache hold int8 [num_blocks, 64, hkv, 128] and these hold one fp32 scale per group
  // of 64 channels, [num_blocks, 64, hkv, 2]
  const float* k_scale;
  const float* v_scale;
  // 4-bit code-book cache (kQ == 2): k_cache / v_cache hold two codes per byte (first channel in the low nibble),
  // [num_blocks, 64, hkv, 64] bytes; a value is lut[code] * scale with the scales laid out as for the int8 cache
  float lut[16];
};

// One thread's share of a [64][128] int8 key or value block in flight: four 16-byte pieces and their scales.
struct Q8Regs {
  uint4 d[4];
  float s[4];
};
__device__ __forceinline__ void q8_fetch(Q8Regs& r, const int8_t* base, const float* sbase, long long row_stride,
                                         long long srow_stride) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int idx = threadIdx.x + i * kAttnThreads;   // 0..511
    const int row = idx >> 3, c = idx & 7;            // 16 channels [16c, 16c+16)
    r.d[i] = __ldg(reinterpret_cast<const uint4*>(base + row * row_stride + c * 16));
    r.s[i] = __ldg(sbase + row * srow_stride + (c >> 2));
  }
}
// expand to bf16 and store into the swizzled [64][128] tile that the MMA fragments read
__device__ __forceinline__ void q8_store(const Q8Regs& r, uint8_t* smem_tile) {
  const uint32_t sbase = smem_addr(smem_tile);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int idx = threadIdx.x + i * kAttnThreads;
    const int row = idx >> 3, c = idx & 7;
    const uint32_t w[4] = {r.d[i].x, r.d[i].y, r.d[i].z, r.d[i].w};
    uint32_t o[8];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float f0 = static_cast<float>(static_cast<int8_t>(w[q] & 0xff)) * r.s[i];
      const float f1 = static_cast<float>(static_cast<int8_t>((w[q] >> 8) & 0xff)) * r.s[i];
      const float f2 = static_cast<float>(static_cast<int8_t>((w[q] >> 16) & 0xff)) * r.s[i];
      const float f3 = static_cast<float>(static_cast<int8_t>(w[q] >> 24)) * r.s[i];
      o[2 * q] = pack2(f0, f1);
      o[2 * q + 1] = pack2(f2, f3);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t dst = sbase + row * 256 + (((2 * c + h) ^ (row & 7)) << 4);
      asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(o[4 * h]), "r"(o[4 * h + 1]),
                   "r"(o[4 * h + 2]), "r"(o[4 * h + 3])
                   : "memory");
    }
  }
}

// One thread's share of a [64][128] block of 4-bit codes (64 bytes per row): two 16-byte pieces of 32 codes each.
struct Q4Regs {
  uint4 d[2];
  float s[2];
};
__device__ __forceinline__ void q4_fetch(Q4Regs& r, const uint8_t* base, const float* sbase, long long row_stride_bytes,
                                         long long srow_stride) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int idx = threadIdx.x + i * kAttnThreads;   // 0..255
    const int row = idx >> 2, c = idx & 3;            // 32 channels [32c, 32c+32)
    r.d[i] = __ldg(reinterpret_cast<const uint4*>(base + row * row_stride_bytes + c * 16));
    r.s[i] = __ldg(sbase + row * srow_stride + (c >> 1));
  }
}
__device__ __forceinline__ void q4_store(const Q4Regs& r, uint8_t* smem_tile, const float* lut) {
  const uint32_t sbase = smem_addr(smem_tile);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int idx = threadIdx.x + i * kAttnThreads;
    const int row = idx >> 2, c = idx & 3;
    const uint32_t w[4] = {r.d[i].x, r.d[i].y, r.d[i].z, r.d[i].w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {                     // one word = 8 codes = one 16-byte chunk of bf16
      uint32_t o[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const uint32_t byte = (w[q] >> (8 * b)) & 0xffu;
        o[b] = pack2(lut[byte & 15u] * r.s[i], lut[byte >> 4] * r.s[i]);
      }
      const uint32_t dst = sbase + row * 256 + (((4 * c + q) ^ (row & 7)) << 4);
      asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                   : "memory");
    }
  }
}

template <int kQ>
__global__ void __launch_bounds__(kAttnThreads) paged_attn_kernel(const PagedParams p) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kTileBytes;       // 2 buffers
  uint8_t* sV = smem + 3 * kTileBytes;   // 2 buffers
  const int seq = blockIdx.x / p.q_tiles, row_base = (blockIdx.x % p.q_tiles) * kTile;
  const int hk = blockIdx.y, split = blockIdx.z;
  const int rep = p.hq / p.hkv;
  const int q_len = p.q_lens[seq], q0 = p.q_start[seq], kv_len = p.seq_lens[seq];
  const int nq = q_len * rep - row_base;   // valid rows of this 64-row tile
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  if (q_len <= 0 || kv_len <= 0 || nq <= 0) return;

  // keys visible to the last row of this tile bound the block range (causal)
  const int last_row = min(row_base + kTile, q_len * rep) - 1;
  const int n_blocks = (kv_len - q_len + last_row / rep) / kTile + 1;
  const int per = (n_blocks + p.n_split - 1) / p.n_split;
  const int b0 = split * per, b1 = min(n_blocks, b0 + per);

  // gather the query rows into the swizzled tile (rows >= nq are zero)
  {
    const uint32_t sbase = smem_addr(sQ);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = threadIdx.x + i * kAttnThreads;
      const int r = idx >> 4, c = idx & 15;
      const uint32_t dst = sbase + r * 256 + ((c ^ (r & 7)) << 4);
      if (r < nq) {
        const int gr = row_base + r;
        const int qi = gr / rep, gh = gr - qi * rep;
        cp_async16(dst, p.q + (static_cast<long long>(q0 + qi) * p.hq + hk * rep + gh) * kD + c * 8);
      } else {
        asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(dst), "r"(0) : "memory");
      }
    }
  }
  const long long row_stride = static_cast<long long>(p.hkv) * kD;
  const int* bt = p.block_table + static_cast<long long>(seq) * p.max_blocks;
  auto kv_base = [&](const __nv_bfloat16* cache, int blk) {
    return cache + (static_cast<long long>(bt[blk]) * kTile * p.hkv + hk) * kD;
  };
  // with a sliding window, key blocks that no row of this tile can see are skipped (their table entries may be stale:
  // the cache manager recycles such blocks): a block is dead when it ends before the window of the tile's first row
  // and starts after the sink
  const int lim_first = kv_len - q_len + row_base / rep;
  auto dead = [&](int blk) {
    return p.window > 0 && blk * kTile + kTile - 1 < lim_first - p.window + 1 && blk * kTile >= p.sink;
  };
  auto next_live = [&](int blk) {
    while (blk < b1 && dead(blk)) ++blk;
    return blk;
  };
  Q8Regs rk, rv;
  Q4Regs rk4, rv4;
  __shared__ float s_lut[16];
  if (kQ == 2) {
    if (threadIdx.x < 16) s_lut[threadIdx.x] = p.lut[threadIdx.x];
    __syncthreads();
  }
  auto fetch_q8 = [&](int blk) {
    const long long off = (static_cast<long long>(bt[blk]) * kTile * p.hkv + hk);
    if (kQ == 2) {
      q4_fetch(rk4, reinterpret_cast<const uint8_t*>(p.k_cache) + off * (kD / 2), p.k_scale + off * 2,
               static_cast<long long>(p.hkv) * (kD / 2), static_cast<long long>(p.hkv) * 2);
      q4_fetch(rv4, reinterpret_cast<const uint8_t*>(p.v_cache) + off * (kD / 2), p.v_scale + off * 2,
               static_cast<long long>(p.hkv) * (kD / 2), static_cast<long long>(p.hkv) * 2);
      return;
    }
    q8_fetch(rk, reinterpret_cast<const int8_t*>(p.k_cache) + off * kD, p.k_scale + off * 2, row_stride,
             static_cast<long long>(p.hkv) * 2);
    q8_fetch(rv, reinterpret_cast<const int8_t*>(p.v_cache) + off * kD, p.v_scale + off * 2, row_stride,
             static_cast<long long>(p.hkv) * 2);
  };
  auto store_q8 = [&](uint8_t* dk, uint8_t* dv) {
    if (kQ == 2) {
      q4_store(rk4, dk, s_lut);
      q4_store(rv4, dv, s_lut);
    } else {
      q8_store(rk, dk);
      q8_store(rv, dv);
    }
  };
  int b_cur = next_live(b0);
  if (b_cur < b1) {
    if (kQ) {
      fetch_q8(b_cur);
      store_q8(sK, sV);
    } else {
      load_tile(sK, kv_base(p.k_cache, b_cur), row_stride, 0, kTile);
      load_tile(sV, kv_base(p.v_cache, b_cur), row_stride, 0, kTile);
    }
  }
  cp_async_commit();

  float o_acc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float sl2 = p.scale * kLog2e;
  const uint32_t q_tile = smem_addr(sQ);
  const bool warp_active = warp * 16 < nq;
  const int r_lo = warp * 16 + g;
  // visible-key limit (inclusive) for the two rows this thread owns
  const int lim_lo = kv_len - q_len + ((row_base + r_lo) / rep), lim_hi = kv_len - q_len + ((row_base + r_lo + 8) / rep);

  int it = 0;
  for (int b = b_cur; b < b1; ++it) {
    const int buf = it & 1;
    const int b_next = next_live(b + 1);
    if (kQ) {
      if (b_next < b1) fetch_q8(b_next);          // global loads stay in flight while this block is processed
      cp_async_wait<0>();                         // the query tile (first iteration)
    } else if (b_next < b1) {
      load_tile(sK + (buf ^ 1) * kTileBytes, kv_base(p.k_cache, b_next), row_stride, 0, kTile);
      load_tile(sV + (buf ^ 1) * kTileBytes, kv_base(p.v_cache, b_next), row_stride, 0, kTile);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (warp_active) {
      const uint32_t k_tile = smem_addr(sK + buf * kTileBytes);
      const uint32_t v_tile = smem_addr(sV + buf * kTileBytes);
      float s[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        uint32_t a[4];
        load_a_frag(q_tile, warp * 16, kk * 16, lane, a);
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t bb[4];
          load_b_frag_nt(k_tile, np * 16, kk * 16, lane, bb);
          mma_bf16(s[2 * np], a[0], a[1], a[2], a[3], bb[0], bb[1]);
          mma_bf16(s[2 * np + 1], a[0], a[1], a[2], a[3], bb[2], bb[3]);
        }
      }
      const int j0 = b * kTile;
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = j0 + nt * 8 + 2 * t4 + (e & 1);
          const int lim = (e < 2) ? lim_lo : lim_hi;
          bool ok = j <= lim;
          if (p.window > 0) ok = ok && (lim - j < p.window || j < p.sink);
          const float v = ok ? s[nt][e] * sl2 : -INFINITY;
          s[nt][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
      float corr[2], m_use[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_run[r], mx[r]);
        m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
        corr[r] = (m_run[r] == -INFINITY) ? 0.f : exp2f(m_run[r] - m_use[r]);
        m_run[r] = m_new;
        l_run[r] *= corr[r];
      }
      float rs[2] = {0.f, 0.f};
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pv = exp2f(s[nt][e] - m_use[e >> 1]);
          s[nt][e] = pv;
          rs[e >> 1] += pv;
        }
      l_run[0] += rs[0];
      l_run[1] += rs[1];
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) {
        o_acc[nt][0] *= corr[0]; o_acc[nt][1] *= corr[0];
        o_acc[nt][2] *= corr[1]; o_acc[nt][3] *= corr[1];
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const uint32_t a0 = pack2(s[2 * kk][0], s[2 * kk][1]);
        const uint32_t a1 = pack2(s[2 * kk][2], s[2 * kk][3]);
        const uint32_t a2 = pack2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        const uint32_t a3 = pack2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int np = 0; np < 8; ++np) {
          uint32_t bb[4];
          load_b_frag_nn(v_tile, kk * 16, np * 16, lane, bb);
          mma_bf16(o_acc[2 * np], a0, a1, a2, a3, bb[0], bb[1]);
          mma_bf16(o_acc[2 * np + 1], a0, a1, a2, a3, bb[2], bb[3]);
        }
      }
    }
    if (kQ && b_next < b1) {      // the other buffer was last read one iteration ago (barrier at the end of it)
      store_q8(sK + (buf ^ 1) * kTileBytes, sV + (buf ^ 1) * kTileBytes);
    }
    __syncthreads();
    b = b_next;
  }
  if (!warp_active) return;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if (r_lo + r * 8 >= nq) continue;
    const int row = row_base + r_lo + r * 8;
    const int qi = row / rep, gh = row - qi * rep;
    const long long orow = (static_cast<long long>(q0 + qi) * p.hq + hk * rep + gh);
    if (p.n_split == 1) {
      const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
      __nv_bfloat16* o = p.out + orow * kD;
#pragma unroll
      for (int nt = 0; nt < 16; ++nt)
        *reinterpret_cast<uint32_t*>(o + nt * 8 + 2 * t4) = pack2(o_acc[nt][2 * r] * inv, o_acc[nt][2 * r + 1] * inv);
    } else {
      float* o = p.part_o + (static_cast<long long>(split) * p.total_q * p.hq + orow) * kD;
#pragma unroll
      for (int nt = 0; nt < 16; ++nt)
        *reinterpret_cast<float2*>(o + nt * 8 + 2 * t4) = make_float2(o_acc[nt][2 * r], o_acc[nt][2 * r + 1]);
      if (t4 == 0) {
        float* ml = p.part_ml + (static_cast<long long>(split) * p.total_q * p.hq + orow) * 2;
        ml[0] = m_run[r];
        ml[1] = l_run[r];
      }
    }
  }
}

// Merge the per-slice partials: one warp per (query row, head).
__global__ void paged_attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                          __nv_bfloat16* __restrict__ out, int rows, int n_split) {
  pdl_launch_dependents();
  pdl_wait();
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (gw >= rows) return;
  float m = -INFINITY;
  for (int s = 0; s < n_split; ++s) m = fmaxf(m, part_ml[(static_cast<long long>(s) * rows + gw) * 2]);
  float l = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < n_split; ++s) {
    const float ms = part_ml[(static_cast<long long>(s) * rows + gw) * 2];
    const float ls = part_ml[(static_cast<long long>(s) * rows + gw) * 2 + 1];
    if (ms == -INFINITY) continue;
    const float w = exp2f(ms - m);
    l += ls * w;
    const float4 o = *reinterpret_cast<const float4*>(part_o + (static_cast<long long>(s) * rows + gw) * kD + lane * 4);
    acc[0] += o.x * w; acc[1] += o.y * w; acc[2] += o.z * w; acc[3] += o.w * w;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  uint2 ov;
  *reinterpret_cast<__nv_bfloat162*>(&ov.x) = __floats2bfloat162_rn(acc[0] * inv, acc[1] * inv);
  *reinterpret_cast<__nv_bfloat162*>(&ov.y) = __floats2bfloat162_rn(acc[2] * inv, acc[3] * inv);
  *reinterpret_cast<uint2*>(out + static_cast<long long>(gw) * kD + lane * 4) = ov;
}

// Append new keys/values to the paged cache: slot[t] = block_id * 64 + offset for each new token.
__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ k, long long k_stride,
                                 const __nv_bfloat16* __restrict__ v, long long v_stride,
                                 __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                 const long long* __restrict__ slots, int n_tokens, int hkv) {
  const int per_tok = hkv * (kD / 8);   // 16-byte chunks per token
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
       i < static_cast<long long>(n_tokens) * per_tok; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / per_tok), c = static_cast<int>(i - static_cast<long long>(t) * per_tok);
    const long long slot = slots[t];
    if (slot < 0) continue;
    const uint4 kv = *reinterpret_cast<const uint4*>(k + t * k_stride + c * 8);
    const uint4 vv = *reinterpret_cast<const uint4*>(v + t * v_stride + c * 8);
    *reinterpret_cast<uint4*>(k_cache + slot * hkv * kD + c * 8) = kv;
    *reinterpret_cast<uint4*>(v_cache + slot * hkv * kD + c * 8) = vv;
  }
}

}  // namespace pm

// Scratch (part_o / part_ml) is needed only when n_split > 1:
//   part_o  : n_split * total_q * hq * 128 floats,  part_ml : n_split * total_q * hq * 2 floats
// k_scale / v_scale non-null: the caches hold int8 with one fp32 scale per (token, kv head, 64-channel group).
// sink: with window > 0, the first `sink` keys of a sequence stay visible.
static int paged_attn_launch(const void* q, const void* k_cache, const void* v_cache, void* out, const int* block_table,
                             const int* seq_lens, const int* q_start, const int* q_lens, float* part_o, float* part_ml,
                             int num_seqs, int max_blocks, int total_q, int max_q, int hq, int hkv, int n_split,
                             float scale, int window, int sink, const float* k_scale, const float* v_scale,
                             const float* lut16, cudaStream_t st) {
  if (hq % hkv || num_seqs <= 0) return -1;
  if (n_split < 1 || (n_split > 1 && (!part_o || !part_ml))) return -2;
  if ((k_scale == nullptr) != (v_scale == nullptr)) return -4;
  if (lut16 && !k_scale) return -5;
  PagedParams p{};
  p.sink = sink; p.k_scale = k_scale; p.v_scale = v_scale;
  if (lut16)
    for (int i = 0; i < 16; ++i) p.lut[i] = lut16[i];
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.block_table = block_table; p.seq_lens = seq_lens; p.q_start = q_start; p.q_lens = q_lens;
  p.part_o = part_o; p.part_ml = part_ml;
  p.max_blocks = max_blocks; p.hq = hq; p.hkv = hkv; p.n_split = n_split; p.total_q = total_q;
  p.scale = scale; p.window = window;
  p.q_tiles = (max_q * (hq / hkv) + kTile - 1) / kTile;
  if (p.q_tiles < 1) p.q_tiles = 1;
  const int smem = 5 * kTileBytes;
  static DeviceOnce once;
  if (once.pending()) {
    int e = set_smem(reinterpret_cast<const void*>(paged_attn_kernel<0>), smem);
    if (e) return e;
    e = set_smem(reinterpret_cast<const void*>(paged_attn_kernel<1>), smem);
    if (e) return e;
    e = set_smem(reinterpret_cast<const void*>(paged_attn_kernel<2>), smem);
    if (e) return e;
    once.mark();
  }
  dim3 grid(num_seqs * p.q_tiles, hkv, n_split);
  int e;
  if (lut16) e = static_cast<int>(launch_pdl(paged_attn_kernel<2>, grid, dim3(kAttnThreads), static_cast<size_t>(smem), st, p));
  else if (k_scale) e = static_cast<int>(launch_pdl(paged_attn_kernel<1>, grid, dim3(kAttnThreads), static_cast<size_t>(smem), st, p));
  else e = static_cast<int>(launch_pdl(paged_attn_kernel<0>, grid, dim3(kAttnThreads), static_cast<size_t>(smem), st, p));
  if (e || n_split == 1) return e;
  const int rows = total_q * hq;
  return static_cast<int>(launch_pdl(paged_attn_combine_kernel, dim3((rows + 7) / 8), dim3(256), 0, st,
                                     static_cast<const float*>(part_o), static_cast<const float*>(part_ml),
                                     static_cast<__nv_bfloat16*>(out), rows, n_split));
}

extern "C" int pm_paged_attn_ex(const void* q, const void* k_cache, const void* v_cache, void* out,
                                const int* block_table, const int* seq_lens, const int* q_start, const int* q_lens,
                                float* part_o, float* part_ml, int num_seqs, int max_blocks, int total_q, int max_q,
                                int hq, int hkv, int n_split, float scale, int window, int sink, const float* k_scale,
                                const float* v_scale, cudaStream_t st) {
  return paged_attn_launch(q, k_cache, v_cache, out, block_table, seq_lens, q_start, q_lens, part_o, part_ml, num_seqs,
                           max_blocks, total_q, max_q, hq, hkv, n_split, scale, window, sink, k_scale, v_scale, nullptr, st);
}

// 4-bit code-book cache: k_cache / v_cache hold two codes per byte [num_blocks, 64, hkv, 64]; a cached value is
// lut16[code] * scale (scales as for the int8 cache). lut16: 16 floats on the host. The query and the output live in
// whatever basis the cached vectors were quantised in (the caller rotates the query and un-rotates the output).
extern "C" int pm_paged_attn_q4(const void* q, const void* k_cache, const void* v_cache, void* out,
                                const int* block_table, const int* seq_lens, const int* q_start, const int* q_lens,
                                float* part_o, float* part_ml, int num_seqs, int max_blocks, int total_q, int max_q,
                                int hq, int hkv, int n_split, float scale, int window, int sink, const float* k_scale,
                                const float* v_scale, const float* lut16, cudaStream_t st) {
  if (!lut16) return -5;
  return paged_attn_launch(q, k_cache, v_cache, out, block_table, seq_lens, q_start, q_lens, part_o, part_ml, num_seqs,
                           max_blocks, total_q, max_q, hq, hkv, n_split, scale, window, sink, k_scale, v_scale, lut16, st);
}

extern "C" int pm_paged_attn(const void* q, const void* k_cache, const void* v_cache, void* out, const int* block_table,
                             const int* seq_lens, const int* q_start, const int* q_lens, float* part_o, float* part_ml,
                             int num_seqs, int max_blocks, int total_q, int max_q, int hq, int hkv, int n_split,
                             float scale, int window, cudaStream_t st) {
  return pm_paged_attn_ex(q, k_cache, v_cache, out, block_table, seq_lens, q_start, q_lens, part_o, part_ml, num_seqs,
                          max_blocks, total_q, max_q, hq, hkv, n_split, scale, window, 0, nullptr, nullptr, st);
}

// int8 cache append: one warp per (token, kv head) row of 128 channels; each half (64 channels) gets its own scale
// absmax / 127 (symmetric), stored next to the codes.
__global__ void kv_append_q8_kernel(const __nv_bfloat16* __restrict__ k, long long k_stride,
                                    const __nv_bfloat16* __restrict__ v, long long v_stride, int8_t* __restrict__ k_cache,
                                    int8_t* __restrict__ v_cache, float* __restrict__ k_scale,
                                    float* __restrict__ v_scale, const long long* __restrict__ slots, int n_tokens,
                                    int hkv) {
  const int lane = threadIdx.x & 31;
  const long long rows = static_cast<long long>(n_tokens) * hkv * 2;      // K rows then V rows per (token, head)
  for (long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5; w < rows;
       w += (static_cast<long long>(gridDim.x) * blockDim.x) >> 5) {
    const int is_v = static_cast<int>(w & 1);
    const long long th = w >> 1;
    const int t = static_cast<int>(th / hkv), h = static_cast<int>(th - static_cast<long long>(t) * hkv);
    const long long slot = slots[t];
    if (slot < 0) continue;
    const __nv_bfloat16* src = (is_v ? v + t * v_stride : k + t * k_stride) + h * pm::kD + lane * 4;
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    float f[4];
    f[0] = __uint_as_float(raw.x << 16); f[1] = __uint_as_float(raw.x & 0xffff0000u);
    f[2] = __uint_as_float(raw.y << 16); f[3] = __uint_as_float(raw.y & 0xffff0000u);
    float mx = fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(fabsf(f[2]), fabsf(f[3])));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));   // within each half-warp
    const float sc = mx > 0.f ? mx / 127.f : 1.f;
    const float inv = 1.f / sc;
    uint32_t packed = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      int q = __float2int_rn(f[e] * inv);
      q = max(-127, min(127, q));
      packed |= (static_cast<uint32_t>(q) & 0xffu) << (8 * e);
    }
    const long long row = slot * hkv + h;
    *reinterpret_cast<uint32_t*>((is_v ? v_cache : k_cache) + row * pm::kD + lane * 4) = packed;
    if ((lane & 15) == 0) (is_v ? v_scale : k_scale)[row * 2 + (lane >> 4)] = sc;
  }
}

extern "C" int pm_kv_append_q8(const void* k, long long k_stride, const void* v, long long v_stride, void* k_cache,
                               void* v_cache, float* k_scale, float* v_scale, const long long* slots, int n_tokens,
                               int hkv, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  const long long warps = static_cast<long long>(n_tokens) * hkv * 2;
  int grid = static_cast<int>((warps + 7) / 8);
  if (grid > num_sms() * 8) grid = num_sms() * 8;
  kv_append_q8_kernel<<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(k), k_stride,
                                            static_cast<const __nv_bfloat16*>(v), v_stride,
                                            static_cast<int8_t*>(k_cache), static_cast<int8_t*>(v_cache), k_scale,
                                            v_scale, slots, n_tokens, hkv);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------- rotated 4-bit cache
// Signed Walsh-Hadamard transform of a 128-vector held four consecutive elements per lane (natural order):
// two butterfly stages inside the thread, five across lanes.
__device__ __forceinline__ void fwht128(float (&f)[4], int lane) {
  float a = f[0] + f[1], b = f[0] - f[1], c = f[2] + f[3], d = f[2] - f[3];
  f[0] = a + c; f[1] = b + d; f[2] = a - c; f[3] = b - d;
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
    const bool upper = (lane & m) != 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float o = __shfl_xor_sync(0xffffffffu, f[e], m);
      f[e] = upper ? o - f[e] : f[e] + o;
    }
  }
}

// y = H (x * sign) / sqrt(128) (forward) or (H y) / sqrt(128) * sign (inverse); rows of 128, one warp per row.
__global__ void tq_rotate_kernel(const __nv_bfloat16* __restrict__ x, long long x_stride, const float* __restrict__ sign,
                                 __nv_bfloat16* __restrict__ y, long long y_stride, long long rows, int heads, int inverse) {
  const int lane = threadIdx.x & 31;
  const float s0 = sign[lane * 4], s1 = sign[lane * 4 + 1], s2 = sign[lane * 4 + 2], s3 = sign[lane * 4 + 3];
  for (long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5; w < rows;
       w += (static_cast<long long>(gridDim.x) * blockDim.x) >> 5) {
    const long long t = w / heads;
    const int h = static_cast<int>(w - t * heads);
    const uint2 raw = *reinterpret_cast<const uint2*>(x + t * x_stride + h * pm::kD + lane * 4);
    float f[4] = {__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16),
                  __uint_as_float(raw.y & 0xffff0000u)};
    if (!inverse) { f[0] *= s0; f[1] *= s1; f[2] *= s2; f[3] *= s3; }
    fwht128(f, lane);
    const float r = 0.08838834764831845f;       // 1 / sqrt(128)
    f[0] *= r; f[1] *= r; f[2] *= r; f[3] *= r;
    if (inverse) { f[0] *= s0; f[1] *= s1; f[2] *= s2; f[3] *= s3; }
    uint2 o;
    o.x = pack2(f[0], f[1]);
    o.y = pack2(f[2], f[3]);
    *reinterpret_cast<uint2*>(y + t * y_stride + h * pm::kD + lane * 4) = o;
  }
}

// Append to the rotated 4-bit cache: one warp per (token, kv head, K or V) row. The row is rotated, its norm taken, every
// coordinate of the unit-variance vector  H(x sign) / |x|  is mapped to the cell of a 16-level scalar quantiser
// (thr: its 15 decision thresholds), codes are packed two per byte, and |x| / sqrt(128) is stored as the row's scale.
__global__ void kv_append_tq4_kernel(const __nv_bfloat16* __restrict__ k, long long k_stride,
                                     const __nv_bfloat16* __restrict__ v, long long v_stride, uint8_t* __restrict__ k_cache,
                                     uint8_t* __restrict__ v_cache, float* __restrict__ k_scale,
                                     float* __restrict__ v_scale, const long long* __restrict__ slots,
                                     const float* __restrict__ sign, const float* __restrict__ thr, int n_tokens, int hkv) {
  __shared__ float s_thr[15];
  if (threadIdx.x < 15) s_thr[threadIdx.x] = thr[threadIdx.x];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const float s0 = sign[lane * 4], s1 = sign[lane * 4 + 1], s2 = sign[lane * 4 + 2], s3 = sign[lane * 4 + 3];
  const long long rows = static_cast<long long>(n_tokens) * hkv * 2;
  for (long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5; w < rows;
       w += (static_cast<long long>(gridDim.x) * blockDim.x) >> 5) {
    const int is_v = static_cast<int>(w & 1);
    const long long th = w >> 1;
    const int t = static_cast<int>(th / hkv), h = static_cast<int>(th - static_cast<long long>(t) * hkv);
    const long long slot = slots[t];
    if (slot < 0) continue;
    const __nv_bfloat16* src = (is_v ? v + t * v_stride : k + t * k_stride) + h * pm::kD + lane * 4;
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    float f[4] = {__uint_as_float(raw.x << 16) * s0, __uint_as_float(raw.x & 0xffff0000u) * s1,
                  __uint_as_float(raw.y << 16) * s2, __uint_as_float(raw.y & 0xffff0000u) * s3};
    float ss = f[0] * f[0] + f[1] * f[1] + f[2] * f[2] + f[3] * f[3];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float norm = sqrtf(ss);
    fwht128(f, lane);                      // |H x|^2 = 128 |x|^2: H x / |x| has unit-variance coordinates
    const float inv = norm > 1e-12f ? 1.f / norm : 0.f;
    uint32_t codes = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float y = f[e] * inv;
      int c = 0;
#pragma unroll
      for (int j = 0; j < 15; ++j) c += (s_thr[j] < y) ? 1 : 0;
      codes |= static_cast<uint32_t>(c) << (4 * e);
    }
    const long long row = slot * hkv + h;
    *reinterpret_cast<uint16_t*>((is_v ? v_cache : k_cache) + row * (pm::kD / 2) + lane * 2) = static_cast<uint16_t>(codes);
    if ((lane & 15) == 0) (is_v ? v_scale : k_scale)[row * 2 + (lane >> 4)] = norm * 0.08838834764831845f;
  }
}

// sign: 128 floats (+-1) on the device; thr: 15 ascending thresholds on the device.
extern "C" int pm_kv_append_tq4(const void* k, long long k_stride, const void* v, long long v_stride, void* k_cache,
                                void* v_cache, float* k_scale, float* v_scale, const long long* slots, const float* sign,
                                const float* thr, int n_tokens, int hkv, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  const long long warps = static_cast<long long>(n_tokens) * hkv * 2;
  int grid = static_cast<int>((warps + 7) / 8);
  if (grid > num_sms() * 8) grid = num_sms() * 8;
  kv_append_tq4_kernel<<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(k), k_stride,
                                             static_cast<const __nv_bfloat16*>(v), v_stride,
                                             static_cast<uint8_t*>(k_cache), static_cast<uint8_t*>(v_cache), k_scale,
                                             v_scale, slots, sign, thr, n_tokens, hkv);
  return static_cast<int>(cudaGetLastError());
}

// x, y: [rows / heads, heads, 128] bf16 with token strides x_stride / y_stride (elements); inverse 0: y = H (x sign) / sqrt(d),
// inverse 1: y = (H x) / sqrt(d) * sign.
extern "C" int pm_tq_rotate(const void* x, long long x_stride, const float* sign, void* y, long long y_stride,
                            long long tokens, int heads, int inverse, cudaStream_t st) {
  if (tokens <= 0) return 0;
  const long long rows = tokens * heads;
  int grid = static_cast<int>((rows + 7) / 8);
  if (grid > num_sms() * 8) grid = num_sms() * 8;
  tq_rotate_kernel<<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), x_stride, sign,
                                         static_cast<__nv_bfloat16*>(y), y_stride, rows, heads, inverse);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int pm_kv_append(const void* k, long long k_stride, const void* v, long long v_stride, void* k_cache,
                            void* v_cache, const long long* slots, int n_tokens, int hkv, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  const long long work = static_cast<long long>(n_tokens) * hkv * 16;
  int grid = static_cast<int>((work + 255) / 256);
  if (grid > num_sms() * 8) grid = num_sms() * 8;
  kv_append_kernel<<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(k), k_stride,
                                         static_cast<const __nv_bfloat16*>(v), v_stride,
                                         static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), slots,
                                         n_tokens, hkv);
  return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------ allocation-free split-KV entry point
// Same kernels as pm_paged_attn; the partials live in a static device array (see paged_attn_static.h).
#include "paged_attn_static.h"

namespace pm {
// [rows][128] partial outputs followed by [rows][2] (max, sum); rows = n_split * total_q * hq
static __device__ __align__(256) float g_paged_static_scratch[PM_PAGED_STATIC_MAX_ROWS * (kD + 2)];
constexpr int kMaxStaticDevices = 64;
static float* g_paged_static_ptr[kMaxStaticDevices] = {};
}  // namespace pm

extern "C" int pm_paged_attn_static_max_rows(void) { return PM_PAGED_STATIC_MAX_ROWS; }

extern "C" const char* pm_paged_attn_static_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case PM_PAGED_STATIC_E_BAD_HEADS: return "hq must be a multiple of hkv and num_seqs must be positive";
    case PM_PAGED_STATIC_E_BAD_SPLIT: return "n_split must be at least 1";
    case PM_PAGED_STATIC_E_TOO_LARGE:
      return "n_split * total_q * hq exceeds PM_PAGED_STATIC_MAX_ROWS (4096): use pm_paged_attn with caller scratch";
    case PM_PAGED_STATIC_E_DEVICE: return "current device index is outside the per-device scratch table";
    default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "unknown error";
  }
}

extern "C" int pm_paged_attn_static(const void* q, const void* k_cache, const void* v_cache, void* out,
                                    const int* block_table, const int* seq_lens, const int* q_start, const int* q_lens,
                                    int num_seqs, int max_blocks, int total_q, int max_q, int hq, int hkv, int n_split,
                                    float scale, int window, cudaStream_t st) {
  using namespace pm;
  if (hkv <= 0 || hq % hkv || num_seqs <= 0) return PM_PAGED_STATIC_E_BAD_HEADS;
  if (n_split < 1) return PM_PAGED_STATIC_E_BAD_SPLIT;
  const long long rows_all = static_cast<long long>(n_split) * total_q * hq;
  if (total_q <= 0 || rows_all > PM_PAGED_STATIC_MAX_ROWS) return PM_PAGED_STATIC_E_TOO_LARGE;
  int dev = 0;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) return static_cast<int>(ce);
  if (dev < 0 || dev >= kMaxStaticDevices) return PM_PAGED_STATIC_E_DEVICE;
  if (!g_paged_static_ptr[dev]) {   // once per device; not a capturable call, so it must precede any capture
    float* ptr = nullptr;
    ce = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_paged_static_scratch);
    if (ce != cudaSuccess) return static_cast<int>(ce);
    if (!ptr) return static_cast<int>(cudaErrorInvalidSymbol);
    g_paged_static_ptr[dev] = ptr;
  }
  float* part_o = g_paged_static_ptr[dev];
  float* part_ml = part_o + static_cast<long long>(PM_PAGED_STATIC_MAX_ROWS) * kD;
  if (n_split > 1) {
    ce = cudaMemsetAsync(part_ml, 0, static_cast<size_t>(rows_all) * 2 * sizeof(float), st);
    if (ce != cudaSuccess) return static_cast<int>(ce);
  }
  return pm_paged_attn(q, k_cache, v_cache, out, block_table, seq_lens, q_start, q_lens, part_o, part_ml, num_seqs,
                       max_blocks, total_q, max_q, hq, hkv, n_split, scale, window, st);
}
