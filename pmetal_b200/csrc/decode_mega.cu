// One launch per decode step for all transformer layers of a dense decoder (Qwen3 / Llama shape, head_dim 128).
//
// A decode step of a small model is a chain of ~170 tiny dependent kernels; each costs 5-8 us of launch, prologue and
// tail latency for 1-3 us of weight streaming, so the step runs at ~1 TB/s instead of the 7 TB/s the memory system can
// deliver. This kernel keeps one CTA per SM resident for the whole step (cooperative launch) and walks the layers in
// phases separated by a grid barrier:
//
//   P1  qkv   = RMSNorm(x) Wqkv^T                      (tensor-core mat-vec: the <= 16 rows are the A operand of
//                                                        mma.m16n8k16, a CTA owns 8 output columns, its warps split K)
//   P2  attn  = softmax(q k^T) v over the paged cache: one CTA per (row, kv head, key split), its warps take slices
//               of the keys eight at a time and merge through shared memory; the new token's q/k get their per-head
//               RMSNorm and rotary embedding here and the new k/v are appended to the cache by the last split; with
//               several splits the last CTA to finish a (row, kv head) merges the partial results
//   P3  h     = x + attn Wo^T
//   P4  act   = SwiGLU(RMSNorm(h) Wgate_up^T)
//   P5  x     = h + act Wdown^T
//
// Before a warp arrives at a barrier it asks for the weight rows of its next phase to be pulled into L2, so the DRAM
// stream continues while the barrier settles. Activations that other CTAs wrote are read with ld.global.cg (L1 is not
// coherent across SMs); weights go through the read-only path. The barrier is a monotonic arrival counter with a
// bounded wait: on a timeout the kernel records a status code, raises an abort word that every CTA polls, and returns.
//
// The reference gets the same effect from compiling its decode layers into one MLX graph
// (crates/pmetal-bridge/cpp/bridge_compiled.cpp:213-400, crates/pmetal-bridge/src/compile.rs:3-8).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "host_util.cuh"
#include <stdlib.h>

#include "pdl.cuh"
#include "pmetal_b200.h"

namespace pm {

constexpr int kDmThreads = 256;
constexpr int kDmWarps = 8;
constexpr int kDmPad = 32;            // row padding of staged activations (bank spread for the fragment loads)
constexpr int kDmMaxNT = 4;           // output tiles a CTA works on at once
constexpr int kDmPre = 24;            // weight loads a lane keeps in flight across a barrier
constexpr int kStatusDecodeBarrier = 109;
constexpr unsigned long long kDmBarrierLimitNs = 1000000000ull;   // 1 s

struct DmLayer {
  const __nv_bfloat16* ln1;
  const __nv_bfloat16* wqkv;     // [(hq + 2 hkv) * 128, H]
  const __nv_bfloat16* qn;       // [128] or null
  const __nv_bfloat16* kn;
  const __nv_bfloat16* wo;       // [H, hq * 128]
  const __nv_bfloat16* ln2;
  const __nv_bfloat16* wgu;      // [2 I, H]: gate rows then up rows
  const __nv_bfloat16* wdown;    // [H, I]
  __nv_bfloat16* kc;             // [blocks, 64, hkv, 128]
  __nv_bfloat16* vc;
};

struct DmParams {
  const DmLayer* layers;
  int n_layers;
  int M, H, hq, hkv, I;
  float eps, scale;
  __nv_bfloat16* x;              // [M, H] in: embeddings, out: last layer's output
  __nv_bfloat16* h;              // [M, H]
  __nv_bfloat16* qkv;            // [M, (hq + 2 hkv) * 128]
  __nv_bfloat16* attn;           // [M, hq * 128]
  __nv_bfloat16* act;            // [M, I]
  float* part_o;                 // [n_split, M, hq, 128]
  float* part_ml;                // [n_split, M, hq, 2]
  unsigned* counters;            // [M * hkv] arrival counters of the attention splits (zero between uses)
  const float* cs;               // [M, 64] rotary cos / sin of every row's position
  const float* sn;
  const int* block_table;        // [M, max_blocks]
  const int* seq_lens;           // [M] keys including the new token
  const long long* slots;        // [M] cache slot of the new token
  int max_blocks, n_split;
  unsigned* bar;                 // [0] arrivals (zero at launch), [1] abort word
  int* status;
  unsigned long long* trace;     // optional [n_layers * 16] timestamps taken by CTA 0 (phase starts, ends, barrier exits)
};

__device__ __forceinline__ unsigned dm_ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long dm_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ float dm_warp_sum(float v) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float dm_warp_max(float v) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ void dm_mma(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Returns false when the step was abandoned (another CTA or this one ran into the wait limit).
__device__ __forceinline__ bool dm_grid_barrier(const DmParams& p, unsigned& epoch, int* s_flag) {
  __syncthreads();
  if (threadIdx.x == 0) {
    ++epoch;
    const unsigned target = epoch * gridDim.x;
    __threadfence();
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.bar) : "memory");
    unsigned long long t0 = 0;     // the global timer is slow to read: first looked at after 1024 failed polls
    unsigned spins = 0;
    int ok = 1;
    while (static_cast<int>(dm_ld_acquire(p.bar) - target) < 0) {
      if ((++spins & 63u) == 0u) {
        if (dm_ld_acquire(p.bar + 1) != 0u) { ok = 0; break; }
        bool late = false;
        if (spins >= 1024u) {
          const unsigned long long now = dm_now();
          if (t0 == 0) t0 = now;
          late = now - t0 > kDmBarrierLimitNs;
        }
        if (late) {
          atomicCAS(p.status, 0, kStatusDecodeBarrier);
          atomicExch(p.bar + 1, 1u);
          ok = 0;
          break;
        }
      }
    }
    *s_flag = ok;
  }
  __syncthreads();
  return *s_flag != 0;
}

// Stage M rows of `src` ([M, K], written by other CTAs) into shared memory rows of stride `lds`, optionally
// RMS-normalised. Rows >= M are zeroed once at kernel start and never written again.
__device__ __forceinline__ void dm_stage(__nv_bfloat16* sx, int lds, float* s_rstd, const __nv_bfloat16* src, int M,
                                         int K, const __nv_bfloat16* norm_w, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (norm_w) {
    for (int m = warp; m < M; m += kDmWarps) {
      float ss = 0.f;
      for (int k0 = lane * 8; k0 < K; k0 += 1024) {
        uint4 raw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          raw[u] = k0 + u * 256 < K ? __ldcg(reinterpret_cast<const uint4*>(src + static_cast<long long>(m) * K + k0 + u * 256))
                                    : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h2[e]);
            ss += f.x * f.x + f.y * f.y;
          }
        }
      }
      ss = dm_warp_sum(ss);
      if (lane == 0) s_rstd[m] = rsqrtf(ss / static_cast<float>(K) + eps);
    }
    __syncthreads();
  }
  const int per_row = K / 8, total = M * per_row;
  for (int i0 = threadIdx.x; i0 < total; i0 += kDmThreads * 4) {
    uint4 raw[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * kDmThreads;
      if (i < total) {
        const int m = i / per_row, k = (i - m * per_row) * 8;
        raw[u] = __ldcg(reinterpret_cast<const uint4*>(src + static_cast<long long>(m) * K + k));
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * kDmThreads;
      if (i >= total) break;
      const int m = i / per_row, k = (i - m * per_row) * 8;
      if (norm_w) {
        const uint4 nw = __ldg(reinterpret_cast<const uint4*>(norm_w + k));
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw[u]);
        const __nv_bfloat162* n2 = reinterpret_cast<const __nv_bfloat162*>(&nw);
        const float rs = s_rstd[m];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h2[e]), g = __bfloat1622float2(n2[e]);
          const float a = __bfloat162float(__float2bfloat16(f.x * rs)) * g.x;     // rounding points of the RMSNorm kernel
          const float b = __bfloat162float(__float2bfloat16(f.y * rs)) * g.y;
          h2[e] = __floats2bfloat162_rn(a, b);
        }
      }
      *reinterpret_cast<uint4*>(sx + static_cast<long long>(m) * lds + k) = raw[u];
    }
  }
  __syncthreads();
}

// Ask L2 for the weight rows of the tiles this CTA will work on in a mat-vec phase over w [N (x2), K].
__device__ __forceinline__ void dm_prefetch_tiles(const __nv_bfloat16* w, int N, int K, bool two_halves) {
  const int n_tiles = (N + 7) / 8;
  const int per_tile = two_halves ? 16 : 8;
  for (int idx = threadIdx.x; idx < kDmMaxNT * per_tile; idx += kDmThreads) {
    const int tile = blockIdx.x + (idx / per_tile) * gridDim.x;
    if (tile >= n_tiles) break;
    const int j = idx % per_tile;
    const int n = tile * 8 + (j & 7);
    if (n >= N) continue;
    l2_prefetch_bulk(w + (static_cast<long long>(n) + (j >= 8 ? N : 0)) * K, static_cast<unsigned>(K) * 2u);
  }
}

// First batch of weight loads of a mat-vec phase (tiles base .. of this CTA, chunks r0 = 0 ..): issued before the grid
// barrier that precedes the phase, consumed by dm_matvec after it. pre holds NT x RB loads (two halves of NT x RB / 2
// each for SwiGLU), up to kDmPre per lane.
template <int NT, int RB, bool SWIGLU>
__device__ __forceinline__ void dm_load_batch(const __nv_bfloat16* __restrict__ w, int N, int K, int base, int r0,
                                              uint4 (&pre)[kDmPre]) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane & 3, col = lane >> 2;
  const int n_tiles = (N + 7) / 8, rounds = (K + 255) / 256;
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int tile = base + j * gridDim.x;
    const int n = min(tile * 8 + col, N - 1);
    const __nv_bfloat16* wr = w + static_cast<long long>(n) * K;
#pragma unroll
    for (int u = 0; u < RB; ++u) {
      const int k = ((r0 + u) * kDmWarps + warp) * 32 + g * 8;
      const bool ok = tile < n_tiles && r0 + u < rounds && k < K;
      pre[j * RB + u] = ok ? __ldg(reinterpret_cast<const uint4*>(wr + k)) : make_uint4(0u, 0u, 0u, 0u);
      if (SWIGLU)
        pre[NT * RB + j * RB + u] = ok ? __ldg(reinterpret_cast<const uint4*>(wr + static_cast<long long>(N) * K + k))
                                 : make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

// y[m, n] = epi(sum_k sx[m][k] w[n][k]). A CTA owns NT tiles of 8 columns at a time; warp w takes the 32-wide k chunks
// w, w + 8, ... of all of them, RB chunks per tile are loaded before the MMAs that use them, and the partial
// accumulators of the 8 warps are summed through `red`. Fragment slot assignment: lane group g = lane % 4 holds
// k = 8 g .. 8 g + 7 of a chunk for column lane / 4; MMA j of the chunk contracts k = 8 g + 4 j + {0, 1} and {2, 3}.
template <int NT, int RB, bool SWIGLU, typename Epi>
__device__ __forceinline__ void dm_matvec(const __nv_bfloat16* sx, int lds, const __nv_bfloat16* __restrict__ w, int N,
                                          int K, int M, float* red, uint4 (&pre)[kDmPre], Epi epi) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane & 3, col = lane >> 2;
  const int n_tiles = (N + 7) / 8;
  const int rounds = (K + 255) / 256;
  bool first = true;
  for (int base = blockIdx.x; base < n_tiles; base += NT * gridDim.x) {
    float c[NT][4], c2[SWIGLU ? NT : 1][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      c[j][0] = c[j][1] = c[j][2] = c[j][3] = 0.f;
      if (SWIGLU) c2[j][0] = c2[j][1] = c2[j][2] = c2[j][3] = 0.f;
    }
    for (int r0 = 0; r0 < rounds; r0 += RB) {
      if (!first) dm_load_batch<NT, RB, SWIGLU>(w, N, K, base, r0, pre);
      first = false;
#pragma unroll
      for (int u = 0; u < RB; ++u) {
        const int k = ((r0 + u) * kDmWarps + warp) * 32 + g * 8;
        if (r0 + u >= rounds || k >= K) break;
        const uint4 xa = *reinterpret_cast<const uint4*>(sx + col * lds + k);
        const uint4 xb = *reinterpret_cast<const uint4*>(sx + (col + 8) * lds + k);
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          const uint4 wv = pre[j * RB + u];
          dm_mma(c[j], xa.x, xb.x, xa.y, xb.y, wv.x, wv.y);
          dm_mma(c[j], xa.z, xb.z, xa.w, xb.w, wv.z, wv.w);
          if (SWIGLU) {
            const uint4 wv2 = pre[NT * RB + j * RB + u];
            dm_mma(c2[j], xa.x, xb.x, xa.y, xb.y, wv2.x, wv2.y);
            dm_mma(c2[j], xa.z, xb.z, xa.w, xb.w, wv2.z, wv2.w);
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      float* my = red + ((warp * kDmMaxNT + j) * 2) * 128;
      *reinterpret_cast<float4*>(my + lane * 4) = make_float4(c[j][0], c[j][1], c[j][2], c[j][3]);
      if (SWIGLU) *reinterpret_cast<float4*>(my + 128 + lane * 4) = make_float4(c2[j][0], c2[j][1], c2[j][2], c2[j][3]);
    }
    __syncthreads();
    for (int j = threadIdx.x >> 7; j < NT; j += 2) {
      const int tile = base + j * gridDim.x;
      if (tile >= n_tiles) break;
      const int e = threadIdx.x & 127;
      float v = 0.f, v2 = 0.f;
#pragma unroll
      for (int ww = 0; ww < kDmWarps; ++ww) {
        v += red[((ww * kDmMaxNT + j) * 2) * 128 + e];
        if (SWIGLU) v2 += red[((ww * kDmMaxNT + j) * 2 + 1) * 128 + e];
      }
      const int src = e >> 2, reg = e & 3;
      const int m = (src >> 2) + ((reg & 2) ? 8 : 0), n = tile * 8 + (src & 3) * 2 + (reg & 1);
      if (m < M && n < N) epi(m, n, v, v2);
    }
    __syncthreads();
  }
}

// Runtime choice of how many tiles a CTA keeps in flight: as many as 16 weight loads per lane allow. The same choice
// is made by the preload before the barrier and by the phase after it.
template <bool SWIGLU>
__device__ __forceinline__ void dm_preload(const __nv_bfloat16* w, int N, int K, uint4 (&pre)[kDmPre]) {
  const int rounds = (K + 255) / 256;
  if (SWIGLU) {
    if (rounds <= 4) dm_load_batch<3, 4, true>(w, N, K, blockIdx.x, 0, pre);
    else dm_load_batch<1, 8, true>(w, N, K, blockIdx.x, 0, pre);
  } else {
    if (rounds <= 4) dm_load_batch<4, 4, false>(w, N, K, blockIdx.x, 0, pre);
    else if (rounds <= 8) dm_load_batch<2, 8, false>(w, N, K, blockIdx.x, 0, pre);
    else dm_load_batch<1, 16, false>(w, N, K, blockIdx.x, 0, pre);
  }
}
template <bool SWIGLU, typename Epi>
__device__ __forceinline__ void dm_matvec_auto(const __nv_bfloat16* sx, int lds, const __nv_bfloat16* w, int N, int K,
                                               int M, float* red, uint4 (&pre)[kDmPre], Epi epi) {
  const int rounds = (K + 255) / 256;
  if (SWIGLU) {
    if (rounds <= 4) dm_matvec<3, 4, true>(sx, lds, w, N, K, M, red, pre, epi);
    else dm_matvec<1, 8, true>(sx, lds, w, N, K, M, red, pre, epi);
  } else {
    if (rounds <= 4) dm_matvec<4, 4, false>(sx, lds, w, N, K, M, red, pre, epi);
    else if (rounds <= 8) dm_matvec<2, 8, false>(sx, lds, w, N, K, M, red, pre, epi);
    else dm_matvec<1, 16, false>(sx, lds, w, N, K, M, red, pre, epi);
  }
}

// Per-head RMSNorm (optional) and rotary embedding of one 128-wide head held as 4 values per lane (dims 4 lane ..).
// nwr: the lane's four norm weights (raw bf16), c / s: the lane's cos / sin values; all loaded by the caller up front.
__device__ __forceinline__ void dm_norm_rope(float x[4], bool has_norm, uint2 nwr, float eps, float4 c, float4 s,
                                             int lane) {
  if (has_norm) {
    const float ss = dm_warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3]);
    const float rs = rsqrtf(ss / 128.f + eps);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&nwr.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&nwr.y));
    x[0] *= rs * a.x; x[1] *= rs * a.y; x[2] *= rs * b.x; x[3] *= rs * b.y;
  }
  const float cc[4] = {c.x, c.y, c.z, c.w}, ss4[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float partner = __shfl_xor_sync(0xffffffffu, x[i], 16);
    const float o = (lane < 16) ? (x[i] * cc[i] - partner * ss4[i]) : (x[i] * cc[i] + partner * ss4[i]);
    x[i] = __bfloat162float(__float2bfloat16(o));      // what the bf16 q tensor / key cache would hold
  }
}
__device__ __forceinline__ void dm_unpack4(const uint2 raw, float x[4]) {
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
}
__device__ __forceinline__ uint2 dm_pack4(const float x[4]) {
  uint2 o;
  *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(x[0], x[1]);
  *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(x[2], x[3]);
  return o;
}

// Attention of one new token per row over the paged cache. One CTA per (row, kv head, key split); the CTA's warps
// take interleaved groups of eight keys (all sixteen loads of a group are issued before the arithmetic), merge their
// running (max, sum, output) through shared memory, and REP query heads of the kv head are processed together.
// `sm` is scratch of at least 8 * REP * 132 floats.
// Splits actually used for a row: one per 64 cached keys (eight warps x one group of eight keys, all requested before
// the barrier), so that short contexts need no second round of key loads and few partial results to merge.
__device__ __forceinline__ int dm_eff_splits(int cached, int ns) { return max(1, min(ns, (cached + 63) / 64)); }

// First group of eight keys / values of this CTA's first attention item, requested before the barrier that precedes
// the attention phase (cached keys do not depend on the projections of the current step).
__device__ __forceinline__ void dm_attn_preload(const DmParams& p, const DmLayer& L, uint2 (&pk)[8], uint2 (&pv)[8]) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hkv = p.hkv, ns = p.n_split;
  const int it = blockIdx.x;
  if (it >= p.M * hkv * ns) return;
  const int split = it % ns, kvh = (it / ns) % hkv, m = it / (ns * hkv);
  const int cached = __ldg(p.seq_lens + m) - 1;
  const int nse = dm_eff_splits(cached, ns);
  if (split >= nse) return;
  const int per = (cached + nse - 1) / nse;
  const int j0 = min(split * per, cached), j1 = min(j0 + per, cached);
  const int jb = j0 + warp * 8;
  if (jb >= j1) return;
  const int* table = p.block_table + static_cast<long long>(m) * p.max_blocks;
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int j = min(jb + u, j1 - 1);
    const long long sl = static_cast<long long>(__ldg(table + (j >> 6))) * 64 + (j & 63);
    pk[u] = __ldcg(reinterpret_cast<const uint2*>(L.kc + (sl * hkv + kvh) * 128 + lane * 4));
    pv[u] = __ldcg(reinterpret_cast<const uint2*>(L.vc + (sl * hkv + kvh) * 128 + lane * 4));
  }
}

template <int REP>
__device__ __forceinline__ void dm_attention(const DmParams& p, const DmLayer& L, float* sm, uint2 (&pk)[8],
                                             uint2 (&pv)[8]) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hq = p.hq, hkv = p.hkv, ns = p.n_split;
  const int ld = (hq + 2 * hkv) * 128;
  const int items = p.M * hkv * ns;
  __shared__ int s_last;
  for (int it = blockIdx.x; it < items; it += gridDim.x) {
    const int split = it % ns, kvh = (it / ns) % hkv, m = it / (ns * hkv);
    const int kv_len = __ldg(p.seq_lens + m);
    const int nse = dm_eff_splits(kv_len - 1, ns);      // CTA-uniform
    if (split >= nse) continue;
    const long long slot = __ldg(p.slots + m);
    const __nv_bfloat16* row = p.qkv + static_cast<long long>(m) * ld;
    const float* cs = p.cs + static_cast<long long>(m) * 64;
    const float* sn = p.sn + static_cast<long long>(m) * 64;
    // every global value this item needs besides the cached keys is requested here, before the first use
    const bool newtok = split == nse - 1 && warp == kDmWarps - 1;
    uint2 qraw[REP];
#pragma unroll
    for (int r = 0; r < REP; ++r) qraw[r] = __ldcg(reinterpret_cast<const uint2*>(row + (kvh * REP + r) * 128 + lane * 4));
    uint2 kraw = make_uint2(0u, 0u), vraw = make_uint2(0u, 0u);
    if (newtok) {
      kraw = __ldcg(reinterpret_cast<const uint2*>(row + (hq + kvh) * 128 + lane * 4));
      vraw = __ldcg(reinterpret_cast<const uint2*>(row + (hq + hkv + kvh) * 128 + lane * 4));
    }
    const uint2 qnw = L.qn ? __ldg(reinterpret_cast<const uint2*>(L.qn + lane * 4)) : make_uint2(0u, 0u);
    const uint2 knw = L.kn ? __ldg(reinterpret_cast<const uint2*>(L.kn + lane * 4)) : make_uint2(0u, 0u);
    const float4 cs4 = __ldg(reinterpret_cast<const float4*>(cs + (lane & 15) * 4));
    const float4 sn4 = __ldg(reinterpret_cast<const float4*>(sn + (lane & 15) * 4));
    float q[REP][4];
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      dm_unpack4(qraw[r], q[r]);
      dm_norm_rope(q[r], L.qn != nullptr, qnw, p.eps, cs4, sn4, lane);
    }
    // cached keys [0, kv_len - 1) are divided among the splits; the new key belongs to the last split
    const int cached = kv_len - 1;
    const int per = (cached + nse - 1) / nse;
    const int j0 = min(split * per, cached), j1 = min(j0 + per, cached);
    float mx[REP], l[REP], acc[REP][4];
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      mx[r] = -INFINITY;
      l[r] = 0.f;
      acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;
    }
    auto visit = [&](const float kx[4], const float vx[4]) {
#pragma unroll
      for (int r = 0; r < REP; ++r) {
        const float s = dm_warp_sum(q[r][0] * kx[0] + q[r][1] * kx[1] + q[r][2] * kx[2] + q[r][3] * kx[3]) * p.scale;
        const float mn = fmaxf(mx[r], s);
        const float corr = __expf(mx[r] - mn), pe = __expf(s - mn);
        l[r] = l[r] * corr + pe;
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[r][i] = acc[r][i] * corr + pe * vx[i];
        mx[r] = mn;
      }
    };
    const int* table = p.block_table + static_cast<long long>(m) * p.max_blocks;
    for (int jb = j0 + warp * 8; jb < j1; jb += kDmWarps * 8) {
      uint2 kr[8], vr[8];
      if (it == static_cast<int>(blockIdx.x) && jb == j0 + warp * 8) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          kr[u] = pk[u];
          vr[u] = pv[u];
        }
      } else {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int j = min(jb + u, j1 - 1);
          const long long sl = static_cast<long long>(__ldg(table + (j >> 6))) * 64 + (j & 63);
          kr[u] = __ldcg(reinterpret_cast<const uint2*>(L.kc + (sl * hkv + kvh) * 128 + lane * 4));
          vr[u] = __ldcg(reinterpret_cast<const uint2*>(L.vc + (sl * hkv + kvh) * 128 + lane * 4));
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (jb + u >= j1) break;
        float kx[4], vx[4];
        dm_unpack4(kr[u], kx);
        dm_unpack4(vr[u], vx);
        visit(kx, vx);
      }
    }
    if (newtok) {   // the new token: normalise / rotate k, append k and v to the cache, attend to it
      float kx[4], vx[4];
      dm_unpack4(kraw, kx);
      dm_unpack4(vraw, vx);
      dm_norm_rope(kx, L.kn != nullptr, knw, p.eps, cs4, sn4, lane);
      if (slot >= 0) {
        *reinterpret_cast<uint2*>(L.kc + (slot * hkv + kvh) * 128 + lane * 4) = dm_pack4(kx);
        *reinterpret_cast<uint2*>(L.vc + (slot * hkv + kvh) * 128 + lane * 4) = vraw;
      }
      visit(kx, vx);
    }
    // ---- merge the warps of the CTA: sm[(warp * REP + r) * 132 + {0..127: acc, 128: max, 129: sum}]
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      float* d = sm + (warp * REP + r) * 132;
      *reinterpret_cast<float4*>(d + lane * 4) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
      if (lane == 0) {
        d[128] = mx[r];
        d[129] = l[r];
      }
    }
    __syncthreads();
    if (warp < REP) {
      const int r = warp, head = kvh * REP + r;
      float mm = -INFINITY;
#pragma unroll
      for (int ww = 0; ww < kDmWarps; ++ww) mm = fmaxf(mm, sm[(ww * REP + r) * 132 + 128]);
      float lt = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ww = 0; ww < kDmWarps; ++ww) {
        const float* d = sm + (ww * REP + r) * 132;
        const float wgt = d[128] == -INFINITY ? 0.f : __expf(d[128] - mm);
        const float4 po = *reinterpret_cast<const float4*>(d + lane * 4);
        lt += d[129] * wgt;
        o[0] += po.x * wgt; o[1] += po.y * wgt; o[2] += po.z * wgt; o[3] += po.w * wgt;
      }
      if (nse == 1) {
        const float inv = lt > 0.f ? 1.f / lt : 0.f;
        o[0] *= inv; o[1] *= inv; o[2] *= inv; o[3] *= inv;
        *reinterpret_cast<uint2*>(p.attn + (static_cast<long long>(m) * hq + head) * 128 + lane * 4) = dm_pack4(o);
      } else {
        const long long pr = (static_cast<long long>(split) * p.M + m) * hq + head;
        *reinterpret_cast<float4*>(p.part_o + pr * 128 + lane * 4) = make_float4(o[0], o[1], o[2], o[3]);
        if (lane == 0) *reinterpret_cast<float2*>(p.part_ml + pr * 2) = make_float2(mm, lt);
      }
    }
    if (nse > 1) {
      // the CTA that arrives last merges all splits of this (row, kv head)
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(p.counters + m * hkv + kvh, 1u);
        s_last = prev == static_cast<unsigned>(nse - 1);
        if (s_last) p.counters[m * hkv + kvh] = 0u;
      }
      __syncthreads();
      if (s_last && warp < REP) {
        __threadfence();
        const int head = kvh * REP + warp;
        // lanes take the splits' (max, sum) pairs, then every lane folds its four output dims over the splits
        float mloc = -INFINITY;
        for (int s = lane; s < nse; s += 32)
          mloc = fmaxf(mloc, __ldcg(p.part_ml + ((static_cast<long long>(s) * p.M + m) * hq + head) * 2));
        const float mm = dm_warp_max(mloc);
        float lt = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};
        for (int s0 = 0; s0 < nse; s0 += 8) {
          float4 po[8];
          float2 ml[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const long long pr = (static_cast<long long>(min(s0 + u, nse - 1)) * p.M + m) * hq + head;
            ml[u] = __ldcg(reinterpret_cast<const float2*>(p.part_ml + pr * 2));
            po[u] = __ldcg(reinterpret_cast<const float4*>(p.part_o + pr * 128 + lane * 4));
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            if (s0 + u >= nse) break;
            const float wgt = ml[u].x == -INFINITY ? 0.f : __expf(ml[u].x - mm);
            lt += ml[u].y * wgt;
            o[0] += po[u].x * wgt; o[1] += po[u].y * wgt; o[2] += po[u].z * wgt; o[3] += po[u].w * wgt;
          }
        }
        const float inv = lt > 0.f ? 1.f / lt : 0.f;
        o[0] *= inv; o[1] *= inv; o[2] *= inv; o[3] *= inv;
        *reinterpret_cast<uint2*>(p.attn + (static_cast<long long>(m) * hq + head) * 128 + lane * 4) = dm_pack4(o);
      }
    }
    __syncthreads();
  }
}

__device__ __forceinline__ float dm_ldcg_bf16(const __nv_bfloat16* q) {
  return __bfloat162float(__ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(q))));
}
__device__ __forceinline__ float dm_silu(float v) { return v / (1.f + __expf(-v)); }

__global__ void __launch_bounds__(kDmThreads, 1) decode_layers_kernel(const DmParams p) {
  extern __shared__ __align__(16) uint8_t dm_smem[];
  const int kmax = max(p.H, max(p.hq * 128, p.I));
  const int lds = kmax + kDmPad;
  __nv_bfloat16* sx = reinterpret_cast<__nv_bfloat16*>(dm_smem);                                     // [16][lds]
  float* red = reinterpret_cast<float*>(dm_smem + static_cast<size_t>(16) * lds * 2);                  // 32 KB
  __shared__ float s_rstd[16];
  __shared__ int s_flag;
  unsigned epoch = 0;
  int tix = 0;
  auto stamp = [&]() {
    if (p.trace && blockIdx.x == 0 && threadIdx.x == 0) p.trace[tix] = dm_now();
    ++tix;
  };
  const int qkv_n = (p.hq + 2 * p.hkv) * 128, qd = p.hq * 128;
  const int rep = p.hq / p.hkv;
  uint4 pre[kDmPre];
  uint2 pk[8], pv[8];
  dm_preload<false>(p.layers[0].wqkv, qkv_n, p.H, pre);
  for (int i = threadIdx.x; i < (16 - p.M) * (lds / 8); i += kDmThreads)      // rows >= M stay zero for the whole step
    *reinterpret_cast<uint4*>(sx + static_cast<long long>(p.M) * lds + static_cast<long long>(i) * 8) = make_uint4(0u, 0u, 0u, 0u);
  for (int li = 0; li < p.n_layers; ++li) {
    const DmLayer L = p.layers[li];
    // ---- P1: qkv
    tix = li * 16;
    stamp();
    dm_stage(sx, lds, s_rstd, p.x, p.M, p.H, L.ln1, p.eps);
    stamp();
    dm_matvec_auto<false>(sx, lds, L.wqkv, qkv_n, p.H, p.M, red, pre, [&](int m, int n, float v, float) {
      p.qkv[static_cast<long long>(m) * qkv_n + n] = __float2bfloat16(v);
    });
    dm_attn_preload(p, L, pk, pv);
    dm_prefetch_tiles(L.wo, p.H, qd, false);
    stamp();
    if (!dm_grid_barrier(p, epoch, &s_flag)) return;
    stamp();
    // ---- P2: attention (+ cache append)
    if (rep == 1) dm_attention<1>(p, L, red, pk, pv);
    else if (rep == 2) dm_attention<2>(p, L, red, pk, pv);
    else dm_attention<4>(p, L, red, pk, pv);
    dm_preload<false>(L.wo, p.H, qd, pre);
    dm_prefetch_tiles(L.wgu, p.I, p.H, true);
    stamp();
    if (!dm_grid_barrier(p, epoch, &s_flag)) return;
    stamp();
    // ---- P3: h = x + attn Wo^T
    dm_stage(sx, lds, s_rstd, p.attn, p.M, qd, nullptr, p.eps);
    stamp();
    dm_matvec_auto<false>(sx, lds, L.wo, p.H, qd, p.M, red, pre, [&](int m, int n, float v, float) {
      const long long i = static_cast<long long>(m) * p.H + n;
      p.h[i] = __float2bfloat16(v + dm_ldcg_bf16(p.x + i));
    });
    dm_preload<true>(L.wgu, p.I, p.H, pre);
    dm_prefetch_tiles(L.wdown, p.H, p.I, false);
    stamp();
    if (!dm_grid_barrier(p, epoch, &s_flag)) return;
    stamp();
    // ---- P4: act = SwiGLU(norm(h) Wgu^T)
    dm_stage(sx, lds, s_rstd, p.h, p.M, p.H, L.ln2, p.eps);
    stamp();
    dm_matvec_auto<true>(sx, lds, L.wgu, p.I, p.H, p.M, red, pre, [&](int m, int n, float v, float v2) {
      p.act[static_cast<long long>(m) * p.I + n] = __float2bfloat16(dm_silu(v) * v2);
    });
    dm_preload<false>(L.wdown, p.H, p.I, pre);
    if (li + 1 < p.n_layers) dm_prefetch_tiles(p.layers[li + 1].wqkv, qkv_n, p.H, false);
    stamp();
    if (!dm_grid_barrier(p, epoch, &s_flag)) return;
    stamp();
    // ---- P5: x = h + act Wdown^T
    dm_stage(sx, lds, s_rstd, p.act, p.M, p.I, nullptr, p.eps);
    stamp();
    dm_matvec_auto<false>(sx, lds, L.wdown, p.H, p.I, p.M, red, pre, [&](int m, int n, float v, float) {
      const long long i = static_cast<long long>(m) * p.H + n;
      p.x[i] = __float2bfloat16(v + dm_ldcg_bf16(p.h + i));
    });
    if (li + 1 < p.n_layers) dm_preload<false>(p.layers[li + 1].wqkv, qkv_n, p.H, pre);
    stamp();
    if (!dm_grid_barrier(p, epoch, &s_flag)) return;
    stamp();
  }
}

}  // namespace pm

using namespace pm;

static size_t dm_smem_bytes(int H, int hq, int I) {
  const int kmax = max(H, max(hq * 128, I));
  return static_cast<size_t>(16) * (kmax + kDmPad) * 2 + static_cast<size_t>(kDmWarps) * kDmMaxNT * 2 * 128 * sizeof(float);
}

// 1 when one launch can run the step: up to 16 rows, 1 / 2 / 4 query heads per kv head, reduction sizes that are
// multiples of 32, and the staged activations fit in shared memory.
extern "C" int pm_decode_layers_supported(int M, int H, int hq, int hkv, int I) {
  if (M < 1 || M > 16 || hkv < 1 || hq % hkv) return 0;
  const int rep = hq / hkv;
  if (rep != 1 && rep != 2 && rep != 4) return 0;
  if ((H % 32) || (I % 32)) return 0;
  return dm_smem_bytes(H, hq, I) <= 200 * 1024 ? 1 : 0;
}

// layers: device array of n_layers DmLayer records (10 pointers each). bar: 2 words, counters: M * hkv words, all zero
// at launch (a completed launch leaves the counters zero; the caller clears bar before every launch).
extern "C" int pm_decode_layers(const void* layers, int n_layers, int M, int H, int hq, int hkv, int I, float eps,
                                float scale, void* x, void* h, void* qkv, void* attn, void* act, float* part_o,
                                float* part_ml, unsigned* counters, const float* cs, const float* sn,
                                const int* block_table, const int* seq_lens, const long long* slots, int max_blocks,
                                int n_split, unsigned* bar, int* status, unsigned long long* trace,
                                cudaStream_t st) {
  if (!pm_decode_layers_supported(M, H, hq, hkv, I) || n_split < 1) return -1;
  DmParams p{};
  p.layers = static_cast<const DmLayer*>(layers);
  p.n_layers = n_layers;
  p.M = M; p.H = H; p.hq = hq; p.hkv = hkv; p.I = I; p.eps = eps; p.scale = scale;
  p.x = static_cast<__nv_bfloat16*>(x); p.h = static_cast<__nv_bfloat16*>(h);
  p.qkv = static_cast<__nv_bfloat16*>(qkv); p.attn = static_cast<__nv_bfloat16*>(attn);
  p.act = static_cast<__nv_bfloat16*>(act);
  p.part_o = part_o; p.part_ml = part_ml; p.counters = counters; p.cs = cs; p.sn = sn;
  p.block_table = block_table; p.seq_lens = seq_lens; p.slots = slots; p.max_blocks = max_blocks; p.n_split = n_split;
  p.bar = bar; p.status = status; p.trace = trace;
  const size_t smem = dm_smem_bytes(H, hq, I);
  const void* fn = reinterpret_cast<const void*>(decode_layers_kernel);
  static DeviceMax configured;
  if (smem > 40 * 1024 && smem > configured.get()) {
    cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured.set(200 * 1024);
  }
  int dev = 0, sms = 0, per_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_layers_kernel, kDmThreads, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (per_sm < 1) return -2;      // the cooperative grid of one CTA per SM would not be co-resident
  void* args[] = {&p};
  e = cudaLaunchCooperativeKernel(fn, dim3(sms), dim3(kDmThreads), args, smem, st);
  return static_cast<int>(e);
}
