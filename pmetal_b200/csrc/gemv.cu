// Skinny linear layers for decode: y[M, N] = f(x)[M, K] * W[N, K]^T for M <= 16 rows.
//
// A decode step multiplies a handful of token rows by every weight matrix of the model: the work is one pass over the
// weights and is bound by HBM bandwidth, so tensor cores (and the 128-row tiles they want) buy nothing. Each warp owns
// a few output columns and streams their weight rows with 16-byte loads while all M activations sit in shared memory;
// partial sums are reduced with warp shuffles. Around that core the kernel fuses what a decoder layer needs, so a layer
// is six launches instead of a dozen:
//   * RMSNorm prologue: x is normalised (and scaled by the norm weight) while it is staged into shared memory
//   * SwiGLU epilogue: with gate rows [0, I) and up rows [I, 2I) a warp computes column j of both and stores
//     silu(g) * u, so the [M, 2I] intermediate never exists
//   * residual add
//   * LoRA: y += t[:, seg*r : (seg+1)*r] . B[n, :] with t = s * x A^T from a small launch of this same kernel
// The reference's decode path has the same shape (compiled fused layers, crates/pmetal-bridge/cpp/bridge_compiled.cpp:213-400;
// fused gate/up + SwiGLU and dequant mat-vec Metal kernels, crates/pmetal-metal/src/kernels/metal/fused_moe.metal).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "host_util.cuh"

#include "pdl.cuh"
#include "pmetal_b200.h"

namespace pm {

constexpr int kGvThreads = 256;
constexpr int kGvWarps = kGvThreads / 32;

struct GemvParams {
  const __nv_bfloat16* x;        // [M, ldx]
  int ldx;
  const __nv_bfloat16* w;        // [N_w, K] row-major (N_w = 2 * N when swiglu)
  int ldw;
  const __nv_bfloat16* norm_w;   // [K] or null: RMSNorm prologue
  float eps;
  const __nv_bfloat16* residual; // [M, ldr] or null
  int ldr;
  __nv_bfloat16* y;              // [M, ldy]
  int ldy;
  int M, N, K;                   // N = output columns
  int swiglu;                    // 1: y[:, j] = silu(x w_j) * (x w_{N + j})
  float alpha;
  // LoRA (all null / 0 when unused): t [M, ldt] bf16 (scale folded in), lora_b [N_w, r] fp32
  const __nv_bfloat16* t;
  int ldt;
  const float* lora_b;
  int r;
  int seg_end[4];                // cumulative output-row boundaries of the stacked projections (0x7fffffff padding)
  int prefetch_iters;            // groups per warp whose weight rows are pulled into L2 before the dependency wait
  // 4-bit weights (NF4 / FP4 codes, two per byte, first element in the high nibble; w is null then)
  const uint8_t* qdata;          // [N_w * K / 2]
  const float* absmax;           // per block, or null when double-quantised
  const uint8_t* absmax_q;
  float am_scale, am_offset;
  int qblock;                    // elements per absmax block (multiple of 32)
  int fp4;
};

__device__ __forceinline__ float gv_silu(float v) { return v / (1.f + __expf(-v)); }

// MR rows of x, C output columns per warp at a time, KU 16-byte weight loads in flight per column and lane.
template <int MR, int C, int KU, bool SWIGLU>
__global__ void __launch_bounds__(kGvThreads) gemv_kernel(const GemvParams p) {
  extern __shared__ __align__(16) uint8_t gv_smem[];
  __nv_bfloat16* sx = reinterpret_cast<__nv_bfloat16*>(gv_smem);   // [MR][K] (rows >= M are zero)
  __shared__ float s_rstd[MR];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = p.K;
  const int n_groups = (p.N + C - 1) / C;

  // ---- before the previous kernel's output is needed: let the next kernel be scheduled, and start pulling this
  // warp's first weight rows into L2 (weights do not depend on the previous kernel)
  pdl_launch_dependents();
  {
    const int per_group = C * (SWIGLU ? 2 : 1);
    const unsigned row_bytes = static_cast<unsigned>(K) * 2u;
    for (int idx = lane; idx < p.prefetch_iters * per_group; idx += 32) {
      const int it = idx / per_group, j = idx - it * per_group;
      const int g = blockIdx.x * kGvWarps + warp + it * gridDim.x * kGvWarps;
      if (g >= n_groups) continue;
      const int n = min(g * C + (j % C), p.N - 1) + (j >= C ? p.N : 0);
      l2_prefetch_bulk(p.w + static_cast<long long>(n) * p.ldw, row_bytes);
    }
  }
  pdl_wait();

  // ---- stage x (optionally RMS-normalised) into shared memory
  if (p.norm_w) {
    for (int m = warp; m < MR; m += kGvWarps) {
      float ss = 0.f;
      if (m < p.M)
        for (int k = lane * 8; k < K; k += 256) {
          const uint4 raw = *reinterpret_cast<const uint4*>(p.x + static_cast<long long>(m) * p.ldx + k);
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h2[e]);
            ss += f.x * f.x + f.y * f.y;
          }
        }
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) s_rstd[m] = rsqrtf(ss / static_cast<float>(K) + p.eps);
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < MR * (K / 8); i += kGvThreads) {
    const int m = i / (K / 8), k = (i - m * (K / 8)) * 8;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (m < p.M) {
      raw = *reinterpret_cast<const uint4*>(p.x + static_cast<long long>(m) * p.ldx + k);
      if (p.norm_w) {
        const uint4 nw = *reinterpret_cast<const uint4*>(p.norm_w + k);
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
        const __nv_bfloat162* n2 = reinterpret_cast<const __nv_bfloat162*>(&nw);
        const float rs = s_rstd[m];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h2[e]), g = __bfloat1622float2(n2[e]);
          // same rounding points as the stand-alone RMSNorm kernel: bf16(x * rstd) * w
          const float a = __bfloat162float(__float2bfloat16(f.x * rs)) * g.x;
          const float b = __bfloat162float(__float2bfloat16(f.y * rs)) * g.y;
          h2[e] = __floats2bfloat162_rn(a, b);
        }
      }
    }
    *reinterpret_cast<uint4*>(sx + static_cast<long long>(m) * K + k) = raw;
  }
  __syncthreads();

  // ---- each warp walks groups of C output columns
  for (int g = blockIdx.x * kGvWarps + warp; g < n_groups; g += gridDim.x * kGvWarps) {
    float acc[MR][C], acc2[MR][C];
#pragma unroll
    for (int m = 0; m < MR; ++m)
#pragma unroll
      for (int c = 0; c < C; ++c) { acc[m][c] = 0.f; acc2[m][c] = 0.f; }
    const int n0 = g * C;
    for (int k0 = lane * 8; k0 < K; k0 += 256 * KU) {
      // issue every load of this chunk before any arithmetic: the kernel lives on bytes in flight
      uint4 wv[KU][C], wv2[SWIGLU ? KU : 1][SWIGLU ? C : 1];
#pragma unroll
      for (int u = 0; u < KU; ++u) {
        const int k = k0 + u * 256;
#pragma unroll
        for (int c = 0; c < C; ++c) {
          const int n = min(n0 + c, p.N - 1);
          if (k < K) {
            wv[u][c] = __ldg(reinterpret_cast<const uint4*>(p.w + static_cast<long long>(n) * p.ldw + k));
            if (SWIGLU) wv2[u][c] = __ldg(reinterpret_cast<const uint4*>(p.w + static_cast<long long>(n + p.N) * p.ldw + k));
          }
        }
      }
#pragma unroll
      for (int u = 0; u < KU; ++u) {
        const int k = k0 + u * 256;
        if (k >= K) break;
#pragma unroll
        for (int m = 0; m < MR; ++m) {
          const uint4 xv = *reinterpret_cast<const uint4*>(sx + m * K + k);
          const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
          float xf[8];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(x2[e]);
            xf[2 * e] = f.x;
            xf[2 * e + 1] = f.y;
          }
#pragma unroll
          for (int c = 0; c < C; ++c) {
            const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv[u][c]);
            float s = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = __bfloat1622float2(w2[e]);
              s = fmaf(xf[2 * e], f.x, s);
              s = fmaf(xf[2 * e + 1], f.y, s);
            }
            acc[m][c] += s;
            if (SWIGLU) {
              const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&wv2[u][c]);
              float s2 = 0.f;
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(u2[e]);
                s2 = fmaf(xf[2 * e], f.x, s2);
                s2 = fmaf(xf[2 * e + 1], f.y, s2);
              }
              acc2[m][c] += s2;
            }
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < MR; ++m)
#pragma unroll
      for (int c = 0; c < C; ++c) {
        float v = acc[m][c], v2 = acc2[m][c];
        for (int o = 16; o > 0; o >>= 1) {
          v += __shfl_xor_sync(0xffffffffu, v, o);
          if (SWIGLU) v2 += __shfl_xor_sync(0xffffffffu, v2, o);
        }
        acc[m][c] = v;
        acc2[m][c] = v2;
      }
    // lanes 0 .. M*C-1 each finish one output element
    const int e = lane;
    if (e < p.M * C) {
      const int m = e / C, c = e - m * C, n = n0 + c;
      if (n < p.N) {
        // pick this lane's values without dynamic register indexing
        float v = 0.f, v2 = 0.f;
#pragma unroll
        for (int mm = 0; mm < MR; ++mm)
#pragma unroll
          for (int cc = 0; cc < C; ++cc)
            if (mm == m && cc == c) { v = acc[mm][cc]; v2 = acc2[mm][cc]; }
        if (p.t) {
          auto lora = [&](int row) {
            int seg = 0;
#pragma unroll
            for (int i = 0; i < 3; ++i) seg += (row >= p.seg_end[i]) ? 1 : 0;
            const __nv_bfloat16* tr = p.t + static_cast<long long>(m) * p.ldt + seg * p.r;
            const float* br = p.lora_b + static_cast<long long>(row) * p.r;
            float s = 0.f;
            for (int j = 0; j < p.r; ++j) s = fmaf(__bfloat162float(tr[j]), br[j], s);
            return s;
          };
          v += lora(n);
          if (SWIGLU) v2 += lora(n + p.N);
        }
        v *= p.alpha;
        if (SWIGLU) v = gv_silu(v) * (v2 * p.alpha);
        if (p.residual) v += __bfloat162float(p.residual[static_cast<long long>(m) * p.ldr + n]);
        p.y[static_cast<long long>(m) * p.ldy + n] = __float2bfloat16(v);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Tensor-core variant for up to 16 rows (no LoRA term): the rows of x are the 16-row A operand of mma.m16n8k16, eight
// weight rows are the B operand, so the arithmetic per weight byte drops from ~4 CUDA-core instructions per row to a
// fraction of one and the kernel is bound by the weight stream for every M <= 16.
//
// A CTA owns 8 output columns at a time; its 8 warps split K (warp w takes the 32-wide k chunks w, w + 8, ...), all
// weight loads of a warp are issued before the activations are even staged, and the partial accumulators are summed
// through shared memory. Each lane's 16-byte weight load (8 consecutive k of column lane / 4) feeds two MMAs: the MMA
// only needs A and B to agree on which k sits in which fragment slot, so the slots are assigned to match the load
// (lane group g = lane % 4 owns k = 8 g .. 8 g + 7 of the chunk; MMA j uses k = 8 g + 4 j + {0, 1} and {2, 3}), and
// the A fragments are read from the staged x with the same assignment: one 16-byte shared load per row half.
constexpr int kTcThreads = 256;
constexpr int kTcWarps = 8;
constexpr int kTcKU = 8;            // 16-byte weight loads in flight per lane (per gate/up half)
constexpr int kTcPad = 32;          // row padding of the staged activations (bank spread for the fragment loads)

__device__ __forceinline__ void mma_16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// LoRA term of one output element: t[m, seg * r ..] . lora_b[row, :], seg from the stacked-projection boundaries.
__device__ __forceinline__ float gv_lora(const GemvParams& p, int m, int row) {
  int seg = 0;
#pragma unroll
  for (int i = 0; i < 3; ++i) seg += (row >= p.seg_end[i]) ? 1 : 0;
  const __nv_bfloat16* tr = p.t + static_cast<long long>(m) * p.ldt + seg * p.r;
  const float* br = p.lora_b + static_cast<long long>(row) * p.r;
  float s = 0.f;
  for (int j = 0; j < p.r; ++j) s = fmaf(__bfloat162float(tr[j]), br[j], s);
  return s;
}

// Stage x (optionally RMS-normalised) as [rows][lds] bf16 (rows = 8 when M <= 8, else 16); rows >= M are zero. Shared by
// the tensor-core kernels; with M <= 8 the upper half of the MMA's A operand is passed as zero registers instead.
__device__ __forceinline__ void gv_stage16(const GemvParams& p, __nv_bfloat16* sx, int lds, float* s_rstd) {
  const int rows = p.M > 8 ? 16 : 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, K = p.K;
  if (p.norm_w) {
    for (int m = warp; m < p.M; m += kTcWarps) {
      float ss = 0.f;
      for (int k = lane * 8; k < K; k += 256) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p.x + static_cast<long long>(m) * p.ldx + k);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h2[e]);
          ss += f.x * f.x + f.y * f.y;
        }
      }
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) s_rstd[m] = rsqrtf(ss / static_cast<float>(K) + p.eps);
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < rows * (K / 8); i += kTcThreads) {
    const int m = i / (K / 8), k = (i - m * (K / 8)) * 8;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (m < p.M) {
      raw = *reinterpret_cast<const uint4*>(p.x + static_cast<long long>(m) * p.ldx + k);
      if (p.norm_w) {
        const uint4 nw = *reinterpret_cast<const uint4*>(p.norm_w + k);
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
        const __nv_bfloat162* n2 = reinterpret_cast<const __nv_bfloat162*>(&nw);
        const float rs = s_rstd[m];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h2[e]), gg = __bfloat1622float2(n2[e]);
          const float a = __bfloat162float(__float2bfloat16(f.x * rs)) * gg.x;
          const float b = __bfloat162float(__float2bfloat16(f.y * rs)) * gg.y;
          h2[e] = __floats2bfloat162_rn(a, b);
        }
      }
    }
    *reinterpret_cast<uint4*>(sx + static_cast<long long>(m) * lds + k) = raw;
  }
  __syncthreads();
}

// Sum the 8 warps' partial accumulators of one 8-column tile and finish the outputs (scale, LoRA, SwiGLU, residual).
template <bool SWIGLU>
__device__ __forceinline__ void gv_tile_epilogue(const GemvParams& p, const float* red, int tile) {
  if (threadIdx.x < 128) {
    const int e = threadIdx.x;
    float v = 0.f, v2 = 0.f;
#pragma unroll
    for (int w = 0; w < kTcWarps; ++w) {
      v += red[(w * 2) * 128 + e];
      if (SWIGLU) v2 += red[(w * 2 + 1) * 128 + e];
    }
    const int src = e >> 2, reg = e & 3;
    const int m = (src >> 2) + ((reg & 2) ? 8 : 0), n = tile * 8 + (src & 3) * 2 + (reg & 1);
    if (m < p.M && n < p.N) {
      if (p.t) {
        v += gv_lora(p, m, n);
        if (SWIGLU) v2 += gv_lora(p, m, n + p.N);
      }
      v *= p.alpha;
      if (SWIGLU) v = gv_silu(v) * (v2 * p.alpha);
      if (p.residual) v += __bfloat162float(p.residual[static_cast<long long>(m) * p.ldr + n]);
      p.y[static_cast<long long>(m) * p.ldy + n] = __float2bfloat16(v);
    }
  }
}

template <bool SWIGLU>
__global__ void __launch_bounds__(kTcThreads) gemv_tc_kernel(const GemvParams p) {
  extern __shared__ __align__(16) uint8_t gv_smem[];
  const int K = p.K, lds = K + kTcPad;
  __nv_bfloat16* sx = reinterpret_cast<__nv_bfloat16*>(gv_smem);                      // [16][lds]
  float* red = reinterpret_cast<float*>(gv_smem + static_cast<size_t>(16) * lds * 2);   // [warps][2][128]
  __shared__ float s_rstd[16];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane & 3, col = lane >> 2;
  const int n_tiles = (p.N + 7) / 8;
  const int rounds = (K + 255) / 256;            // 32-wide k chunks per warp

  auto load_batch = [&](int tile, int r0, uint4 wv[kTcKU], uint4 wv2[SWIGLU ? kTcKU : 1]) {
    const int n = min(tile * 8 + col, p.N - 1);
    const __nv_bfloat16* wr = p.w + static_cast<long long>(n) * p.ldw;
#pragma unroll
    for (int u = 0; u < kTcKU; ++u) {
      const int k = ((r0 + u) * kTcWarps + warp) * 32 + g * 8;
      if (r0 + u < rounds && k < K) {
        wv[u] = __ldg(reinterpret_cast<const uint4*>(wr + k));
        if (SWIGLU) wv2[u] = __ldg(reinterpret_cast<const uint4*>(wr + static_cast<long long>(p.N) * p.ldw + k));
      } else {
        wv[u] = make_uint4(0u, 0u, 0u, 0u);
        if (SWIGLU) wv2[u] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };

  // the first tile's weights are requested before anything that depends on the previous kernel's output
  uint4 wv[kTcKU], wv2[SWIGLU ? kTcKU : 1];
  int tile = blockIdx.x;
  if (tile < n_tiles) load_batch(tile, 0, wv, wv2);

  gv_stage16(p, sx, lds, s_rstd);

  for (; tile < n_tiles; tile += gridDim.x) {
    float c[4] = {0.f, 0.f, 0.f, 0.f}, c2[4] = {0.f, 0.f, 0.f, 0.f};
    for (int r0 = 0; r0 < rounds; r0 += kTcKU) {
      if (r0 > 0) load_batch(tile, r0, wv, wv2);
#pragma unroll
      for (int u = 0; u < kTcKU; ++u) {
        const int k = ((r0 + u) * kTcWarps + warp) * 32 + g * 8;
        if (r0 + u >= rounds || k >= K) break;
        const uint4 xa = *reinterpret_cast<const uint4*>(sx + col * lds + k);
        const uint4 xb = p.M > 8 ? *reinterpret_cast<const uint4*>(sx + (col + 8) * lds + k) : make_uint4(0u, 0u, 0u, 0u);
        mma_16816(c, xa.x, xb.x, xa.y, xb.y, wv[u].x, wv[u].y);
        mma_16816(c, xa.z, xb.z, xa.w, xb.w, wv[u].z, wv[u].w);
        if (SWIGLU) {
          mma_16816(c2, xa.x, xb.x, xa.y, xb.y, wv2[u].x, wv2[u].y);
          mma_16816(c2, xa.z, xb.z, xa.w, xb.w, wv2[u].z, wv2[u].w);
        }
      }
    }
    // the next tile's first batch goes out before the reduction of this one
    const int next = tile + gridDim.x;
    if (next < n_tiles) load_batch(next, 0, wv, wv2);
    float* my = red + (warp * 2) * 128;
    *reinterpret_cast<float4*>(my + lane * 4) = make_float4(c[0], c[1], c[2], c[3]);
    if (SWIGLU) *reinterpret_cast<float4*>(my + 128 + lane * 4) = make_float4(c2[0], c2[1], c2[2], c2[3]);
    __syncthreads();
    gv_tile_epilogue<SWIGLU>(p, red, tile);
    __syncthreads();
  }
}

// 4-bit weights: the same tiling, but a lane's 16-byte load holds 32 consecutive codes of one column (lane group g owns
// k = 32 g .. 32 g + 31 of a 128-wide chunk); they are expanded to bf16 in registers (table lookup times the block's
// absmax) eight at a time, each eight feeding two MMAs. The weight stream is a quarter of the bf16 one.
__constant__ float kGvNf4[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                                 -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                                 0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
                                 0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};
__constant__ float kGvFp4[16] = {0.0f, 0.0052083333f, 0.6666667f, 1.0f, 0.3333333f, 0.5f, 0.1666667f, 0.25f,
                                 -0.0f, -0.0052083333f, -0.6666667f, -1.0f, -0.3333333f, -0.5f, -0.1666667f, -0.25f};
constexpr int kQ4KU = 4;            // 16-byte code loads in flight per lane (per gate/up half)

__device__ __forceinline__ uint32_t gv_pack2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <bool SWIGLU>
__global__ void __launch_bounds__(kTcThreads) gemv_q4_tc_kernel(const GemvParams p) {
  extern __shared__ __align__(16) uint8_t gv_smem[];
  const int K = p.K, lds = K + kTcPad;
  __nv_bfloat16* sx = reinterpret_cast<__nv_bfloat16*>(gv_smem);
  float* red = reinterpret_cast<float*>(gv_smem + static_cast<size_t>(16) * lds * 2);
  __shared__ float s_rstd[16];
  __shared__ float lut[16];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane & 3, col = lane >> 2;
  const int n_tiles = (p.N + 7) / 8;
  const int rounds = (K + 1023) / 1024;          // 128-wide k chunks per warp
  if (threadIdx.x < 16) lut[threadIdx.x] = p.fp4 ? kGvFp4[threadIdx.x] : kGvNf4[threadIdx.x];

  auto load_batch = [&](int tile, int r0, uint4 q[kQ4KU], float am[kQ4KU], uint4 q2[SWIGLU ? kQ4KU : 1],
                        float am2[SWIGLU ? kQ4KU : 1]) {
    const long long n = min(tile * 8 + col, p.N - 1);
#pragma unroll
    for (int u = 0; u < kQ4KU; ++u) {
      const int k = ((r0 + u) * kTcWarps + warp) * 128 + g * 32;
      const bool ok = r0 + u < rounds && k < K;
      const long long e0 = n * K + k, e1 = (n + p.N) * K + k;
      q[u] = ok ? __ldg(reinterpret_cast<const uint4*>(p.qdata + e0 / 2)) : make_uint4(0x77777777u, 0x77777777u, 0x77777777u, 0x77777777u);
      am[u] = !ok ? 0.f : (p.absmax ? __ldg(p.absmax + e0 / p.qblock)
                                    : static_cast<float>(__ldg(p.absmax_q + e0 / p.qblock)) * p.am_scale + p.am_offset);
      if (SWIGLU) {
        q2[u] = ok ? __ldg(reinterpret_cast<const uint4*>(p.qdata + e1 / 2)) : make_uint4(0x77777777u, 0x77777777u, 0x77777777u, 0x77777777u);
        am2[u] = !ok ? 0.f : (p.absmax ? __ldg(p.absmax + e1 / p.qblock)
                                       : static_cast<float>(__ldg(p.absmax_q + e1 / p.qblock)) * p.am_scale + p.am_offset);
      }
    }
  };
  uint4 q[kQ4KU], q2[SWIGLU ? kQ4KU : 1];
  float am[kQ4KU], am2[SWIGLU ? kQ4KU : 1];
  int tile = blockIdx.x;
  if (tile < n_tiles) load_batch(tile, 0, q, am, q2, am2);
  gv_stage16(p, sx, lds, s_rstd);

  // expand one 32-bit word (8 codes, first element in the high nibble of the first byte) and run its two MMAs
  auto word_mma = [&](float c[4], uint32_t w, float scale, const uint4& xa, const uint4& xb) {
    float e[8];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const uint32_t byte = (w >> (8 * b)) & 0xffu;
      e[2 * b] = lut[byte >> 4] * scale;
      e[2 * b + 1] = lut[byte & 0xfu] * scale;
    }
    mma_16816(c, xa.x, xb.x, xa.y, xb.y, gv_pack2(e[0], e[1]), gv_pack2(e[2], e[3]));
    mma_16816(c, xa.z, xb.z, xa.w, xb.w, gv_pack2(e[4], e[5]), gv_pack2(e[6], e[7]));
  };

  for (; tile < n_tiles; tile += gridDim.x) {
    float c[4] = {0.f, 0.f, 0.f, 0.f}, c2[4] = {0.f, 0.f, 0.f, 0.f};
    for (int r0 = 0; r0 < rounds; r0 += kQ4KU) {
      if (r0 > 0) load_batch(tile, r0, q, am, q2, am2);
#pragma unroll
      for (int u = 0; u < kQ4KU; ++u) {
        if (r0 + u >= rounds) break;
        const int k = ((r0 + u) * kTcWarps + warp) * 128 + g * 32;
        const uint32_t words[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
        const uint32_t words2[4] = {SWIGLU ? q2[u].x : 0u, SWIGLU ? q2[u].y : 0u, SWIGLU ? q2[u].z : 0u, SWIGLU ? q2[u].w : 0u};
#pragma unroll
        for (int sidx = 0; sidx < 4; ++sidx) {
          const int kk = k + sidx * 8;
          const bool in = kk < K;
          const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
          const uint4 xa = in ? *reinterpret_cast<const uint4*>(sx + col * lds + kk) : zero;
          const uint4 xb = (in && p.M > 8) ? *reinterpret_cast<const uint4*>(sx + (col + 8) * lds + kk) : zero;
          word_mma(c, words[sidx], am[u], xa, xb);
          if (SWIGLU) word_mma(c2, words2[sidx], am2[u], xa, xb);
        }
      }
    }
    const int next = tile + gridDim.x;
    if (next < n_tiles) load_batch(next, 0, q, am, q2, am2);
    float* my = red + (warp * 2) * 128;
    *reinterpret_cast<float4*>(my + lane * 4) = make_float4(c[0], c[1], c[2], c[3]);
    if (SWIGLU) *reinterpret_cast<float4*>(my + 128 + lane * 4) = make_float4(c2[0], c2[1], c2[2], c2[3]);
    __syncthreads();
    gv_tile_epilogue<SWIGLU>(p, red, tile);
    __syncthreads();
  }
}

template <bool SWIGLU>
static int launch_gemv_q4(const GemvParams& p, cudaStream_t st) {
  const size_t smem = static_cast<size_t>(16) * (p.K + kTcPad) * 2 + kTcWarps * 2 * 128 * sizeof(float);
  static DeviceMax configured;
  if (smem > 40 * 1024 && smem > configured.get()) {
    cudaError_t e = cudaFuncSetAttribute(gemv_q4_tc_kernel<SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured.set(200 * 1024);
  }
  const int n_tiles = (p.N + 7) / 8;
  const int grid = n_tiles < num_sms() * 2 ? n_tiles : num_sms() * 2;
  return static_cast<int>(launch_pdl(gemv_q4_tc_kernel<SWIGLU>, dim3(grid), dim3(kTcThreads), smem, st, p));
}

template <bool SWIGLU>
static int launch_gemv_tc(const GemvParams& p, cudaStream_t st) {
  const size_t smem = static_cast<size_t>(16) * (p.K + kTcPad) * 2 + kTcWarps * 2 * 128 * sizeof(float);
  static DeviceMax configured;
  if (smem > 40 * 1024 && smem > configured.get()) {
    cudaError_t e = cudaFuncSetAttribute(gemv_tc_kernel<SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured.set(200 * 1024);
  }
  const int n_tiles = (p.N + 7) / 8;
  const int grid = n_tiles < num_sms() * 2 ? n_tiles : num_sms() * 2;      // each CTA stages x once and loops over its tiles
  return static_cast<int>(launch_pdl(gemv_tc_kernel<SWIGLU>, dim3(grid), dim3(kTcThreads), smem, st, p));
}

template <int MR, int C, int KU, bool SWIGLU>
static int launch_gemv(const GemvParams& p, cudaStream_t st) {
  const size_t smem = static_cast<size_t>(MR) * p.K * 2;
  static DeviceMax configured;
  if (smem > 40 * 1024 && smem > configured.get()) {   // static shared memory counts against the 48 KB default too
    cudaError_t e = cudaFuncSetAttribute(gemv_kernel<MR, C, KU, SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         200 * 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured.set(200 * 1024);
  }
  const int groups = (p.N + C - 1) / C;
  int grid = (groups + kGvWarps - 1) / kGvWarps;
  const int cap = num_sms() * 4;
  if (grid > cap) grid = cap;
  return static_cast<int>(launch_pdl(gemv_kernel<MR, C, KU, SWIGLU>, dim3(grid), dim3(kGvThreads), smem, st, p));
}

}  // namespace pm

using namespace pm;

// Returns 0, a negative argument error, or a CUDA error code. K % 8 == 0, row strides % 8 == 0, M <= 16,
// M * cols-per-warp <= 32.
extern "C" int pm_gemv(const void* x, int ldx, const void* w, int ldw, const void* norm_w, float eps, const void* residual,
                       int ldr, void* y, int ldy, int M, int N, int K, int swiglu, float alpha, const void* t, int ldt,
                       const float* lora_b, int r, const int* seg_end, cudaStream_t st) {
  if (M < 1 || M > 16 || N < 1 || K < 8 || (K % 8) || (ldx % 8) || (ldw % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return -2;
  if (norm_w && (reinterpret_cast<uintptr_t>(norm_w) & 15)) return -2;
  if (static_cast<size_t>(M <= 4 ? 4 : (M <= 8 ? 8 : 16)) * K * 2 > 200 * 1024) return -3;
  GemvParams p{};
  p.x = static_cast<const __nv_bfloat16*>(x); p.ldx = ldx;
  p.w = static_cast<const __nv_bfloat16*>(w); p.ldw = ldw;
  p.norm_w = static_cast<const __nv_bfloat16*>(norm_w); p.eps = eps;
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.y = static_cast<__nv_bfloat16*>(y); p.ldy = ldy;
  p.M = M; p.N = N; p.K = K; p.swiglu = swiglu; p.alpha = alpha;
  p.t = static_cast<const __nv_bfloat16*>(t); p.ldt = ldt; p.lora_b = lora_b; p.r = r;
  for (int i = 0; i < 4; ++i) p.seg_end[i] = seg_end ? seg_end[i] : 0x7fffffff;
  static int prefetch = -1;
  if (prefetch < 0) {
    const char* e = getenv("PMETAL_GEMV_PREFETCH");
    prefetch = e ? atoi(e) : 2;
  }
  p.prefetch_iters = prefetch;
  static int use_tc = -1;
  if (use_tc < 0) {
    const char* e = getenv("PMETAL_GEMV_TC");
    use_tc = e ? atoi(e) : 1;
  }
  if (use_tc && (K % 32) == 0 && static_cast<size_t>(16) * (K + kTcPad) * 2 + 8192 <= 200 * 1024)
    return swiglu ? launch_gemv_tc<true>(p, st) : launch_gemv_tc<false>(p, st);
  // wide outputs: several columns per warp; narrow outputs: one column per warp (so that every SM gets work) with a
  // deeper load pipeline instead
  const bool wide = N >= num_sms() * kGvWarps * 2;
  if (swiglu) {
    if (M <= 4) return launch_gemv<4, 2, 4, true>(p, st);
    if (M <= 8) return launch_gemv<8, 1, 4, true>(p, st);
    return launch_gemv<16, 1, 2, true>(p, st);
  }
  if (M <= 4) return wide ? launch_gemv<4, 4, 4, false>(p, st) : launch_gemv<4, 1, 8, false>(p, st);
  if (M <= 8) return wide ? launch_gemv<8, 2, 4, false>(p, st) : launch_gemv<8, 1, 8, false>(p, st);
  return wide ? launch_gemv<16, 2, 2, false>(p, st) : launch_gemv<16, 1, 4, false>(p, st);
}

// 4-bit weights: qdata holds N_w * K / 2 bytes (two codes per byte, first element in the high nibble), absmax one fp32
// per qblock elements or absmax_q one byte per block with scale / offset (double quantisation). K % 32 == 0,
// qblock % 32 == 0. Other arguments as pm_gemv.
extern "C" int pm_gemv_q4(const void* x, int ldx, const void* qdata, const float* absmax, const void* absmax_q,
                          float am_scale, float am_offset, int qblock, int fp4, const void* norm_w, float eps,
                          const void* residual, int ldr, void* y, int ldy, int M, int N, int K, int swiglu, float alpha,
                          const void* t, int ldt, const float* lora_b, int r, const int* seg_end, cudaStream_t st) {
  if (M < 1 || M > 16 || N < 1 || K < 32 || (K % 32) || (ldx % 8) || qblock < 32 || (qblock % 32)) return -1;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(qdata)) & 15) return -2;
  if (!absmax && !absmax_q) return -2;
  if (static_cast<size_t>(16) * (K + kTcPad) * 2 + 8192 > 200 * 1024) return -3;
  GemvParams p{};
  p.x = static_cast<const __nv_bfloat16*>(x); p.ldx = ldx;
  p.qdata = static_cast<const uint8_t*>(qdata); p.absmax = absmax; p.absmax_q = static_cast<const uint8_t*>(absmax_q);
  p.am_scale = am_scale; p.am_offset = am_offset; p.qblock = qblock; p.fp4 = fp4;
  p.norm_w = static_cast<const __nv_bfloat16*>(norm_w); p.eps = eps;
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.y = static_cast<__nv_bfloat16*>(y); p.ldy = ldy;
  p.M = M; p.N = N; p.K = K; p.swiglu = swiglu; p.alpha = alpha;
  p.t = static_cast<const __nv_bfloat16*>(t); p.ldt = ldt; p.lora_b = lora_b; p.r = r;
  for (int i = 0; i < 4; ++i) p.seg_end[i] = seg_end ? seg_end[i] : 0x7fffffff;
  return swiglu ? launch_gemv_q4<true>(p, st) : launch_gemv_q4<false>(p, st);
}
