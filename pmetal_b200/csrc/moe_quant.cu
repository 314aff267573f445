// MoE routing kernels, GGUF block dequantisation to bf16, and block-scaled FP8 (E4M3) weight quantisation.
//
// MoE (reference: crates/pmetal-metal/src/kernels/metal/moe_routing.metal — moe_topk_selection,
// moe_compute_indices, moe_compute_expert_offsets, moe_sort_indices; crates/pmetal-models/src/moe_routing.rs:52-108):
//   moe_router_kernel   softmax over experts, top-k by repeated warp argmax, optional renormalisation of the k weights
//   moe_count_kernel    tokens per expert
//   moe_scan_kernel     exclusive prefix sum of the counts (one block)
//   moe_sort_kernel     stable counting sort of the (token, slot) pairs by expert: perm[pos] = token*k + slot,
//                       inv[token*k + slot] = pos. One block per expert walks the pairs in order, so the result is
//                       deterministic (no atomics on positions).
// GGUF dequantisation (reference: crates/pmetal-metal/src/kernels/metal/dequant.metal — dequantize_q4_0; layouts of
// crates/pmetal-gguf/src/dequant.rs:92-730): Q4_0, Q8_0, Q4_K, Q6_K blocks -> bf16 rows feeding the GEMM.
// FP8 (reference: crates/pmetal-metal/src/kernels/metal/fp8_training.metal:212-407 — fp8_act_quant_block,
// fp8_weight_dequant_block; block size 128): per-128-element scale = amax / 448, values stored as E4M3.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include "host_util.cuh"
#include "pmetal_b200.h"

namespace pm {

// ------------------------------------------------------------------------------------------------ MoE routing
// One warp per token. E <= 1024 experts (NV = ceil(E / 32) per lane, kept in registers), k <= 16.
template <int NV>
__device__ __forceinline__ void moe_route_token_nv(const __nv_bfloat16* __restrict__ logits_bf16,
                                                   const float* __restrict__ logits_f32, int t, int E, int k, int renorm,
                                                   int* __restrict__ topk_idx, float* __restrict__ topk_w, int lane) {
  float v[NV];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int e = i * 32 + lane;
    float x = -INFINITY;
    if (e < E) x = logits_f32 ? logits_f32[static_cast<long long>(t) * E + e]
                              : __bfloat162float(logits_bf16[static_cast<long long>(t) * E + e]);
    v[i] = x;
    mx = fmaxf(mx, x);
  }
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float z = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    v[i] = (i * 32 + lane < E) ? __expf(v[i] - mx) : -1.f;
    if (v[i] > 0.f) z += v[i];
  }
  for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
  const float inv_z = 1.f / z;
  float wsum = 0.f, my_w = 0.f;
  int my_idx = 0;
  for (int j = 0; j < k; ++j) {
    float bv = -1.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int e = i * 32 + lane;
      if (v[i] > bv) { bv = v[i]; bi = e; }     // ascending e within a lane: first maximum wins
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((bi & 31) == lane) {
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (i == (bi >> 5)) v[i] = -1.f;
    }
    const float w = bv * inv_z;
    wsum += w;
    if (lane == j) { my_w = w; my_idx = bi; }
  }
  if (lane < k) {
    topk_idx[static_cast<long long>(t) * k + lane] = my_idx;
    topk_w[static_cast<long long>(t) * k + lane] = renorm ? my_w / wsum : my_w;
  }
}

__device__ __forceinline__ void moe_route_token(const __nv_bfloat16* __restrict__ logits_bf16,
                                                const float* __restrict__ logits_f32, int t, int E, int k, int renorm,
                                                int* __restrict__ topk_idx, float* __restrict__ topk_w, int lane) {
  if (E <= 64) moe_route_token_nv<2>(logits_bf16, logits_f32, t, E, k, renorm, topk_idx, topk_w, lane);
  else if (E <= 128) moe_route_token_nv<4>(logits_bf16, logits_f32, t, E, k, renorm, topk_idx, topk_w, lane);
  else if (E <= 256) moe_route_token_nv<8>(logits_bf16, logits_f32, t, E, k, renorm, topk_idx, topk_w, lane);
  else moe_route_token_nv<32>(logits_bf16, logits_f32, t, E, k, renorm, topk_idx, topk_w, lane);
}

__global__ void moe_router_kernel(const __nv_bfloat16* __restrict__ logits_bf16, const float* __restrict__ logits_f32,
                                  int T, int E, int k, int renorm, int* __restrict__ topk_idx,
                                  float* __restrict__ topk_w) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  moe_route_token(logits_bf16, logits_f32, t, E, k, renorm, topk_idx, topk_w, threadIdx.x & 31);
}

// Few tokens (T * k <= 1024): routing, counting, offsets and the stable sort in one CTA, so that a decode step pays one
// launch instead of four. Thread e owns expert e and walks the (token, slot) list in order, which keeps the sort stable
// and deterministic. offsets2 (optional) receives a second copy of the offsets (the expert-parallel exchange buffer).
constexpr int kRouteSmallMax = 1024;
__global__ void __launch_bounds__(1024) moe_route_small_kernel(const __nv_bfloat16* __restrict__ logits_bf16,
                                                               const float* __restrict__ logits_f32, int T, int E, int k,
                                                               int renorm, int* __restrict__ topk_idx,
                                                               float* __restrict__ topk_w, int* __restrict__ counts,
                                                               int* __restrict__ offsets, int* __restrict__ offsets2,
                                                               int* __restrict__ perm, int* __restrict__ inv) {
  __shared__ int s_idx[kRouteSmallMax];
  __shared__ int s_off[1024 + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n = T * k;
  for (int t = warp; t < T; t += 32) moe_route_token(logits_bf16, logits_f32, t, E, k, renorm, topk_idx, topk_w, lane);
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) s_idx[i] = topk_idx[i];
  __syncthreads();
  const int e = threadIdx.x;
  int c = 0;
  if (e < E)
    for (int i = 0; i < n; ++i) c += (s_idx[i] == e);
  if (e < E) s_off[e + 1] = c;
  if (e == 0) s_off[0] = 0;
  __syncthreads();
  if (threadIdx.x == 0)
    for (int j = 1; j <= E; ++j) s_off[j] += s_off[j - 1];
  __syncthreads();
  if (e <= E) {
    offsets[e] = s_off[e];
    if (offsets2) offsets2[e] = s_off[e];
  }
  if (e < E) {
    counts[e] = c;
    int pos = s_off[e];
    for (int i = 0; i < n; ++i)
      if (s_idx[i] == e) {
        perm[pos] = i;
        inv[i] = pos;
        ++pos;
      }
  }
}

// Replicated-token expert parallelism (every rank sees every token, each rank applies its own experts and the partial
// outputs are summed across ranks): routing for all E experts, then the padded expert-sorted layout of the assignments
// that fall on this rank's experts [e0, e0 + e_loc). One CTA; T * k <= 4096.
//   off[e_loc + 1]  row offsets of the local experts' slabs, each padded to a multiple of `align`
//   dest[T * k]     row of assignment i in the padded buffer, -1 when its expert lives on another rank
//   src[cap]        assignment index of every row of the padded buffer, -1 for padding (rows >= off[e_loc] untouched)
constexpr int kRouteLocalMax = 4096;
__global__ void __launch_bounds__(1024) moe_route_local_kernel(const __nv_bfloat16* __restrict__ logits_bf16,
                                                               const float* __restrict__ logits_f32, int T, int E, int k,
                                                               int renorm, int e0, int e_loc, int align,
                                                               int* __restrict__ topk_idx, float* __restrict__ topk_w,
                                                               int* __restrict__ off, int* __restrict__ dest,
                                                               int* __restrict__ src) {
  __shared__ int s_idx[kRouteLocalMax];
  __shared__ int s_off[1024 + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n = T * k;
  for (int t = warp; t < T; t += 32) moe_route_token(logits_bf16, logits_f32, t, E, k, renorm, topk_idx, topk_w, lane);
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int x = topk_idx[i];
    s_idx[i] = x;
    if (x < e0 || x >= e0 + e_loc) dest[i] = -1;
  }
  if (threadIdx.x == 0) s_off[0] = 0;
  __syncthreads();
  // one warp per local expert: count its assignments 32 at a time
  for (int e = warp; e < e_loc; e += 32) {
    int c = 0;
    for (int i0 = 0; i0 < n; i0 += 32) {
      const int i = i0 + lane;
      c += __popc(__ballot_sync(0xffffffffu, i < n && s_idx[i] == e0 + e));
    }
    if (lane == 0) s_off[e + 1] = (c + align - 1) / align * align;
  }
  __syncthreads();
  if (warp == 0) {            // inclusive scan of the padded counts, 32 experts per round
    int carry = 0;
    for (int j0 = 1; j0 <= e_loc; j0 += 32) {
      const int j = j0 + lane;
      int v = j <= e_loc ? s_off[j] : 0;
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
      }
      v += carry;
      if (j <= e_loc) s_off[j] = v;
      carry = __shfl_sync(0xffffffffu, v, 31);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= e_loc; e += blockDim.x) off[e] = s_off[e];
  // placement: rows of one expert keep the order of their assignment index
  for (int e = warp; e < e_loc; e += 32) {
    int pos = s_off[e];
    for (int i0 = 0; i0 < n; i0 += 32) {
      const int i = i0 + lane;
      const bool hit = i < n && s_idx[i] == e0 + e;
      const unsigned m = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const int r = pos + __popc(m & ((1u << lane) - 1u));
        dest[i] = r;
        src[r] = i;
      }
      pos += __popc(m);
    }
    for (int r = pos + lane; r < s_off[e + 1]; r += 32) src[r] = -1;
  }
}

// xs[row] = x[src[row] / k] for the rows of the local experts' slabs (zeros for padding rows)
__global__ void moe_gather_padded_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ src,
                                         const int* __restrict__ off_end, int k, __nv_bfloat16* __restrict__ xs, int H) {
  const int rows = *off_end;
  const int per = H / 8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < static_cast<long long>(rows) * per;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(i / per), c = static_cast<int>(i - static_cast<long long>(row) * per);
    const int a = src[row];
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (a >= 0) v = *reinterpret_cast<const uint4*>(x + static_cast<long long>(a / k) * H + c * 8);
    *reinterpret_cast<uint4*>(xs + static_cast<long long>(row) * H + c * 8) = v;
  }
}

// y[t] = (residual[t]) + sum over the token's local assignments of w[t, slot] * z[dest[t * k + slot]]
__global__ void moe_combine_local_kernel(const __nv_bfloat16* __restrict__ z, const int* __restrict__ dest,
                                         const float* __restrict__ w, int k, const __nv_bfloat16* __restrict__ residual,
                                         __nv_bfloat16* __restrict__ y, long long T, int H) {
  const int per = H / 8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < T * per;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / per;
    const int c = static_cast<int>(i - t * per) * 8;
    float acc[8];
    if (residual) {
      const uint4 rv = *reinterpret_cast<const uint4*>(residual + t * H + c);
      const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[2 * e] = __uint_as_float(rw[e] << 16);
        acc[2 * e + 1] = __uint_as_float(rw[e] & 0xffff0000u);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    }
    for (int s = 0; s < k; ++s) {
      const int d = dest[t * k + s];
      if (d < 0) continue;
      const float ws = w[t * k + s];
      const uint4 zv = *reinterpret_cast<const uint4*>(z + static_cast<long long>(d) * H + c);
      const uint32_t zw[4] = {zv.x, zv.y, zv.z, zv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[2 * e] += ws * __uint_as_float(zw[e] << 16);
        acc[2 * e + 1] += ws * __uint_as_float(zw[e] & 0xffff0000u);
      }
    }
    uint4 o;
    *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(acc[0], acc[1]);
    *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(acc[2], acc[3]);
    *reinterpret_cast<__nv_bfloat162*>(&o.z) = __floats2bfloat162_rn(acc[4], acc[5]);
    *reinterpret_cast<__nv_bfloat162*>(&o.w) = __floats2bfloat162_rn(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(y + t * H + c) = o;
  }
}

__global__ void moe_count_kernel(const int* __restrict__ topk_idx, long long n, int* __restrict__ counts) {
  const int e = blockIdx.x;
  int c = 0;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) c += (topk_idx[i] == e);
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  __shared__ int red[32];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int s = 0;
    for (int w = 0; w < (blockDim.x >> 5); ++w) s += red[w];
    counts[e] = s;
  }
}

__global__ void moe_scan_kernel(const int* __restrict__ counts, int E, int* __restrict__ offsets /*E+1*/) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) { offsets[e] = acc; acc += counts[e]; }
    offsets[E] = acc;
  }
}

__global__ void __launch_bounds__(256) moe_sort_kernel(const int* __restrict__ topk_idx, long long n,
                                                       const int* __restrict__ offsets, int* __restrict__ perm,
                                                       int* __restrict__ inv) {
  const int e = blockIdx.x;
  __shared__ int warp_cnt[8];
  __shared__ int base_s;
  if (threadIdx.x == 0) base_s = offsets[e];
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (long long c0 = 0; c0 < n; c0 += 256) {
    const long long i = c0 + threadIdx.x;
    const bool hit = i < n && topk_idx[i] == e;
    const unsigned bm = __ballot_sync(0xffffffffu, hit);
    if (lane == 0) warp_cnt[warp] = __popc(bm);
    __syncthreads();
    int before = 0, total = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      if (w < warp) before += warp_cnt[w];
      total += warp_cnt[w];
    }
    if (hit) {
      const int pos = base_s + before + __popc(bm & ((1u << lane) - 1u));
      perm[pos] = static_cast<int>(i);
      inv[i] = pos;
    }
    __syncthreads();
    if (threadIdx.x == 0) base_s += total;
    __syncthreads();
  }
}

// gather rows: out[pos] = x[perm[pos] / k]; and weighted scatter-combine: y[t] = sum_j w[t,j] * z[inv[t*k+j]]
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ perm, int k,
                                  __nv_bfloat16* __restrict__ out, long long n, int H) {
  const int per_row = H / 8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n * per_row;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long pos = i / per_row;
    const int c = static_cast<int>(i - pos * per_row);
    const int src = perm[pos] / k;
    reinterpret_cast<uint4*>(out + pos * H)[c] = reinterpret_cast<const uint4*>(x + static_cast<long long>(src) * H)[c];
  }
}
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ z, const int* __restrict__ inv,
                                   const float* __restrict__ w, int k, const __nv_bfloat16* __restrict__ residual,
                                   __nv_bfloat16* __restrict__ y, long long T, int H) {
  const int per_row = H / 8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < T * per_row;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / per_row;
    const int c = static_cast<int>(i - t * per_row);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      const float wj = w[t * k + j];
      const uint4 raw = reinterpret_cast<const uint4*>(z + static_cast<long long>(inv[t * k + j]) * H)[c];
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(h2[q]);
        acc[2 * q] += wj * f.x;
        acc[2 * q + 1] += wj * f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) o2[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
    if (residual) {      // y = bf16(sum) + residual, the rounding an unfused add would make
      const uint4 rr = reinterpret_cast<const uint4*>(residual + t * H)[c];
      const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rr);
#pragma unroll
      for (int q = 0; q < 4; ++q) o2[q] = __hadd2(o2[q], r2[q]);
    }
    reinterpret_cast<uint4*>(y + t * H)[c] = o;
  }
}

// ------------------------------------------------------------------------------------------------ GGUF dequant
__device__ __forceinline__ float h2f(const uint8_t* p) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(p[0] | (p[1] << 8))));
}
__device__ __forceinline__ void k4_scale_min(int j, const uint8_t* q, int* sc, int* mn) {
  if (j < 4) {
    *sc = q[j] & 63;
    *mn = q[j + 4] & 63;
  } else {
    *sc = (q[j + 4] & 15) | ((q[j - 4] >> 6) << 4);
    *mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

// type ids: 2 = Q4_0, 8 = Q8_0, 12 = Q4_K, 14 = Q6_K. One thread per 32 consecutive outputs.
__global__ void gguf_dequant_kernel(const uint8_t* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n,
                                    int type) {
  const long long groups = n / 32;
  for (long long g = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; g < groups;
       g += static_cast<long long>(gridDim.x) * blockDim.x) {
    float y[32];
    if (type == 2) {
      const uint8_t* b = src + g * 18;
      const float d = h2f(b);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        y[i] = d * static_cast<float>((b[2 + i] & 15) - 8);
        y[i + 16] = d * static_cast<float>((b[2 + i] >> 4) - 8);
      }
    } else if (type == 8) {
      const uint8_t* b = src + g * 34;
      const float d = h2f(b);
#pragma unroll
      for (int i = 0; i < 32; ++i) y[i] = d * static_cast<float>(static_cast<int8_t>(b[2 + i]));
    } else if (type == 12) {
      const uint8_t* b = src + (g >> 3) * 144;
      const int j = static_cast<int>(g & 7);          // sub-block of 32 within the 256 block
      const float d = h2f(b), dmin = h2f(b + 2);
      int sc, mn;
      k4_scale_min(j, b + 4, &sc, &mn);
      const uint8_t* qs = b + 16 + (j >> 1) * 32;
      const float ds = d * static_cast<float>(sc), dm = dmin * static_cast<float>(mn);
#pragma unroll
      for (int i = 0; i < 32; ++i) y[i] = ds * static_cast<float>((j & 1) ? (qs[i] >> 4) : (qs[i] & 15)) - dm;
    } else {
      const uint8_t* b = src + (g >> 3) * 210;
      const int j = static_cast<int>(g & 7);          // 0..7: half = j / 4, quarter = j % 4
      const int half = j >> 2, quarter = j & 3;
      const uint8_t* ql = b + 64 * half + ((quarter & 1) ? 32 : 0);
      const uint8_t* qh = b + 128 + 32 * half;
      const int8_t* scs = reinterpret_cast<const int8_t*>(b + 192) + 8 * half + 2 * quarter;
      const float d = h2f(b + 208);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int lo = (quarter >> 1) ? (ql[i] >> 4) : (ql[i] & 15);
        const int hi = (qh[i] >> (2 * quarter)) & 3;
        y[i] = d * static_cast<float>(scs[i >> 4]) * static_cast<float>((lo | (hi << 4)) - 32);
      }
    }
    uint4* o = reinterpret_cast<uint4*>(dst + g * 32);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint4 v;
      __nv_bfloat162* v2 = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int q = 0; q < 4; ++q) v2[q] = __floats2bfloat162_rn(y[c * 8 + 2 * q], y[c * 8 + 2 * q + 1]);
      o[c] = v;
    }
  }
}

// ------------------------------------------------------------------------------------------------ FP8 E4M3 blocks
// One warp per 128-element block: scale = amax / 448 (1 if the block is all zero), q = e4m3(x / scale).
__global__ void fp8_quant_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scales,
                                 long long n_blocks) {
  const long long b = blockIdx.x * static_cast<long long>(blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (b >= n_blocks) return;
  const uint2 raw = reinterpret_cast<const uint2*>(x + b * 128)[lane];
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 a = __bfloat1622float2(h2[0]), c = __bfloat1622float2(h2[1]);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(c.x), fabsf(c.y)));
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = amax > 0.f ? amax / 448.f : 1.f;
  const float inv = 1.f / scale;
  uint32_t packed = 0;
  const float vals[4] = {a.x * inv, a.y * inv, c.x * inv, c.y * inv};
#pragma unroll
  for (int i = 0; i < 4; ++i)
    packed |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(vals[i], __NV_SATFINITE, __NV_E4M3)) << (8 * i);
  reinterpret_cast<uint32_t*>(q + b * 128)[lane] = packed;
  if (lane == 0) scales[b] = scale;
}
__global__ void fp8_dequant_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scales,
                                   __nv_bfloat16* __restrict__ y, long long n_blocks) {
  const long long b = blockIdx.x * static_cast<long long>(blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (b >= n_blocks) return;
  const uint32_t packed = reinterpret_cast<const uint32_t*>(q + b * 128)[lane];
  const float s = scales[b];
  float v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half_raw hr = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>((packed >> (8 * i)) & 255), __NV_E4M3);
    v[i] = __half2float(__half(hr)) * s;
  }
  uint2 o;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
  o2[0] = __floats2bfloat162_rn(v[0], v[1]);
  o2[1] = __floats2bfloat162_rn(v[2], v[3]);
  reinterpret_cast<uint2*>(y + b * 128)[lane] = o;
}

static inline int grid_cap(long long work, int per_block, int cap = 0) {
  if (cap <= 0) cap = num_sms() * 16;
  long long g = (work + per_block - 1) / per_block;
  return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace pm

using namespace pm;

// offsets2: optional second destination for the [E + 1] offsets (may be null).
extern "C" int pm_moe_route2(const void* logits, int is_f32, int T, int E, int k, int renorm, int* topk_idx,
                             float* topk_w, int* counts, int* offsets, int* offsets2, int* perm, int* inv,
                             cudaStream_t st) {
  if (T <= 0 || E <= 0 || E > 1024 || k <= 0 || k > 16 || k > E) return -1;
  const long long n = static_cast<long long>(T) * k;
  if (n <= kRouteSmallMax && E < 1024) {
    moe_route_small_kernel<<<1, 1024, 0, st>>>(is_f32 ? nullptr : static_cast<const __nv_bfloat16*>(logits),
                                               is_f32 ? static_cast<const float*>(logits) : nullptr, T, E, k, renorm,
                                               topk_idx, topk_w, counts, offsets, offsets2, perm, inv);
    return static_cast<int>(cudaGetLastError());
  }
  moe_router_kernel<<<(T + 7) / 8, 256, 0, st>>>(is_f32 ? nullptr : static_cast<const __nv_bfloat16*>(logits),
                                                 is_f32 ? static_cast<const float*>(logits) : nullptr, T, E, k, renorm,
                                                 topk_idx, topk_w);
  moe_count_kernel<<<E, 256, 0, st>>>(topk_idx, n, counts);
  moe_scan_kernel<<<1, 32, 0, st>>>(counts, E, offsets);
  moe_sort_kernel<<<E, 256, 0, st>>>(topk_idx, n, offsets, perm, inv);
  if (offsets2) {
    cudaError_t e = cudaMemcpyAsync(offsets2, offsets, sizeof(int) * (E + 1), cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int pm_moe_route(const void* logits, int is_f32, int T, int E, int k, int renorm, int* topk_idx,
                            float* topk_w, int* counts, int* offsets, int* perm, int* inv, cudaStream_t st) {
  return pm_moe_route2(logits, is_f32, T, E, k, renorm, topk_idx, topk_w, counts, offsets, nullptr, perm, inv, st);
}

// Routing plus the padded layout of the assignments that belong to experts [e0, e0 + e_loc) (see the kernel).
extern "C" int pm_moe_route_local(const void* logits, int is_f32, int T, int E, int k, int renorm, int e0, int e_loc,
                                  int align, int* topk_idx, float* topk_w, int* off, int* dest, int* src,
                                  cudaStream_t st) {
  if (T <= 0 || E <= 0 || E > 1024 || k <= 0 || k > 16 || k > E || e_loc < 1 || e_loc > 1024 || e0 < 0 ||
      e0 + e_loc > E || align < 1)
    return -1;
  if (static_cast<long long>(T) * k > kRouteLocalMax) return -2;
  moe_route_local_kernel<<<1, 1024, 0, st>>>(is_f32 ? nullptr : static_cast<const __nv_bfloat16*>(logits),
                                             is_f32 ? static_cast<const float*>(logits) : nullptr, T, E, k, renorm, e0,
                                             e_loc, align, topk_idx, topk_w, off, dest, src);
  return static_cast<int>(cudaGetLastError());
}

// off_end points at the device int holding the number of rows in use (off[e_loc]); cap bounds the launch.
extern "C" int pm_moe_gather_padded(const void* x, const int* src, const int* off_end, int k, void* xs, int cap, int H,
                                    cudaStream_t st) {
  if (H % 8) return -1;
  if (cap <= 0) return 0;
  moe_gather_padded_kernel<<<grid_cap(static_cast<long long>(cap) * (H / 8), 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), src, off_end, k, static_cast<__nv_bfloat16*>(xs), H);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int pm_moe_combine_local(const void* z, const int* dest, const float* w, int k, const void* residual, void* y,
                                    long long T, int H, cudaStream_t st) {
  if (H % 8) return -1;
  if (T <= 0) return 0;
  moe_combine_local_kernel<<<grid_cap(T * (H / 8), 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(z), dest, w, k, static_cast<const __nv_bfloat16*>(residual),
      static_cast<__nv_bfloat16*>(y), T, H);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int pm_moe_gather(const void* x, const int* perm, int k, void* out, long long n, int H, cudaStream_t st) {
  if (H % 8) return -1;
  if (n <= 0) return 0;
  moe_gather_kernel<<<grid_cap(n * (H / 8), 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), perm, k,
                                                                static_cast<__nv_bfloat16*>(out), n, H);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int pm_moe_combine2(const void* z, const int* inv, const float* w, int k, const void* residual, void* y,
                               long long T, int H, cudaStream_t st) {
  if (H % 8) return -1;
  if (T <= 0) return 0;
  moe_combine_kernel<<<grid_cap(T * (H / 8), 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(z), inv, w, k,
                                                                 static_cast<const __nv_bfloat16*>(residual),
                                                                 static_cast<__nv_bfloat16*>(y), T, H);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int pm_moe_combine(const void* z, const int* inv, const float* w, int k, void* y, long long T, int H,
                              cudaStream_t st) {
  return pm_moe_combine2(z, inv, w, k, nullptr, y, T, H, st);
}

extern "C" int pm_gguf_dequant_bf16(const void* src, void* dst, long long n, int type, cudaStream_t st) {
  if (type != 2 && type != 8 && type != 12 && type != 14) return -1;
  if (n % ((type == 2 || type == 8) ? 32 : 256)) return -2;
  if (n <= 0) return 0;
  gguf_dequant_kernel<<<grid_cap(n / 32, 128), 128, 0, st>>>(static_cast<const uint8_t*>(src),
                                                             static_cast<__nv_bfloat16*>(dst), n, type);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int pm_fp8_quant(const void* x, void* q, float* scales, long long n, cudaStream_t st) {
  if (n % 128) return -1;
  if (n <= 0) return 0;
  const long long nb = n / 128;
  fp8_quant_kernel<<<static_cast<unsigned>((nb + 7) / 8), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
                                                                        static_cast<uint8_t*>(q), scales, nb);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int pm_fp8_dequant(const void* q, const float* scales, void* y, long long n, cudaStream_t st) {
  if (n % 128) return -1;
  if (n <= 0) return 0;
  const long long nb = n / 128;
  fp8_dequant_kernel<<<static_cast<unsigned>((nb + 7) / 8), 256, 0, st>>>(static_cast<const uint8_t*>(q), scales,
                                                                          static_cast<__nv_bfloat16*>(y), nb);
  return static_cast<int>(cudaGetLastError());
}
