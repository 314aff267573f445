// Bandwidth-bound fused kernels: RMSNorm (+residual add) fwd/bwd, per-head QK-RMSNorm + RoPE
// fwd/bwd, SwiGLU fwd/bwd, softmax-cross-entropy over a logits chunk (loss + gradient in place),
// sum of squares, and the flat multi-tensor AdamW update with global-norm clipping.
//
// They restate the reference's Metal kernels for sm_100a: fused_norm_lora.metal (RMSNorm),
// fused_rope.metal (rope_qk_with_positions), fused_swiglu.metal, fused_cross_entropy.metal and
// fused_training.metal (fused_adamw_update_bias_corrected, gradient_norm_squared_partial),
// all under crates/pmetal-metal/src/kernels/metal/.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "host_util.cuh"

#include "pdl.cuh"
#include "pmetal_b200.h"

namespace pm {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const bf16x8 t = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = __bfloat1622float2(t.v[i]);
    f[2 * i] = a.x;
    f[2 * i + 1] = a.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  bf16x8 t;
#pragma unroll
  for (int i = 0; i < 4; ++i) t.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<bf16x8*>(p) = t;
}

// ------------------------------------------------------------------------------------ RMSNorm
// One warp per row. h = x (+ res); y = h * rsqrt(mean(h^2) + eps) * w. H % 8 == 0.
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd, int T, int H,
                                   float eps) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= T) return;
  const __nv_bfloat16* xr = x + static_cast<size_t>(row) * H;
  const __nv_bfloat16* rr = res ? res + static_cast<size_t>(row) * H : nullptr;
  __nv_bfloat16* hr = h_out ? h_out + static_cast<size_t>(row) * H : nullptr;
  float ss = 0.f;
  for (int c = lane * 8; c < H; c += 256) {
    float f[8];
    load8(xr + c, f);
    if (rr) {
      float g[8];
      load8(rr + c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] += g[i];
      // the residual stream is kept in bf16: round before use so that y matches norm(h_out)
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(__float2bfloat16(f[i]));
      store8(hr + c, f);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  ss = warp_sum(ss);
  const float rs = rsqrtf(ss / H + eps);
  if (lane == 0) rstd[row] = rs;
  const __nv_bfloat16* src = rr ? hr : xr;
  __nv_bfloat16* yr = y + static_cast<size_t>(row) * H;
  for (int c = lane * 8; c < H; c += 256) {
    float f[8], g[8];
    load8(src + c, f);
    load8(w + c, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = f[i] * rs * g[i];
    store8(yr + c, f);
  }
}

// Few rows (decode, verification): one 256-thread CTA per row, so that 64 rows occupy 64 SMs instead of 8. Each thread
// keeps its (up to two) 8-element chunks in registers between the reduction and the scaling. H <= 4096, H % 8 == 0.
__global__ void __launch_bounds__(256) rmsnorm_fwd_row_kernel(const __nv_bfloat16* __restrict__ x,
                                                              const __nv_bfloat16* __restrict__ res,
                                                              const __nv_bfloat16* __restrict__ w,
                                                              __nv_bfloat16* __restrict__ y,
                                                              __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd,
                                                              int H, float eps) {
  __shared__ float red[8];
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t base = static_cast<size_t>(row) * H;
  float f[2][8];
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int c = (u * 256 + threadIdx.x) * 8;
    if (c < H) {
      load8(x + base + c, f[u]);
      if (res) {
        float g[8];
        load8(res + base + c, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[u][i] = __bfloat162float(__float2bfloat16(f[u][i] + g[i]));
        store8(h_out + base + c, f[u]);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[u][i] * f[u][i];
    }
  }
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float rs = rsqrtf(tot / H + eps);
  if (threadIdx.x == 0) rstd[row] = rs;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int c = (u * 256 + threadIdx.x) * 8;
    if (c < H) {
      float g[8];
      load8(w + c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[u][i] = f[u][i] * rs * g[i];
      store8(y + base + c, f[u]);
    }
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dh_add);  optional dw += sum_rows dy * xhat
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                                   const __nv_bfloat16* __restrict__ dh_add, __nv_bfloat16* __restrict__ dx,
                                   float* __restrict__ dw, int T, int H) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= T) return;
  const size_t off = static_cast<size_t>(row) * H;
  const float rs = rstd[row];
  float dot = 0.f;
  for (int c = lane * 8; c < H; c += 256) {
    float a[8], b[8], g[8];
    load8(dy + off + c, a);
    load8(h + off + c, b);
    load8(w + c, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) dot += a[i] * g[i] * b[i] * rs;
  }
  dot = warp_sum(dot) / H;
  for (int c = lane * 8; c < H; c += 256) {
    float a[8], b[8], g[8], o[8];
    load8(dy + off + c, a);
    load8(h + off + c, b);
    load8(w + c, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = rs * (a[i] * g[i] - b[i] * rs * dot);
    if (dh_add) {
      float e[8];
      load8(dh_add + off + c, e);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] += e[i];
    }
    store8(dx + off + c, o);
    if (dw) {
#pragma unroll
      for (int i = 0; i < 8; ++i) atomicAdd(dw + c + i, a[i] * b[i] * rs);
    }
  }
}

// Same, for H = NC * 256 with the row held in registers: every lane issues its 2 NC (3 NC with dh_add) 16-byte loads
// before the first use, and nothing is read twice.
template <int NC>
__global__ void __launch_bounds__(256) rmsnorm_bwd_reg_kernel(const __nv_bfloat16* __restrict__ dy,
                                                              const __nv_bfloat16* __restrict__ h,
                                                              const __nv_bfloat16* __restrict__ w,
                                                              const float* __restrict__ rstd,
                                                              const __nv_bfloat16* __restrict__ dh_add,
                                                              __nv_bfloat16* __restrict__ dx, float* __restrict__ dw,
                                                              int T) {
  constexpr int H = NC * 256;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= T) return;
  const size_t off = static_cast<size_t>(row) * H;
  float a[NC][8], b[NC][8], e[NC][8];
#pragma unroll
  for (int u = 0; u < NC; ++u) {
    load8(dy + off + u * 256 + lane * 8, a[u]);
    load8(h + off + u * 256 + lane * 8, b[u]);
  }
  if (dh_add) {
#pragma unroll
    for (int u = 0; u < NC; ++u) load8(dh_add + off + u * 256 + lane * 8, e[u]);
  }
  const float rs = rstd[row];
  float dot = 0.f;
#pragma unroll
  for (int u = 0; u < NC; ++u) {
    float g[8];
    load8(w + u * 256 + lane * 8, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      b[u][i] *= rs;                       // xhat
      if (dw) atomicAdd(dw + u * 256 + lane * 8 + i, a[u][i] * b[u][i]);
      a[u][i] *= g[i];                     // dy * w
      dot += a[u][i] * b[u][i];
    }
  }
  dot = warp_sum(dot) / H;
#pragma unroll
  for (int u = 0; u < NC; ++u) {
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = rs * (a[u][i] - b[u][i] * dot) + (dh_add ? e[u][i] : 0.f);
    store8(dx + off + u * 256 + lane * 8, o);
  }
}

// ------------------------------------------------------------------------------------ RoPE table
__global__ void rope_table_kernel(const int* __restrict__ pos, float* __restrict__ cs, float* __restrict__ sn, int T,
                                  int half, float theta, float inv_scale) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * half) return;
  const int t = i / half, j = i - t * half;
  const float inv_freq = powf(theta, -static_cast<float>(j) / half) * inv_scale;
  float s, c;
  sincosf(static_cast<float>(pos[t]) * inv_freq, &s, &c);
  cs[i] = c;
  sn[i] = s;
}

// Same table from a precomputed frequency vector (llama3 / yarn / NTK / longrope schedules are built once on the host);
// `mscale` is the schedule's attention factor, applied to both cos and sin.
__global__ void rope_table_freqs_kernel(const int* __restrict__ pos, const float* __restrict__ inv_freq,
                                        float* __restrict__ cs, float* __restrict__ sn, int T, int half, float mscale) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * half) return;
  const int t = i / half, j = i - t * half;
  float s, c;
  sincosf(static_cast<float>(pos[t]) * inv_freq[j], &s, &c);
  cs[i] = c * mscale;
  sn[i] = s * mscale;
}

// ------------------------------------------------------------------------------------ QK-norm + RoPE (D = 128)
// One warp per (token, head). Lane l owns elements {4l..4l+3} of the vector: the first 16 lanes hold
// the first half (j < 64), the last 16 the second half; rotation partners are exchanged by shuffle.
__global__ void qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, int ld,
                                       const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw,
                                       const float* __restrict__ cs, const float* __restrict__ sn,
                                       __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_out, int T,
                                       int hq, int hkv, float eps) {
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads = hq + hkv;
  if (gw >= T * heads) return;
  const int t = gw / heads, hh = gw - t * heads;
  const bool is_q = hh < hq;
  const __nv_bfloat16* src = qkv + static_cast<size_t>(t) * ld + hh * 128 + lane * 4;
  const __nv_bfloat16* wv = is_q ? qw : kw;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  float x[4];
  {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
  }
  if (wv) {
    float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / 128.f + eps);
    const uint2 wr = *reinterpret_cast<const uint2*>(wv + lane * 4);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wr.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wr.y));
    x[0] *= rs * a.x; x[1] *= rs * a.y; x[2] *= rs * b.x; x[3] *= rs * b.y;
  }
  const int j = (lane & 15) * 4;
  const float4 c = *reinterpret_cast<const float4*>(cs + static_cast<size_t>(t) * 64 + j);
  const float4 s = *reinterpret_cast<const float4*>(sn + static_cast<size_t>(t) * 64 + j);
  const float cc[4] = {c.x, c.y, c.z, c.w}, ssn[4] = {s.x, s.y, s.z, s.w};
  float o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float partner = __shfl_xor_sync(0xffffffffu, x[i], 16);
    // first half: x1*c - x2*s ; second half: x2*c + x1*s
    o[i] = (lane < 16) ? (x[i] * cc[i] - partner * ssn[i]) : (x[i] * cc[i] + partner * ssn[i]);
  }
  __nv_bfloat16* dst = is_q ? q_out + (static_cast<size_t>(t) * hq + hh) * 128 + lane * 4
                            : k_out + (static_cast<size_t>(t) * hkv + (hh - hq)) * 128 + lane * 4;
  uint2 ov;
  *reinterpret_cast<__nv_bfloat162*>(&ov.x) = __floats2bfloat162_rn(o[0], o[1]);
  *reinterpret_cast<__nv_bfloat162*>(&ov.y) = __floats2bfloat162_rn(o[2], o[3]);
  *reinterpret_cast<uint2*>(dst) = ov;
}

// Wide variants for whole batches: sixteen lanes per (token, head) and two consecutive heads per half-warp. Lane l owns
// the four rotation pairs j = 4l .. 4l+3, i.e. elements {j} of the first half and {64 + j} of the second (two 8-byte
// loads), so the rotation needs no exchange between lanes; the only shuffles are the four steps of the sum of squares.
// Both heads of a half-warp usually belong to one token and share its cos / sin registers.
__device__ __forceinline__ float half16_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ void unpack4(const uint2& r, float (&f)[4]) {
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ uint2 pack4(const float (&f)[4]) {
  uint2 r;
  *reinterpret_cast<__nv_bfloat162*>(&r.x) = __floats2bfloat162_rn(f[0], f[1]);
  *reinterpret_cast<__nv_bfloat162*>(&r.y) = __floats2bfloat162_rn(f[2], f[3]);
  return r;
}
__device__ __forceinline__ void load4f(const float* __restrict__ p, float (&c)[4]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  c[0] = a.x; c[1] = a.y; c[2] = a.z; c[3] = a.w;
}

constexpr int kQkU = 2;   // heads per half-warp
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }   // null counts as aligned

__global__ void __launch_bounds__(256) qknorm_rope_fwd_wide_kernel(
    const __nv_bfloat16* __restrict__ qkv, int ld, const __nv_bfloat16* __restrict__ qw,
    const __nv_bfloat16* __restrict__ kw, const float* __restrict__ cs, const float* __restrict__ sn,
    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_out, int T, int hq, int hkv, float eps) {
  const long long warp_g = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31, l16 = lane & 15, sub = lane >> 4;
  const int heads = hq + hkv;
  const long long total = static_cast<long long>(T) * heads;
  uint2 lo[kQkU], hi[kQkU];
  int tt[kQkU], hh[kQkU];
  bool ok[kQkU];
#pragma unroll
  for (int u = 0; u < kQkU; ++u) {
    const long long g = (warp_g * 2 + sub) * kQkU + u;
    ok[u] = g < total;
    const long long gc = ok[u] ? g : 0;
    tt[u] = static_cast<int>(gc / heads);
    hh[u] = static_cast<int>(gc - static_cast<long long>(tt[u]) * heads);
    const __nv_bfloat16* src = qkv + static_cast<size_t>(tt[u]) * ld + hh[u] * 128 + l16 * 4;
    lo[u] = ok[u] ? *reinterpret_cast<const uint2*>(src) : make_uint2(0, 0);
    hi[u] = ok[u] ? *reinterpret_cast<const uint2*>(src + 64) : make_uint2(0, 0);
  }
  float c[4], s4[4];
#pragma unroll
  for (int u = 0; u < kQkU; ++u) {
    if (u == 0 || tt[u] != tt[u - 1]) {
      load4f(cs + static_cast<size_t>(tt[u]) * 64 + l16 * 4, c);
      load4f(sn + static_cast<size_t>(tt[u]) * 64 + l16 * 4, s4);
    }
    const bool is_q = hh[u] < hq;
    const __nv_bfloat16* wv = is_q ? qw : kw;
    float x1[4], x2[4];
    unpack4(lo[u], x1);
    unpack4(hi[u], x2);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) ss += x1[i] * x1[i] + x2[i] * x2[i];
    ss = half16_sum(ss);           // every lane takes part; heads without a norm weight keep x
    if (wv) {
      const float rs = rsqrtf(ss / 128.f + eps);
      float w1[4], w2[4];
      unpack4(*reinterpret_cast<const uint2*>(wv + l16 * 4), w1);
      unpack4(*reinterpret_cast<const uint2*>(wv + 64 + l16 * 4), w2);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        x1[i] *= rs * w1[i];
        x2[i] *= rs * w2[i];
      }
    }
    float o1[4], o2[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o1[i] = x1[i] * c[i] - x2[i] * s4[i];
      o2[i] = x2[i] * c[i] + x1[i] * s4[i];
    }
    if (ok[u]) {
      __nv_bfloat16* dst = is_q ? q_out + (static_cast<size_t>(tt[u]) * hq + hh[u]) * 128 + l16 * 4
                                : k_out + (static_cast<size_t>(tt[u]) * hkv + (hh[u] - hq)) * 128 + l16 * 4;
      *reinterpret_cast<uint2*>(dst) = pack4(o1);
      *reinterpret_cast<uint2*>(dst + 64) = pack4(o2);
    }
  }
}

__global__ void __launch_bounds__(256) qknorm_rope_bwd_wide_kernel(
    const __nv_bfloat16* __restrict__ dq, const __nv_bfloat16* __restrict__ dk, const __nv_bfloat16* __restrict__ qkv,
    int ld, const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw, const float* __restrict__ cs,
    const float* __restrict__ sn, __nv_bfloat16* __restrict__ dqkv, int T, int hq, int hkv, float eps) {
  const long long warp_g = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31, l16 = lane & 15, sub = lane >> 4;
  const int heads = hq + hkv;
  const long long total = static_cast<long long>(T) * heads;
  const bool norm = qw != nullptr || kw != nullptr;
  uint2 glo[kQkU], ghi[kQkU], xlo[kQkU], xhi[kQkU];
  int tt[kQkU], hh[kQkU];
  bool ok[kQkU];
#pragma unroll
  for (int u = 0; u < kQkU; ++u) {
    const long long g = (warp_g * 2 + sub) * kQkU + u;
    ok[u] = g < total;
    const long long gc = ok[u] ? g : 0;
    tt[u] = static_cast<int>(gc / heads);
    hh[u] = static_cast<int>(gc - static_cast<long long>(tt[u]) * heads);
    const bool is_q = hh[u] < hq;
    const __nv_bfloat16* gsrc = is_q ? dq + (static_cast<size_t>(tt[u]) * hq + hh[u]) * 128 + l16 * 4
                                     : dk + (static_cast<size_t>(tt[u]) * hkv + (hh[u] - hq)) * 128 + l16 * 4;
    const __nv_bfloat16* xsrc = qkv + static_cast<size_t>(tt[u]) * ld + hh[u] * 128 + l16 * 4;
    glo[u] = ok[u] ? *reinterpret_cast<const uint2*>(gsrc) : make_uint2(0, 0);
    ghi[u] = ok[u] ? *reinterpret_cast<const uint2*>(gsrc + 64) : make_uint2(0, 0);
    xlo[u] = (ok[u] && norm) ? *reinterpret_cast<const uint2*>(xsrc) : make_uint2(0, 0);
    xhi[u] = (ok[u] && norm) ? *reinterpret_cast<const uint2*>(xsrc + 64) : make_uint2(0, 0);
  }
  float c[4], s4[4];
#pragma unroll
  for (int u = 0; u < kQkU; ++u) {
    if (u == 0 || tt[u] != tt[u - 1]) {
      load4f(cs + static_cast<size_t>(tt[u]) * 64 + l16 * 4, c);
      load4f(sn + static_cast<size_t>(tt[u]) * 64 + l16 * 4, s4);
    }
    const bool is_q = hh[u] < hq;
    const __nv_bfloat16* wv = is_q ? qw : kw;
    float g1[4], g2[4], d1[4], d2[4];
    unpack4(glo[u], g1);
    unpack4(ghi[u], g2);
#pragma unroll
    for (int i = 0; i < 4; ++i) {      // transpose of the rotation
      d1[i] = g1[i] * c[i] + g2[i] * s4[i];
      d2[i] = g2[i] * c[i] - g1[i] * s4[i];
    }
    float x1[4], x2[4], w1[4] = {0.f, 0.f, 0.f, 0.f}, w2[4] = {0.f, 0.f, 0.f, 0.f};
    unpack4(xlo[u], x1);
    unpack4(xhi[u], x2);
    if (wv) {
      unpack4(*reinterpret_cast<const uint2*>(wv + l16 * 4), w1);
      unpack4(*reinterpret_cast<const uint2*>(wv + 64 + l16 * 4), w2);
    }
    // both sums are reduced by every lane (the two half-warps may hold heads of different kinds)
    float ss = 0.f, dwx = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      ss += x1[i] * x1[i] + x2[i] * x2[i];
      dwx += d1[i] * w1[i] * x1[i] + d2[i] * w2[i] * x2[i];
    }
    ss = half16_sum(ss);
    dwx = half16_sum(dwx);
    const float rs = rsqrtf(ss / 128.f + eps);
    const float dot = dwx * rs / 128.f;
    float o1[4], o2[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o1[i] = wv ? rs * (d1[i] * w1[i] - x1[i] * rs * dot) : d1[i];
      o2[i] = wv ? rs * (d2[i] * w2[i] - x2[i] * rs * dot) : d2[i];
    }
    if (ok[u]) {
      __nv_bfloat16* dst = dqkv + static_cast<size_t>(tt[u]) * ld + hh[u] * 128 + l16 * 4;
      *reinterpret_cast<uint2*>(dst) = pack4(o1);
      *reinterpret_cast<uint2*>(dst + 64) = pack4(o2);
    }
  }
}

// Decode variant: q heads go to q_out; k heads are normalised, rotated and written straight into the paged key cache
// at the token's slot; v heads are copied into the value cache. One warp per (token, head) over hq + 2 hkv heads.
__global__ void qknorm_rope_cache_kernel(const __nv_bfloat16* __restrict__ qkv, int ld,
                                         const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw,
                                         const float* __restrict__ cs, const float* __restrict__ sn,
                                         __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache,
                                         __nv_bfloat16* __restrict__ v_cache, const long long* __restrict__ slots, int T,
                                         int hq, int hkv, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads = hq + 2 * hkv;
  if (gw >= T * heads) return;
  const int t = gw / heads, hh = gw - t * heads;
  const long long slot = slots[t];
  const uint2 raw = *reinterpret_cast<const uint2*>(qkv + static_cast<size_t>(t) * ld + hh * 128 + lane * 4);
  if (hh >= hq + hkv) {   // value head: plain copy into the cache
    if (slot >= 0) *reinterpret_cast<uint2*>(v_cache + (slot * hkv + (hh - hq - hkv)) * 128 + lane * 4) = raw;
    return;
  }
  const bool is_q = hh < hq;
  const __nv_bfloat16* wv = is_q ? qw : kw;
  float x[4];
  {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
  }
  if (wv) {
    float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / 128.f + eps);
    const uint2 wr = *reinterpret_cast<const uint2*>(wv + lane * 4);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wr.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wr.y));
    x[0] *= rs * a.x; x[1] *= rs * a.y; x[2] *= rs * b.x; x[3] *= rs * b.y;
  }
  const int j = (lane & 15) * 4;
  const float4 c = *reinterpret_cast<const float4*>(cs + static_cast<size_t>(t) * 64 + j);
  const float4 s = *reinterpret_cast<const float4*>(sn + static_cast<size_t>(t) * 64 + j);
  const float cc[4] = {c.x, c.y, c.z, c.w}, ssn[4] = {s.x, s.y, s.z, s.w};
  float o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float partner = __shfl_xor_sync(0xffffffffu, x[i], 16);
    o[i] = (lane < 16) ? (x[i] * cc[i] - partner * ssn[i]) : (x[i] * cc[i] + partner * ssn[i]);
  }
  uint2 ov;
  *reinterpret_cast<__nv_bfloat162*>(&ov.x) = __floats2bfloat162_rn(o[0], o[1]);
  *reinterpret_cast<__nv_bfloat162*>(&ov.y) = __floats2bfloat162_rn(o[2], o[3]);
  if (is_q) *reinterpret_cast<uint2*>(q_out + (static_cast<size_t>(t) * hq + hh) * 128 + lane * 4) = ov;
  else if (slot >= 0) *reinterpret_cast<uint2*>(k_cache + (slot * hkv + (hh - hq)) * 128 + lane * 4) = ov;
}

__global__ void qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dq, const __nv_bfloat16* __restrict__ dk,
                                       const __nv_bfloat16* __restrict__ qkv, int ld,
                                       const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw,
                                       const float* __restrict__ cs, const float* __restrict__ sn,
                                       __nv_bfloat16* __restrict__ dqkv, int T, int hq, int hkv, float eps) {
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads = hq + hkv;
  if (gw >= T * heads) return;
  const int t = gw / heads, hh = gw - t * heads;
  const bool is_q = hh < hq;
  const __nv_bfloat16* gsrc = is_q ? dq + (static_cast<size_t>(t) * hq + hh) * 128 + lane * 4
                                   : dk + (static_cast<size_t>(t) * hkv + (hh - hq)) * 128 + lane * 4;
  const uint2 graw = *reinterpret_cast<const uint2*>(gsrc);
  float g[4];
  {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&graw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&graw.y));
    g[0] = a.x; g[1] = a.y; g[2] = b.x; g[3] = b.y;
  }
  const int j = (lane & 15) * 4;
  const float4 c = *reinterpret_cast<const float4*>(cs + static_cast<size_t>(t) * 64 + j);
  const float4 s = *reinterpret_cast<const float4*>(sn + static_cast<size_t>(t) * 64 + j);
  const float cc[4] = {c.x, c.y, c.z, c.w}, ssn[4] = {s.x, s.y, s.z, s.w};
  float dn[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float partner = __shfl_xor_sync(0xffffffffu, g[i], 16);
    // transpose of the rotation: dn1 = dy1*c + dy2*s ; dn2 = dy2*c - dy1*s
    dn[i] = (lane < 16) ? (g[i] * cc[i] + partner * ssn[i]) : (g[i] * cc[i] - partner * ssn[i]);
  }
  const size_t off = static_cast<size_t>(t) * ld + hh * 128 + lane * 4;
  const __nv_bfloat16* wv = is_q ? qw : kw;
  float o[4];
  if (wv) {
    const uint2 xr = *reinterpret_cast<const uint2*>(qkv + off);
    const uint2 wr = *reinterpret_cast<const uint2*>(wv + lane * 4);
    float x[4], w4[4];
    {
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xr.x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xr.y));
      x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
      const float2 e = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wr.x));
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wr.y));
      w4[0] = e.x; w4[1] = e.y; w4[2] = f.x; w4[3] = f.y;
    }
    float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / 128.f + eps);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) dot += dn[i] * w4[i] * x[i] * rs;
    dot = warp_sum(dot) / 128.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = rs * (dn[i] * w4[i] - x[i] * rs * dot);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = dn[i];
  }
  uint2 ov;
  *reinterpret_cast<__nv_bfloat162*>(&ov.x) = __floats2bfloat162_rn(o[0], o[1]);
  *reinterpret_cast<__nv_bfloat162*>(&ov.y) = __floats2bfloat162_rn(o[2], o[3]);
  *reinterpret_cast<uint2*>(dqkv + off) = ov;
}

// ------------------------------------------------------------------------------------ SwiGLU
// gate_up [T, 2I] (gate | up) -> out [T, I]
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, long long T,
                                  int I) {
  const long long n8 = T * (I / 8);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / (I / 8);
    const int c = static_cast<int>(i - t * (I / 8)) * 8;
    float g[8], u[8], o[8];
    load8(gu + t * 2 * I + c, g);
    load8(gu + t * 2 * I + I + c, u);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = g[k] / (1.f + __expf(-g[k])) * u[k];
    store8(out + t * I + c, o);
  }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, long long T, int I) {
  const long long n8 = T * (I / 8);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / (I / 8);
    const int c = static_cast<int>(i - t * (I / 8)) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gu + t * 2 * I + c, g);
    load8(gu + t * 2 * I + I + c, u);
    load8(dout + t * I + c, d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float sg = 1.f / (1.f + __expf(-g[k]));
      dg[k] = d[k] * u[k] * sg * (1.f + g[k] * (1.f - sg));
      du[k] = d[k] * g[k] * sg;
    }
    store8(dgu + t * 2 * I + c, dg);
    store8(dgu + t * 2 * I + I + c, du);
  }
}

// ------------------------------------------------------------------------------------ gated activations (GLU family)
// out = act(gate) * up with gate and up as separate row-strided matrices (two projections, or the two halves of a fused
// one). kAct: 0 SiLU (SwiGLU), 1 GELU with the tanh approximation (GeGLU of Gemma), 2 exact GELU (erf).
template <int kAct>
__device__ __forceinline__ void glu_act(float g, float* a, float* da) {
  if (kAct == 0) {
    const float sg = 1.f / (1.f + __expf(-g));
    *a = g * sg;
    *da = sg * (1.f + g * (1.f - sg));
  } else if (kAct == 1) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    const float u = k0 * (g + k1 * g * g * g);
    const float t = tanhf(u);
    *a = 0.5f * g * (1.f + t);
    *da = 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * k0 * (1.f + 3.f * k1 * g * g);
  } else {
    const float cdf = 0.5f * (1.f + erff(g * 0.7071067811865476f));
    *a = g * cdf;
    *da = cdf + g * 0.3989422804014327f * __expf(-0.5f * g * g);
  }
}
template <int kAct>
__global__ void glu_fwd_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up, long long ldg,
                               long long ldu, __nv_bfloat16* __restrict__ out, long long T, int I) {
  const long long n8 = T * (I / 8);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / (I / 8);
    const int c = static_cast<int>(i - t * (I / 8)) * 8;
    float g[8], u[8], o[8];
    load8(gate + t * ldg + c, g);
    load8(up + t * ldu + c, u);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float a, da;
      glu_act<kAct>(g[k], &a, &da);
      o[k] = a * u[k];
    }
    store8(out + t * I + c, o);
  }
}
template <int kAct>
__global__ void glu_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ gate,
                               const __nv_bfloat16* __restrict__ up, long long ldg, long long ldu,
                               __nv_bfloat16* __restrict__ dgate, __nv_bfloat16* __restrict__ dup, long long lddg,
                               long long lddu, long long T, int I) {
  const long long n8 = T * (I / 8);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / (I / 8);
    const int c = static_cast<int>(i - t * (I / 8)) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gate + t * ldg + c, g);
    load8(up + t * ldu + c, u);
    load8(dout + t * I + c, d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float a, da;
      glu_act<kAct>(g[k], &a, &da);
      dg[k] = d[k] * u[k] * da;
      du[k] = d[k] * a;
    }
    store8(dgate + t * lddg + c, dg);
    store8(dup + t * lddu + c, du);
  }
}

// ------------------------------------------------------------------------------------ cross-entropy on a logits chunk
// One block per row. logits (bf16, [n, ldl]) are replaced in place by d(loss_sum)/dlogits * grad_scale,
// where grad_scale = *inv_n (1 / number of valid tokens of the whole batch). Adds the row's loss to loss_sum.
// Rows whose label is ignore_index get a zero gradient. Options (compile-time kOpt for the two that touch every element):
//   softcap c > 0:  the logits are c * tanh(x / c) before the softmax (gradient times 1 - tanh^2)
//   smoothing e:    loss = lse - (1 - e) x[label] - e * mean(x)   (gradient  softmax - (1 - e) onehot - e / V)
//   z_coef:         adds z_coef * lse^2 (gradient factor 1 + 2 z_coef lse on the softmax term)
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <bool kOpt>
__global__ void ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, long long ldl, const long long* __restrict__ labels,
                                  float* __restrict__ loss_sum, const float* __restrict__ inv_n,
                                  float* __restrict__ row_loss, const float* __restrict__ row_scale, int V,
                                  long long ignore_index, int write_grad, float z_coef, float* __restrict__ z_sum,
                                  float smooth, float cap) {
  __shared__ float red[32];
  __shared__ float bcast[2];
  const int row = blockIdx.x;
  __nv_bfloat16* lr = logits + static_cast<size_t>(row) * ldl;
  const long long label = labels[row];
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int V8 = V & ~7;
  if (label == ignore_index || label < 0 || label >= V) {
    if (row_loss && tid == 0) row_loss[row] = 0.f;
    if (write_grad) {
      const bf16x8 z = {};
      for (int c = tid * 8; c < V8; c += nthr * 8) *reinterpret_cast<bf16x8*>(lr + c) = z;
      for (int c = V8 + tid; c < V; c += nthr) lr[c] = __float2bfloat16(0.f);
    }
    return;
  }
  const bool capped = kOpt && cap > 0.f;
  const float inv_cap = capped ? 1.f / cap : 0.f;
  // pass 1: online max / sum-exp (and the plain sum of the logits for the smoothing term)
  float m = -INFINITY, s = 0.f, sx = 0.f;
  for (int c = tid * 8; c < V8; c += nthr * 8) {
    float f[8];
    load8(lr + c, f);
    if (kOpt) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (capped) f[i] = cap * tanh_fast(f[i] * inv_cap);
        sx += f[i];
      }
    }
    float lm = f[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) lm = fmaxf(lm, f[i]);
    if (lm > m) { s *= __expf(m - lm); m = lm; }
#pragma unroll
    for (int i = 0; i < 8; ++i) s += __expf(f[i] - m);
  }
  for (int c = V8 + tid; c < V; c += nthr) {
    float f = __bfloat162float(lr[c]);
    if (kOpt) {
      if (capped) f = cap * tanh_fast(f * inv_cap);
      sx += f;
    }
    if (f > m) { s *= __expf(m - f); m = f; }
    s += __expf(f - m);
  }
  // block reduce (m, s)
  const float wm = warp_max(m);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - wm);
  s = warp_sum(s);
  if ((tid & 31) == 0) { red[tid >> 5] = wm; }
  __syncthreads();
  float bm = -INFINITY;
  const int nw = nthr >> 5;
  for (int i = 0; i < nw; ++i) bm = fmaxf(bm, red[i]);
  __syncthreads();
  s = (wm == -INFINITY) ? 0.f : s * __expf(wm - bm);
  if ((tid & 31) == 0) red[tid >> 5] = s;
  __syncthreads();
  float tot = 0.f;
  if (tid == 0)
    for (int i = 0; i < nw; ++i) tot += red[i];
  float sx_tot = 0.f;
  if (kOpt) {                       // second use of the scratch array: the sum of the logits
    __syncthreads();
    sx = warp_sum(sx);
    if ((tid & 31) == 0) red[tid >> 5] = sx;
    __syncthreads();
    if (tid == 0)
      for (int i = 0; i < nw; ++i) sx_tot += red[i];
  }
  if (tid == 0) {
    const float lse = bm + logf(tot);
    bcast[0] = lse;
    float xl = __bfloat162float(lr[label]);
    if (capped) xl = cap * tanh_fast(xl * inv_cap);
    float rl = lse - xl;
    if (kOpt && smooth > 0.f) rl = lse - (1.f - smooth) * xl - smooth * sx_tot / static_cast<float>(V);
    if (row_loss) row_loss[row] = rl;
    if (loss_sum) atomicAdd(loss_sum, rl);
    if (z_sum) atomicAdd(z_sum, lse * lse);
  }
  __syncthreads();
  if (!write_grad) return;
  const float lse = bcast[0];
  const float gs = row_scale ? row_scale[row] : *inv_n;
  // with the z term  z_coef * lse^2  the gradient is  (1 + 2 z_coef lse) softmax - onehot
  const float pz = 1.f + 2.f * z_coef * lse;
  const float hot = kOpt ? 1.f - smooth : 1.f;
  const float uni = kOpt ? smooth / static_cast<float>(V) : 0.f;
  for (int c = tid * 8; c < V8; c += nthr * 8) {
    float f[8];
    load8(lr + c, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float x = f[i], dcap = 1.f;
      if (capped) {
        const float t = tanh_fast(x * inv_cap);
        x = cap * t;
        dcap = 1.f - t * t;
      }
      f[i] = (pz * __expf(x - lse) - ((c + i) == label ? hot : 0.f) - uni) * gs * dcap;
    }
    store8(lr + c, f);
  }
  for (int c = V8 + tid; c < V; c += nthr) {
    float x = __bfloat162float(lr[c]), dcap = 1.f;
    if (capped) {
      const float t = tanh_fast(x * inv_cap);
      x = cap * t;
      dcap = 1.f - t * t;
    }
    lr[c] = __float2bfloat16((pz * __expf(x - lse) - (c == label ? hot : 0.f) - uni) * gs * dcap);
  }
}

// ------------------------------------------------------------------------------------ sum of squares
__global__ void sumsq_kernel(const float* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float red[32];
  float acc = 0.f;
  const long long n4 = n >> 2;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 v = x4[i];
    acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long long i = n4 << 2; i < n; ++i) acc += x[i] * x[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) atomicAdd(out, v);
  }
}

// ------------------------------------------------------------------------------------ flat AdamW
// Reference semantics (crates/pmetal-bridge/src/optimizer.rs:295-336): bias-corrected step, then
// decoupled decay applied to the updated parameter. Per-1024-element chunk lr multiplier and decay.
// gnorm_sq holds the squared global norm of the *unscaled* gradient buffer.
struct AdamwArgs {
  float lr, beta1, beta2, eps, bc1, bc2, grad_scale, max_norm;
};
__global__ void adamw_flat_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                                  float* __restrict__ v, __nv_bfloat16* __restrict__ shadow,
                                  const float* __restrict__ lr_mult, const float* __restrict__ wd,
                                  const float* __restrict__ gnorm_sq, const float* __restrict__ hp, long long n,
                                  AdamwArgs a) {
  if (hp) {   // step-dependent scalars kept on the device so that a captured graph can be replayed
    a.lr = hp[0];
    a.bc1 = hp[1];
    a.bc2 = hp[2];
  }
  float coef = a.grad_scale;
  if (a.max_norm > 0.f) {
    const float norm = sqrtf(*gnorm_sq) * a.grad_scale;
    coef *= fminf(1.f, a.max_norm / (norm + 1e-6f));
  }
  for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 4; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
    const int chunk = static_cast<int>(i >> 10);
    const float lr = a.lr * lr_mult[chunk];
    const float decay = wd[chunk] * lr;
    const float4 g4 = *reinterpret_cast<const float4*>(g + i);
    float4 m4 = *reinterpret_cast<float4*>(m + i);
    float4 v4 = *reinterpret_cast<float4*>(v + i);
    float4 p4 = *reinterpret_cast<float4*>(p + i);
    float gg[4] = {g4.x * coef, g4.y * coef, g4.z * coef, g4.w * coef};
    float mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w}, pp[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      mm[k] = a.beta1 * mm[k] + (1.f - a.beta1) * gg[k];
      vv[k] = a.beta2 * vv[k] + (1.f - a.beta2) * gg[k] * gg[k];
      const float mh = mm[k] / a.bc1, vh = vv[k] / a.bc2;
      pp[k] -= lr * mh / (sqrtf(vh) + a.eps);
      pp[k] -= decay * pp[k];
    }
    *reinterpret_cast<float4*>(m + i) = make_float4(mm[0], mm[1], mm[2], mm[3]);
    *reinterpret_cast<float4*>(v + i) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    *reinterpret_cast<float4*>(p + i) = make_float4(pp[0], pp[1], pp[2], pp[3]);
    if (shadow) {
      uint2 o;
      *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(pp[0], pp[1]);
      *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(pp[2], pp[3]);
      *reinterpret_cast<uint2*>(shadow + i) = o;
    }
  }
}

// rowsum(dO * O) per (token, head): the delta term of the attention backward. One warp per row of 128.
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                  float* __restrict__ delta, int T, int H) {
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (gw >= T * H) return;
  const int t = gw / H, h = gw - t * H;
  const size_t off = static_cast<size_t>(gw) * 128 + lane * 4;
  const uint2 a = *reinterpret_cast<const uint2*>(o + off);
  const uint2 b = *reinterpret_cast<const uint2*>(dout + off);
  const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
  const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
  const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.x));
  const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.y));
  float s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
  s = warp_sum(s);
  if (lane == 0) delta[static_cast<size_t>(h) * T + t] = s;
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    out[i] = __float2bfloat16(in[i]);
}

// ------------------------------------------------------------------------------------ 4-bit block dequantisation
// NF4 / FP4 codes (two per byte, first element in the high nibble) with per-block absmax, optionally
// double-quantised (u8 * scale + offset)  ->  bf16. Layout of crates/pmetal-mlx/src/quantization/nf4.rs.
__constant__ float kNf4Lut[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                                  -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                                  0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
                                  0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};
__constant__ float kFp4Lut[16] = {0.0f, 0.0052083333f, 0.6666667f, 1.0f, 0.3333333f, 0.5f, 0.1666667f, 0.25f,
                                  -0.0f, -0.0052083333f, -0.6666667f, -1.0f, -0.3333333f, -0.5f, -0.1666667f, -0.25f};

__global__ void dequant_4bit_kernel(const uint8_t* __restrict__ data, const float* __restrict__ absmax,
                                    const uint8_t* __restrict__ absmax_q, float am_scale, float am_offset,
                                    __nv_bfloat16* __restrict__ out, long long n, int block_size, int fp4) {
  __shared__ float lut[16];
  if (threadIdx.x < 16) lut[threadIdx.x] = fp4 ? kFp4Lut[threadIdx.x] : kNf4Lut[threadIdx.x];
  __syncthreads();
  const long long n8 = n >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint32_t packed = *reinterpret_cast<const uint32_t*>(data + i * 4);
    const long long blk = (i * 8) / block_size;
    const float am = absmax ? absmax[blk] : (static_cast<float>(absmax_q[blk]) * am_scale + am_offset);
    float f[8];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const uint32_t byte = (packed >> (8 * b)) & 0xFFu;
      f[2 * b] = lut[byte >> 4] * am;
      f[2 * b + 1] = lut[byte & 0xFu] * am;
    }
    store8(out + i * 8, f);
  }
  // tail (n not a multiple of 8)
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (long long e = n8 << 3; e < n; ++e) {
      const uint8_t byte = data[e >> 1];
      const uint32_t code = (e & 1) ? (byte & 0xFu) : (byte >> 4);
      const long long blk = e / block_size;
      const float am = absmax ? absmax[blk] : (static_cast<float>(absmax_q[blk]) * am_scale + am_offset);
      out[e] = __float2bfloat16(lut[code] * am);
    }
  }
}

}  // namespace pm

using namespace pm;

static inline int grid_for(long long work, int per_block, int cap = 0) {
  if (cap <= 0) cap = num_sms() * 16;
  long long g = (work + per_block - 1) / per_block;
  if (g < 1) g = 1;
  return static_cast<int>(g > cap ? cap : g);
}
#define PM_LAUNCH_CHECK() static_cast<int>(cudaGetLastError())

extern "C" int pm_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd, int T,
                              int H, float eps, cudaStream_t st) {
  if (H % 8) return -1;
  if (T <= 592 && H <= 4096) {        // fewer row groups than SMs: spread the rows instead
    rmsnorm_fwd_row_kernel<<<T, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(res),
        static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), static_cast<__nv_bfloat16*>(h_out), rstd, H,
        eps);
    return PM_LAUNCH_CHECK();
  }
  rmsnorm_fwd_kernel<<<(T + 7) / 8, 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(res),
      static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), static_cast<__nv_bfloat16*>(h_out), rstd, T,
      H, eps);
  return PM_LAUNCH_CHECK();
}
extern "C" int pm_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd, const void* dh_add,
                              void* dx, float* dw, int T, int H, cudaStream_t st) {
  if (H % 8) return -1;
  if (H % 256 == 0 && H <= 2048) {
    const dim3 grid((T + 7) / 8);
    const __nv_bfloat16 *a = static_cast<const __nv_bfloat16*>(dy), *b = static_cast<const __nv_bfloat16*>(h),
                        *g = static_cast<const __nv_bfloat16*>(w), *e = static_cast<const __nv_bfloat16*>(dh_add);
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(dx);
    switch (H / 256) {
      case 1: rmsnorm_bwd_reg_kernel<1><<<grid, 256, 0, st>>>(a, b, g, rstd, e, o, dw, T); break;
      case 2: rmsnorm_bwd_reg_kernel<2><<<grid, 256, 0, st>>>(a, b, g, rstd, e, o, dw, T); break;
      case 3: rmsnorm_bwd_reg_kernel<3><<<grid, 256, 0, st>>>(a, b, g, rstd, e, o, dw, T); break;
      case 4: rmsnorm_bwd_reg_kernel<4><<<grid, 256, 0, st>>>(a, b, g, rstd, e, o, dw, T); break;
      case 5: rmsnorm_bwd_reg_kernel<5><<<grid, 256, 0, st>>>(a, b, g, rstd, e, o, dw, T); break;
      case 6: rmsnorm_bwd_reg_kernel<6><<<grid, 256, 0, st>>>(a, b, g, rstd, e, o, dw, T); break;
      case 7: rmsnorm_bwd_reg_kernel<7><<<grid, 256, 0, st>>>(a, b, g, rstd, e, o, dw, T); break;
      default: rmsnorm_bwd_reg_kernel<8><<<grid, 256, 0, st>>>(a, b, g, rstd, e, o, dw, T); break;
    }
    return PM_LAUNCH_CHECK();
  }
  rmsnorm_bwd_kernel<<<(T + 7) / 8, 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(h),
      static_cast<const __nv_bfloat16*>(w), rstd, static_cast<const __nv_bfloat16*>(dh_add),
      static_cast<__nv_bfloat16*>(dx), dw, T, H);
  return PM_LAUNCH_CHECK();
}
extern "C" int pm_rope_table(const int* pos, float* cs, float* sn, int T, int half, float theta, float rope_scale,
                             cudaStream_t st) {
  const long long n = static_cast<long long>(T) * half;
  rope_table_kernel<<<static_cast<int>((n + 255) / 256), 256, 0, st>>>(pos, cs, sn, T, half, theta, 1.f / rope_scale);
  return PM_LAUNCH_CHECK();
}
extern "C" int pm_rope_table_freqs(const int* pos, const float* inv_freq, float* cs, float* sn, int T, int half,
                                   float mscale, cudaStream_t st) {
  const long long n = static_cast<long long>(T) * half;
  rope_table_freqs_kernel<<<static_cast<int>((n + 255) / 256), 256, 0, st>>>(pos, inv_freq, cs, sn, T, half, mscale);
  return PM_LAUNCH_CHECK();
}
extern "C" int pm_qknorm_rope_fwd(const void* qkv, int ld, const void* qw, const void* kw, const float* cs,
                                  const float* sn, void* q_out, void* k_out, int T, int hq, int hkv, float eps,
                                  cudaStream_t st) {
  const long long warps = static_cast<long long>(T) * (hq + hkv);
  if (warps >= 4096 && ld % 8 == 0 && aligned16(qkv) && aligned16(q_out) && aligned16(k_out) && aligned16(qw) &&
      aligned16(kw) && aligned16(cs) && aligned16(sn)) {
    const long long wide = (warps + 2 * kQkU - 1) / (2 * kQkU);
    qknorm_rope_fwd_wide_kernel<<<static_cast<int>((wide + 7) / 8), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(qkv), ld, static_cast<const __nv_bfloat16*>(qw),
        static_cast<const __nv_bfloat16*>(kw), cs, sn, static_cast<__nv_bfloat16*>(q_out),
        static_cast<__nv_bfloat16*>(k_out), T, hq, hkv, eps);
    return PM_LAUNCH_CHECK();
  }
  qknorm_rope_fwd_kernel<<<static_cast<int>((warps + 7) / 8), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(qkv), ld, static_cast<const __nv_bfloat16*>(qw),
      static_cast<const __nv_bfloat16*>(kw), cs, sn, static_cast<__nv_bfloat16*>(q_out),
      static_cast<__nv_bfloat16*>(k_out), T, hq, hkv, eps);
  return PM_LAUNCH_CHECK();
}
extern "C" int pm_qknorm_rope_cache(const void* qkv, int ld, const void* qw, const void* kw, const float* cs,
                                    const float* sn, void* q_out, void* k_cache, void* v_cache, const long long* slots,
                                    int T, int hq, int hkv, float eps, cudaStream_t st) {
  const long long warps = static_cast<long long>(T) * (hq + 2 * hkv);
  return static_cast<int>(launch_pdl(
      qknorm_rope_cache_kernel, dim3(static_cast<unsigned>((warps + 7) / 8)), dim3(256), 0, st,
      static_cast<const __nv_bfloat16*>(qkv), ld, static_cast<const __nv_bfloat16*>(qw),
      static_cast<const __nv_bfloat16*>(kw), cs, sn, static_cast<__nv_bfloat16*>(q_out),
      static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), slots, T, hq, hkv, eps));
}
extern "C" int pm_qknorm_rope_bwd(const void* dq, const void* dk, const void* qkv, int ld, const void* qw,
                                  const void* kw, const float* cs, const float* sn, void* dqkv, int T, int hq, int hkv,
                                  float eps, cudaStream_t st) {
  const long long warps = static_cast<long long>(T) * (hq + hkv);
  if (warps >= 4096 && ld % 8 == 0 && aligned16(qkv) && aligned16(dq) && aligned16(dk) && aligned16(dqkv) &&
      aligned16(qw) && aligned16(kw) && aligned16(cs) && aligned16(sn)) {
    const long long wide = (warps + 2 * kQkU - 1) / (2 * kQkU);
    qknorm_rope_bwd_wide_kernel<<<static_cast<int>((wide + 7) / 8), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(dq), static_cast<const __nv_bfloat16*>(dk),
        static_cast<const __nv_bfloat16*>(qkv), ld, static_cast<const __nv_bfloat16*>(qw),
        static_cast<const __nv_bfloat16*>(kw), cs, sn, static_cast<__nv_bfloat16*>(dqkv), T, hq, hkv, eps);
    return PM_LAUNCH_CHECK();
  }
  qknorm_rope_bwd_kernel<<<static_cast<int>((warps + 7) / 8), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(dq), static_cast<const __nv_bfloat16*>(dk),
      static_cast<const __nv_bfloat16*>(qkv), ld, static_cast<const __nv_bfloat16*>(qw),
      static_cast<const __nv_bfloat16*>(kw), cs, sn, static_cast<__nv_bfloat16*>(dqkv), T, hq, hkv, eps);
  return PM_LAUNCH_CHECK();
}
extern "C" int pm_swiglu_fwd(const void* gu, void* out, long long T, int I, cudaStream_t st) {
  if (I % 8) return -1;
  swiglu_fwd_kernel<<<grid_for(T * (I / 8), 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(gu),
                                                               static_cast<__nv_bfloat16*>(out), T, I);
  return PM_LAUNCH_CHECK();
}
extern "C" int pm_swiglu_bwd(const void* dout, const void* gu, void* dgu, long long T, int I, cudaStream_t st) {
  if (I % 8) return -1;
  swiglu_bwd_kernel<<<grid_for(T * (I / 8), 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(dgu),
      T, I);
  return PM_LAUNCH_CHECK();
}
// act(gate) * up for separate gate / up matrices (row strides in elements, multiples of 8); act: 0 SiLU, 1 GELU-tanh, 2 GELU.
extern "C" int pm_glu_fwd(const void* gate, const void* up, long long ldg, long long ldu, void* out, long long T, int I,
                          int act, cudaStream_t st) {
  if ((I % 8) || (ldg % 8) || (ldu % 8) || act < 0 || act > 2) return -1;
  const __nv_bfloat16 *g = static_cast<const __nv_bfloat16*>(gate), *u = static_cast<const __nv_bfloat16*>(up);
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
  const int grid = grid_for(T * (I / 8), 256);
  if (act == 0) glu_fwd_kernel<0><<<grid, 256, 0, st>>>(g, u, ldg, ldu, o, T, I);
  else if (act == 1) glu_fwd_kernel<1><<<grid, 256, 0, st>>>(g, u, ldg, ldu, o, T, I);
  else glu_fwd_kernel<2><<<grid, 256, 0, st>>>(g, u, ldg, ldu, o, T, I);
  return PM_LAUNCH_CHECK();
}
extern "C" int pm_glu_bwd(const void* dout, const void* gate, const void* up, long long ldg, long long ldu, void* dgate,
                          void* dup, long long lddg, long long lddu, long long T, int I, int act, cudaStream_t st) {
  if ((I % 8) || (ldg % 8) || (ldu % 8) || (lddg % 8) || (lddu % 8) || act < 0 || act > 2) return -1;
  const __nv_bfloat16 *d = static_cast<const __nv_bfloat16*>(dout), *g = static_cast<const __nv_bfloat16*>(gate),
                      *u = static_cast<const __nv_bfloat16*>(up);
  __nv_bfloat16 *dg = static_cast<__nv_bfloat16*>(dgate), *du = static_cast<__nv_bfloat16*>(dup);
  const int grid = grid_for(T * (I / 8), 256);
  if (act == 0) glu_bwd_kernel<0><<<grid, 256, 0, st>>>(d, g, u, ldg, ldu, dg, du, lddg, lddu, T, I);
  else if (act == 1) glu_bwd_kernel<1><<<grid, 256, 0, st>>>(d, g, u, ldg, ldu, dg, du, lddg, lddu, T, I);
  else glu_bwd_kernel<2><<<grid, 256, 0, st>>>(d, g, u, ldg, ldu, dg, du, lddg, lddu, T, I);
  return PM_LAUNCH_CHECK();
}
// row_loss (optional): per-row loss out. row_scale (optional): per-row gradient scale replacing *inv_n.
extern "C" int pm_ce_fwd_bwd(void* logits, long long ldl, const long long* labels, float* loss_sum, const float* inv_n,
                             float* row_loss, const float* row_scale, int n_rows, int V, long long ignore_index,
                             int write_grad, cudaStream_t st) {
  if (ldl % 8) return -1;
  ce_fwd_bwd_kernel<false><<<n_rows, 1024, 0, st>>>(static_cast<__nv_bfloat16*>(logits), ldl, labels, loss_sum, inv_n,
                                                    row_loss, row_scale, V, ignore_index, write_grad, 0.f, nullptr, 0.f, 0.f);
  return PM_LAUNCH_CHECK();
}
// Cross entropy plus the z term z_coef * logsumexp(logits)^2 per valid row: z_sum receives the sum of the squared
// normalisers, and the gradient written over the logits is that of (cross entropy + z_coef * z) summed over rows.
extern "C" int pm_ce_z_fwd_bwd(void* logits, long long ldl, const long long* labels, float* loss_sum, float* z_sum,
                               const float* inv_n, int n_rows, int V, long long ignore_index, int write_grad, float z_coef,
                               cudaStream_t st) {
  if (ldl % 8) return -1;
  ce_fwd_bwd_kernel<false><<<n_rows, 1024, 0, st>>>(static_cast<__nv_bfloat16*>(logits), ldl, labels, loss_sum, inv_n,
                                                    nullptr, nullptr, V, ignore_index, write_grad, z_coef, z_sum, 0.f, 0.f);
  return PM_LAUNCH_CHECK();
}
// The same with label smoothing (0 <= smooth < 1) and soft-capped logits (softcap > 0: cap * tanh(x / cap)).
extern "C" int pm_ce_opt_fwd_bwd(void* logits, long long ldl, const long long* labels, float* loss_sum, float* z_sum,
                                 const float* inv_n, int n_rows, int V, long long ignore_index, int write_grad,
                                 float z_coef, float smooth, float softcap, cudaStream_t st) {
  if (ldl % 8) return -1;
  if (smooth < 0.f || smooth >= 1.f || softcap < 0.f) return -2;
  ce_fwd_bwd_kernel<true><<<n_rows, 1024, 0, st>>>(static_cast<__nv_bfloat16*>(logits), ldl, labels, loss_sum, inv_n,
                                                   nullptr, nullptr, V, ignore_index, write_grad, z_coef, z_sum, smooth,
                                                   softcap);
  return PM_LAUNCH_CHECK();
}
extern "C" int pm_sumsq(const float* x, long long n, float* out, cudaStream_t st) {
  cudaError_t e = cudaMemsetAsync(out, 0, sizeof(float), st);
  if (e != cudaSuccess) return static_cast<int>(e);
  sumsq_kernel<<<grid_for(n / 4 + 1, 256, num_sms() * 4), 256, 0, st>>>(x, n, out);
  return PM_LAUNCH_CHECK();
}
extern "C" int pm_adamw_flat(float* p, const float* g, float* m, float* v, void* shadow, const float* lr_mult,
                             const float* wd, const float* gnorm_sq, const float* hp, long long n, float lr,
                             float beta1, float beta2, float eps, int step, float grad_scale, float max_norm,
                             cudaStream_t st) {
  if (n % 1024) return -1;
  AdamwArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps;
  // step <= 0 selects the variant without bias correction (moments used as they are)
  a.bc1 = step > 0 ? 1.f - powf(beta1, static_cast<float>(step)) : 1.f;
  a.bc2 = step > 0 ? 1.f - powf(beta2, static_cast<float>(step)) : 1.f;
  a.grad_scale = grad_scale; a.max_norm = max_norm;
  adamw_flat_kernel<<<grid_for(n / 4, 256, num_sms() * 8), 256, 0, st>>>(p, g, m, v, static_cast<__nv_bfloat16*>(shadow),
                                                                  lr_mult, wd, gnorm_sq, hp, n, a);
  return PM_LAUNCH_CHECK();
}
extern "C" int pm_attn_delta(const void* o, const void* dout, float* delta, int T, int H, cudaStream_t st) {
  const long long warps = static_cast<long long>(T) * H;
  attn_delta_kernel<<<static_cast<int>((warps + 7) / 8), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(dout), delta, T, H);
  return PM_LAUNCH_CHECK();
}
extern "C" int pm_f32_to_bf16(const float* in, void* out, long long n, cudaStream_t st) {
  f32_to_bf16_kernel<<<grid_for(n, 256), 256, 0, st>>>(in, static_cast<__nv_bfloat16*>(out), n);
  return PM_LAUNCH_CHECK();
}
extern "C" int pm_dequant_4bit(const void* data, const float* absmax, const void* absmax_q, float am_scale,
                               float am_offset, void* out, long long n, int block_size, int fp4, cudaStream_t st) {
  if (block_size % 8) return -1;
  dequant_4bit_kernel<<<grid_for(n / 8 + 1, 256), 256, 0, st>>>(
      static_cast<const uint8_t*>(data), absmax, static_cast<const uint8_t*>(absmax_q), am_scale, am_offset,
      static_cast<__nv_bfloat16*>(out), n, block_size, fp4);
  return PM_LAUNCH_CHECK();
}
