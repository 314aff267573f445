// Manifold-constrained hyper-connections: the residual stream is n parallel streams x [T, n, C]; every layer derives, per
// token, a read mixture H_pre [n], a write gain H_post [n] and a doubly stochastic stream-mixing matrix H_res [n, n] from the
// streams themselves (cf. the reference's eight kernels, crates/pmetal-mhc/src/kernels/metal_shaders.metal:39-521):
//
//   mappings     H~ = alpha_g * (RMSNorm(flatten(x)) . phi) + b          [T, n^2 + 2n], groups g = pre | post | res
//                H_pre = sigmoid(H~_pre), H_post = 2 sigmoid(H~_post), H_res = SinkhornKnopp(exp(H~_res))
//   pre          h_in[t]  = sum_n H_pre[t, n] x[t, n]
//   post + res   x_out[t, m] = sum_n H_res[t, m, n] x[t, n] + H_post[t, m] h_out[t]
//
// and their gradients. The streams are bandwidth: every kernel makes one pass over x with 16-byte loads, one CTA per
// token. The n x n algebra (n <= 8) lives in registers / shared memory; the Sinkhorn backward re-derives the iterates
// from the stored scaling vectors instead of keeping every intermediate matrix.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "host_util.cuh"
#include "pmetal_b200.h"

namespace pm {

constexpr int kMhcMaxN = 8;
constexpr int kMhcThreads = 256;
constexpr float kMhcEps = 1e-6f;        // RMS epsilon
constexpr float kSinkEps = 1e-8f;

__device__ __forceinline__ void mhc_load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ void mhc_store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 o;
  *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(f[0], f[1]);
  *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(f[2], f[3]);
  *reinterpret_cast<__nv_bfloat162*>(&o.z) = __floats2bfloat162_rn(f[4], f[5]);
  *reinterpret_cast<__nv_bfloat162*>(&o.w) = __floats2bfloat162_rn(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = o;
}
__device__ __forceinline__ float mhc_warp_sum(float v) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// sums `cnt` per-thread values across the CTA; results land in out[0..cnt) (shared). red: [8][cnt] scratch.
template <int CNT>
__device__ __forceinline__ void mhc_block_sum(float (&v)[CNT], float* red, float* out) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int j = 0; j < CNT; ++j) {
    const float s = mhc_warp_sum(v[j]);
    if (lane == 0) red[warp * CNT + j] = s;
  }
  __syncthreads();
  for (int j = threadIdx.x; j < CNT; j += blockDim.x) {
    float s = 0.f;
    for (int w = 0; w < kMhcThreads / 32; ++w) s += red[w * CNT + j];
    out[j] = s;
  }
  __syncthreads();
}

// Sinkhorn-Knopp on K = exp(logits) [n, n]: alternate row and column normalisation. M_t = diag(u_t) K diag(v_t); the
// scaling vectors after every half step are returned for the backward pass (us/vs: [iters][n]).
__device__ __forceinline__ void mhc_sinkhorn(const float* logits, int n, int iters, float* M, float* us, float* vs) {
  float u[kMhcMaxN], v[kMhcMaxN], K[kMhcMaxN * kMhcMaxN];
  float mx = -INFINITY;
  for (int i = 0; i < n * n; ++i) mx = fmaxf(mx, logits[i]);
  for (int i = 0; i < n * n; ++i) K[i] = __expf(logits[i] - mx);      // a common factor cancels in the first normalisation
  for (int i = 0; i < n; ++i) { u[i] = 1.f; v[i] = 1.f; }
  for (int t = 0; t < iters; ++t) {
    for (int i = 0; i < n; ++i) {
      float s = kSinkEps;
      for (int j = 0; j < n; ++j) s += u[i] * K[i * n + j] * v[j];
      u[i] /= s;
      if (us) us[t * n + i] = u[i];
    }
    for (int j = 0; j < n; ++j) {
      float s = kSinkEps;
      for (int i = 0; i < n; ++i) s += u[i] * K[i * n + j] * v[j];
      v[j] /= s;
      if (vs) vs[t * n + j] = v[j];
    }
  }
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < n; ++j) M[i * n + j] = u[i] * K[i * n + j] * v[j];
}

// ---------------------------------------------------------------------------------------------- mappings (forward)
// One CTA per token. The projection  raw[t, j] = sum_i x[t, i] phi[i, j]  is a [T, nC] x [nC, n^2 + 2n] GEMM that the
// caller runs on the tensor cores (fp32 output); this kernel adds what needs the whole row: sum x_i^2 for the RMS norm
// (which scales the sums, since the projection is linear), gating, bias and the three constraints. Without `raw` it
// forms the dot products itself (small inputs and tests).
template <int N>
__global__ void __launch_bounds__(kMhcThreads) mhc_mappings_kernel(const __nv_bfloat16* __restrict__ x,
                                                                   const float* __restrict__ phi,
                                                                   const float* __restrict__ raw, int ld_raw,
                                                                   const float* __restrict__ bias,
                                                                   const float* __restrict__ alpha, int C, int iters,
                                                                   float* __restrict__ h_tilde, float* __restrict__ rms_inv,
                                                                   float* __restrict__ h_pre, float* __restrict__ h_post,
                                                                   float* __restrict__ h_res) {
  constexpr int OUT = N * N + 2 * N;
  __shared__ float red[(kMhcThreads / 32) * (OUT + 1)];
  __shared__ float tot[OUT + 1];
  const long long t = blockIdx.x;
  const int nC = N * C;
  const __nv_bfloat16* xt = x + t * nC;
  if (raw) {
    float ss[1] = {0.f};
    for (int i0 = threadIdx.x * 8; i0 < nC; i0 += kMhcThreads * 8) {
      float f[8];
      mhc_load8(xt + i0, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss[0] += f[e] * f[e];
    }
    mhc_block_sum<1>(ss, red, tot + OUT);
    if (threadIdx.x < OUT) tot[threadIdx.x] = raw[t * ld_raw + threadIdx.x];
    __syncthreads();
  } else {
    float acc[OUT + 1];
#pragma unroll
    for (int j = 0; j <= OUT; ++j) acc[j] = 0.f;
    for (int i0 = threadIdx.x * 8; i0 < nC; i0 += kMhcThreads * 8) {
      float f[8];
      mhc_load8(xt + i0, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float* pr = phi + static_cast<long long>(i0 + e) * OUT;
        acc[OUT] += f[e] * f[e];
#pragma unroll
        for (int j = 0; j < OUT; ++j) acc[j] += f[e] * __ldg(pr + j);
      }
    }
    mhc_block_sum<OUT + 1>(acc, red, tot);
  }
  if (threadIdx.x == 0) {
    const float ri = rsqrtf(tot[OUT] / nC + kMhcEps);
    rms_inv[t] = ri;
    float ht[OUT];
    for (int j = 0; j < OUT; ++j) {
      const int g = j < N ? 0 : (j < 2 * N ? 1 : 2);
      ht[j] = alpha[g] * ri * tot[j] + bias[j];
      h_tilde[t * OUT + j] = ht[j];
    }
    for (int j = 0; j < N; ++j) {
      h_pre[t * N + j] = 1.f / (1.f + __expf(-ht[j]));
      h_post[t * N + j] = 2.f / (1.f + __expf(-ht[N + j]));
    }
    float M[kMhcMaxN * kMhcMaxN];
    mhc_sinkhorn(ht + 2 * N, N, iters, M, nullptr, nullptr);
    for (int j = 0; j < N * N; ++j) h_res[t * N * N + j] = M[j];
  }
}

// ---------------------------------------------------------------------------------------------- stream mixing (forward)
template <int N>
__global__ void __launch_bounds__(kMhcThreads) mhc_pre_kernel(const __nv_bfloat16* __restrict__ x,
                                                              const float* __restrict__ h_pre, int C,
                                                              __nv_bfloat16* __restrict__ h_in) {
  const long long t = blockIdx.x;
  float w[N];
#pragma unroll
  for (int n = 0; n < N; ++n) w[n] = h_pre[t * N + n];
  for (int c = threadIdx.x * 8; c < C; c += kMhcThreads * 8) {
    float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int n = 0; n < N; ++n) {
      float f[8];
      mhc_load8(x + (t * N + n) * C + c, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] += w[n] * f[e];
    }
    mhc_store8(h_in + t * C + c, o);
  }
}

template <int N>
__global__ void __launch_bounds__(kMhcThreads) mhc_post_res_kernel(const __nv_bfloat16* __restrict__ x,
                                                                   const __nv_bfloat16* __restrict__ h_out,
                                                                   const float* __restrict__ h_res,
                                                                   const float* __restrict__ h_post, int C,
                                                                   __nv_bfloat16* __restrict__ x_out) {
  __shared__ float sr[N * N], sp[N];
  const long long t = blockIdx.x;
  if (threadIdx.x < N * N) sr[threadIdx.x] = h_res[t * N * N + threadIdx.x];
  if (threadIdx.x < N) sp[threadIdx.x] = h_post[t * N + threadIdx.x];
  __syncthreads();
  for (int c = threadIdx.x * 8; c < C; c += kMhcThreads * 8) {
    float xs[N][8], ho[8];
#pragma unroll
    for (int n = 0; n < N; ++n) mhc_load8(x + (t * N + n) * C + c, xs[n]);
    mhc_load8(h_out + t * C + c, ho);
#pragma unroll
    for (int m = 0; m < N; ++m) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = sp[m] * ho[e];
#pragma unroll
      for (int n = 0; n < N; ++n)
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] += sr[m * N + n] * xs[n][e];
      mhc_store8(x_out + (t * N + m) * C + c, o);
    }
  }
}

// ---------------------------------------------------------------------------------------------- stream mixing (backward)
// Either half may be absent (null dh_in: only the post / res part; null dx_out: only the pre part), since autograd reaches
// the two applications at different times.
// dx[t, n] = H_pre[t, n] dh_in[t] + sum_m H_res[t, m, n] dx_out[t, m];  dh_out[t] = sum_m H_post[t, m] dx_out[t, m]
// dH_pre[t, n] = <x[t, n], dh_in[t]>;  dH_post[t, m] = <dx_out[t, m], h_out[t]>;  dH_res[t, m, n] = <dx_out[t, m], x[t, n]>
template <int N>
__global__ void __launch_bounds__(kMhcThreads) mhc_mix_bwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                                  const __nv_bfloat16* __restrict__ h_out,
                                                                  const __nv_bfloat16* __restrict__ dh_in,
                                                                  const __nv_bfloat16* __restrict__ dx_out,
                                                                  const float* __restrict__ h_pre,
                                                                  const float* __restrict__ h_post,
                                                                  const float* __restrict__ h_res, int C,
                                                                  __nv_bfloat16* __restrict__ dx,
                                                                  __nv_bfloat16* __restrict__ dh_out,
                                                                  float* __restrict__ d_pre, float* __restrict__ d_post,
                                                                  float* __restrict__ d_res) {
  constexpr int CNT = N * N + 2 * N;
  __shared__ float sr[N * N], sp[N], sq[N];
  __shared__ float red[(kMhcThreads / 32) * CNT];
  __shared__ float tot[CNT];
  const long long t = blockIdx.x;
  if (threadIdx.x < N * N) sr[threadIdx.x] = h_res[t * N * N + threadIdx.x];
  if (threadIdx.x < N) { sp[threadIdx.x] = h_post[t * N + threadIdx.x]; sq[threadIdx.x] = h_pre[t * N + threadIdx.x]; }
  __syncthreads();
  float acc[CNT];          // [pre n | post m | res m*N + n]
#pragma unroll
  for (int j = 0; j < CNT; ++j) acc[j] = 0.f;
  for (int c = threadIdx.x * 8; c < C; c += kMhcThreads * 8) {
    float xs[N][8], go[N][8], ho[8], gi[8];
#pragma unroll
    for (int n = 0; n < N; ++n) {
      mhc_load8(x + (t * N + n) * C + c, xs[n]);
      if (dx_out) {
        mhc_load8(dx_out + (t * N + n) * C + c, go[n]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) go[n][e] = 0.f;
      }
    }
    if (dx_out) {
      mhc_load8(h_out + t * C + c, ho);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) ho[e] = 0.f;
    }
    if (dh_in) {
      mhc_load8(dh_in + t * C + c, gi);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) gi[e] = 0.f;
    }
    float dho[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int m = 0; m < N; ++m)
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        dho[e] += sp[m] * go[m][e];
        acc[N + m] += go[m][e] * ho[e];
      }
    if (dx_out) mhc_store8(dh_out + t * C + c, dho);
#pragma unroll
    for (int n = 0; n < N; ++n) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        o[e] = sq[n] * gi[e];
        acc[n] += xs[n][e] * gi[e];
      }
#pragma unroll
      for (int m = 0; m < N; ++m)
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          o[e] += sr[m * N + n] * go[m][e];
          acc[2 * N + m * N + n] += go[m][e] * xs[n][e];
        }
      mhc_store8(dx + (t * N + n) * C + c, o);
    }
  }
  mhc_block_sum<CNT>(acc, red, tot);
  if (threadIdx.x < N) {
    if (dh_in) d_pre[t * N + threadIdx.x] = tot[threadIdx.x];
    if (dx_out) d_post[t * N + threadIdx.x] = tot[N + threadIdx.x];
  }
  if (dx_out && threadIdx.x < N * N) d_res[t * N * N + threadIdx.x] = tot[2 * N + threadIdx.x];
}

// ---------------------------------------------------------------------------------------------- constraints (backward)
// One thread per token: gradients of (H_pre, H_post, H_res) -> gradient of H~. The Sinkhorn iterates are rebuilt from the
// scaling vectors, which are recomputed here and kept in local memory ([iters][n] each).
constexpr int kMhcMaxIters = 32;
__global__ void mhc_constraints_bwd_kernel(const float* __restrict__ h_tilde, const float* __restrict__ d_pre,
                                           const float* __restrict__ d_post, const float* __restrict__ d_res, int T, int n,
                                           int iters, float* __restrict__ d_tilde) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const int out = n * n + 2 * n;
  const float* ht = h_tilde + static_cast<long long>(t) * out;
  float* dt = d_tilde + static_cast<long long>(t) * out;
  for (int j = 0; j < n; ++j) {
    const float s = 1.f / (1.f + __expf(-ht[j]));
    dt[j] = d_pre[static_cast<long long>(t) * n + j] * s * (1.f - s);
    const float s2 = 1.f / (1.f + __expf(-ht[n + j]));
    dt[n + j] = d_post[static_cast<long long>(t) * n + j] * 2.f * s2 * (1.f - s2);
  }
  float us[kMhcMaxIters * kMhcMaxN], vs[kMhcMaxIters * kMhcMaxN], M[kMhcMaxN * kMhcMaxN], K[kMhcMaxN * kMhcMaxN];
  mhc_sinkhorn(ht + 2 * n, n, iters, M, us, vs);
  float mx = -INFINITY;
  for (int i = 0; i < n * n; ++i) mx = fmaxf(mx, ht[2 * n + i]);
  for (int i = 0; i < n * n; ++i) K[i] = __expf(ht[2 * n + i] - mx);
  // g holds dL/dM of the current iterate, starting from the output
  float g[kMhcMaxN * kMhcMaxN];
  for (int i = 0; i < n * n; ++i) g[i] = d_res[static_cast<long long>(t) * n * n + i];
  for (int it = iters - 1; it >= 0; --it) {
    // column step: M'' = M' / colsum(M'), M'' = u_it K v_it (after the step);  dM' = (dM'' - sum_i dM''_ij M''_ij) / colsum_j
    for (int j = 0; j < n; ++j) {
      float dot = 0.f, csum_inv;
      // colsum of M' = 1 / (v_after / v_before): v_before is the previous iteration's v (1 at the start)
      const float v_after = vs[it * n + j], v_before = it > 0 ? vs[(it - 1) * n + j] : 1.f;
      csum_inv = v_after / v_before;
      for (int i = 0; i < n; ++i) dot += g[i * n + j] * (us[it * n + i] * K[i * n + j] * v_after);
      for (int i = 0; i < n; ++i) g[i * n + j] = (g[i * n + j] - dot) * csum_inv;
    }
    // row step: M' = M / rowsum(M), M' = u_it K v_{it-1}
    for (int i = 0; i < n; ++i) {
      float dot = 0.f;
      const float u_after = us[it * n + i], u_before = it > 0 ? us[(it - 1) * n + i] : 1.f;
      const float rsum_inv = u_after / u_before;
      for (int j = 0; j < n; ++j) {
        const float v_prev = it > 0 ? vs[(it - 1) * n + j] : 1.f;
        dot += g[i * n + j] * (u_after * K[i * n + j] * v_prev);
      }
      for (int j = 0; j < n; ++j) g[i * n + j] = (g[i * n + j] - dot) * rsum_inv;
    }
  }
  // g is now dL/dK (K scaled by exp(-mx), which the normalisations cancel): dL/dlogit = g * K
  for (int i = 0; i < n * n; ++i) dt[2 * n + i] = g[i] * K[i];
}

// ---------------------------------------------------------------------------------------------- monitoring, expand, collapse
// gains[0] = max over tokens and rows of sum_j |H_res[t, i, j]| (forward gain), gains[1] = the same over columns
__global__ void mhc_amax_gain_kernel(const float* __restrict__ h_res, int T, int n, float* __restrict__ gains) {
  float fr = 0.f, fc = 0.f;
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < T; t += gridDim.x * blockDim.x) {
    const float* m = h_res + static_cast<long long>(t) * n * n;
    for (int i = 0; i < n; ++i) {
      float r = 0.f, c = 0.f;
      for (int j = 0; j < n; ++j) { r += fabsf(m[i * n + j]); c += fabsf(m[j * n + i]); }
      fr = fmaxf(fr, r);
      fc = fmaxf(fc, c);
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    fr = fmaxf(fr, __shfl_xor_sync(0xffffffffu, fr, o));
    fc = fmaxf(fc, __shfl_xor_sync(0xffffffffu, fc, o));
  }
  if ((threadIdx.x & 31) == 0) {       // non-negative floats order like their bit patterns
    atomicMax(reinterpret_cast<int*>(gains), __float_as_int(fr));
    atomicMax(reinterpret_cast<int*>(gains) + 1, __float_as_int(fc));
  }
}

__global__ void mhc_expand_kernel(const __nv_bfloat16* __restrict__ x, int n, int C, __nv_bfloat16* __restrict__ xs,
                                  long long total8) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long per = C / 8;
    const long long t = i / (n * per), c = i % per;
    reinterpret_cast<uint4*>(xs)[i] = reinterpret_cast<const uint4*>(x)[t * per + c];
  }
}

__global__ void mhc_collapse_kernel(const __nv_bfloat16* __restrict__ xs, int n, int C, __nv_bfloat16* __restrict__ x,
                                    long long total8) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long per = C / 8;
    const long long t = i / per, c = i % per;
    float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < n; ++s) {
      float f[8];
      mhc_load8(xs + ((t * n + s) * per + c) * 8, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] += f[e];
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] /= n;
    mhc_store8(x + i * 8, o);
  }
}

}  // namespace pm

using namespace pm;

#define MHC_DISPATCH(N_, CALL)            \
  switch (N_) {                           \
    case 2: { constexpr int NN = 2; CALL; break; } \
    case 4: { constexpr int NN = 4; CALL; break; } \
    case 8: { constexpr int NN = 8; CALL; break; } \
    default: return -1;                   \
  }

// x [T, n, C] bf16; either phi [n C, n^2 + 2n] fp32 (dot products formed here) or raw [T, ld_raw] fp32 = x . phi computed by
// the caller; bias [n^2 + 2n], alpha [3]; n in {2, 4, 8}, C % 8 == 0, iters <= 32.
extern "C" int pm_mhc_mappings(const void* x, const float* phi, const float* raw, int ld_raw, const float* bias,
                               const float* alpha, int T, int n, int C, int iters, float* h_tilde, float* rms_inv,
                               float* h_pre, float* h_post, float* h_res, cudaStream_t st) {
  if (T <= 0 || (C % 8) || iters < 0 || iters > kMhcMaxIters || (!phi && !raw)) return -2;
  MHC_DISPATCH(n, (mhc_mappings_kernel<NN><<<T, kMhcThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(x), phi, raw,
                                                                      ld_raw, bias, alpha, C, iters, h_tilde, rms_inv,
                                                                      h_pre, h_post, h_res)));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int pm_mhc_pre(const void* x, const float* h_pre, int T, int n, int C, void* h_in, cudaStream_t st) {
  if (T <= 0 || (C % 8)) return -2;
  MHC_DISPATCH(n, (mhc_pre_kernel<NN><<<T, kMhcThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(x), h_pre, C,
                                                                 static_cast<__nv_bfloat16*>(h_in))));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int pm_mhc_post_res(const void* x, const void* h_out, const float* h_res, const float* h_post, int T, int n,
                               int C, void* x_out, cudaStream_t st) {
  if (T <= 0 || (C % 8)) return -2;
  MHC_DISPATCH(n, (mhc_post_res_kernel<NN><<<T, kMhcThreads, 0, st>>>(
                      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(h_out), h_res, h_post, C,
                      static_cast<__nv_bfloat16*>(x_out))));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int pm_mhc_mix_bwd(const void* x, const void* h_out, const void* dh_in, const void* dx_out, const float* h_pre,
                              const float* h_post, const float* h_res, int T, int n, int C, void* dx, void* dh_out,
                              float* d_pre, float* d_post, float* d_res, cudaStream_t st) {
  if (T <= 0 || (C % 8)) return -2;
  MHC_DISPATCH(n, (mhc_mix_bwd_kernel<NN><<<T, kMhcThreads, 0, st>>>(
                      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(h_out),
                      static_cast<const __nv_bfloat16*>(dh_in), static_cast<const __nv_bfloat16*>(dx_out), h_pre, h_post,
                      h_res, C, static_cast<__nv_bfloat16*>(dx), static_cast<__nv_bfloat16*>(dh_out), d_pre, d_post,
                      d_res)));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int pm_mhc_constraints_bwd(const float* h_tilde, const float* d_pre, const float* d_post, const float* d_res,
                                      int T, int n, int iters, float* d_tilde, cudaStream_t st) {
  if (T <= 0 || n < 1 || n > kMhcMaxN || iters < 0 || iters > kMhcMaxIters) return -2;
  mhc_constraints_bwd_kernel<<<(T + 63) / 64, 64, 0, st>>>(h_tilde, d_pre, d_post, d_res, T, n, iters, d_tilde);
  return static_cast<int>(cudaGetLastError());
}

// gains [2] fp32, cleared here: largest absolute row sum and column sum of H_res over all tokens
extern "C" int pm_mhc_amax_gain(const float* h_res, int T, int n, float* gains, cudaStream_t st) {
  if (T <= 0 || n < 1 || n > kMhcMaxN) return -2;
  cudaError_t e = cudaMemsetAsync(gains, 0, 2 * sizeof(float), st);
  if (e != cudaSuccess) return static_cast<int>(e);
  int grid = (T + 255) / 256;
  if (grid > 1024) grid = 1024;
  mhc_amax_gain_kernel<<<grid, 256, 0, st>>>(h_res, T, n, gains);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int pm_mhc_expand(const void* x, int T, int n, int C, void* xs, cudaStream_t st) {
  if (T <= 0 || (C % 8) || n < 1) return -2;
  const long long total8 = static_cast<long long>(T) * n * (C / 8);
  long long grid = (total8 + 255) / 256;
  if (grid > 65535) grid = 65535;
  mhc_expand_kernel<<<static_cast<int>(grid), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), n, C,
                                                           static_cast<__nv_bfloat16*>(xs), total8);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int pm_mhc_collapse(const void* xs, int T, int n, int C, void* x, cudaStream_t st) {
  if (T <= 0 || (C % 8) || n < 1) return -2;
  const long long total8 = static_cast<long long>(T) * (C / 8);
  long long grid = (total8 + 255) / 256;
  if (grid > 65535) grid = 65535;
  mhc_collapse_kernel<<<static_cast<int>(grid), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(xs), n, C,
                                                             static_cast<__nv_bfloat16*>(x), total8);
  return static_cast<int>(cudaGetLastError());
}
