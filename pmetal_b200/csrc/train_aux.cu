// Distillation losses over a logits chunk, and fused model-merge kernels.
//
// Distillation (reference: crates/pmetal-metal/src/kernels/metal/fused_distill.metal:91-1286 —
// fused_kl_divergence_forward_backward and friends; loss definitions in crates/pmetal-distill/src/losses/*.rs):
// one CTA per token row computes, with online softmax over the vocabulary and temperature T, the loss between the
// teacher and student distributions and overwrites the student logits with d loss / d student_logit * row_scale.
//   kind 0: forward KL   sum p_t (log p_t - log p_s)          grad (p_s - p_t) / T
//   kind 1: reverse KL   sum p_s (log p_s - log p_t)          grad p_s ((log p_s - log p_t) - L) / T
//   kind 2: JS(beta)     beta KL(p_t||m) + (1-beta) KL(p_s||m), m = beta p_t + (1-beta) p_s
//                                                             grad (1-beta) p_s (log(p_s/m) - sum p_s log(p_s/m)) / T
//   kind 3: soft CE      -sum p_t log p_s                     grad (p_s - p_t) / T
//   kind 4: total variation 0.5 sum |p_t - p_s|               grad 0.5 p_s (sgn_i - sum p_s sgn) / T, sgn = sign(p_s - p_t)
//
// Merge (reference: crates/pmetal-metal/src/kernels/metal/fused_merge.metal:59-461 — task vectors, sparsify, sign
// consensus, TIES, DARE, linear, SLERP): one pass over up to 8 models forms task vectors, applies per-model
// magnitude thresholds (TIES trimming) or a random keep mask with 1/density rescale (DARE), combines by weighted
// sum or weighted sign consensus, and adds the result back on the base.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include "host_util.cuh"
#include "pmetal_b200.h"

namespace pm {

constexpr int kKdThreads = 512;

__device__ __forceinline__ float kd_block_sum(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  v = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) red[32] = v;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float kd_block_max(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  v = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : -INFINITY;
  if (threadIdx.x < 32) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (threadIdx.x == 0) red[32] = v;
  }
  __syncthreads();
  return red[32];
}

// student: [rows, ld] bf16 (overwritten with the gradient when write_grad), teacher: [rows, ldt] bf16.
// row_scale[r] multiplies the gradient of row r (0 for masked rows: their loss is 0 too); row_loss[r] gets the loss.
__global__ void __launch_bounds__(kKdThreads)
kd_fwd_bwd_kernel(__nv_bfloat16* __restrict__ student, long long ld, const __nv_bfloat16* __restrict__ teacher,
                  long long ldt, int V, float inv_temp, int kind, float beta, const float* __restrict__ row_scale,
                  float* __restrict__ row_loss, float* __restrict__ loss_sum, int write_grad) {
  __shared__ float red[64];
  const int r = blockIdx.x;
  __nv_bfloat16* s = student + static_cast<long long>(r) * ld;
  const __nv_bfloat16* t = teacher + static_cast<long long>(r) * ldt;
  const float scale = row_scale ? row_scale[r] : 1.f;
  if (scale == 0.f) {
    if (write_grad)
      for (int i = threadIdx.x; i < V; i += blockDim.x) s[i] = __float2bfloat16(0.f);
    if (row_loss && threadIdx.x == 0) row_loss[r] = 0.f;
    return;
  }
  float ms = -INFINITY, mt = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    ms = fmaxf(ms, __bfloat162float(s[i]) * inv_temp);
    mt = fmaxf(mt, __bfloat162float(t[i]) * inv_temp);
  }
  ms = kd_block_max(ms, red);
  mt = kd_block_max(mt, red);
  float zs = 0.f, zt = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    zs += __expf(__bfloat162float(s[i]) * inv_temp - ms);
    zt += __expf(__bfloat162float(t[i]) * inv_temp - mt);
  }
  zs = kd_block_sum(zs, red);
  zt = kd_block_sum(zt, red);
  const float lzs = ms + __logf(zs), lzt = mt + __logf(zt);
  // loss and, for the kinds that need it, the inner expectation under p_s
  float loss = 0.f, inner = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float ls = __bfloat162float(s[i]) * inv_temp - lzs, lt = __bfloat162float(t[i]) * inv_temp - lzt;
    const float ps = __expf(ls), pt = __expf(lt);
    if (kind == 0) {
      loss += pt * (lt - ls);
    } else if (kind == 1) {
      loss += ps * (ls - lt);
    } else if (kind == 2) {
      const float m = beta * pt + (1.f - beta) * ps;
      const float lm = __logf(fmaxf(m, 1e-30f));
      loss += beta * pt * (lt - lm) + (1.f - beta) * ps * (ls - lm);
      inner += ps * (ls - lm);
    } else if (kind == 3) {
      loss += -pt * ls;
    } else {
      loss += 0.5f * fabsf(pt - ps);
      inner += ps * ((ps > pt) ? 1.f : ((ps < pt) ? -1.f : 0.f));
    }
  }
  loss = kd_block_sum(loss, red);
  if (kind == 2 || kind == 4) inner = kd_block_sum(inner, red);
  if (threadIdx.x == 0) {
    if (row_loss) row_loss[r] = loss;
    if (loss_sum) atomicAdd(loss_sum, loss * scale);
  }
  if (!write_grad) return;
  const float gs = scale * inv_temp;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float ls = __bfloat162float(s[i]) * inv_temp - lzs, lt = __bfloat162float(t[i]) * inv_temp - lzt;
    const float ps = __expf(ls), pt = __expf(lt);
    float g;
    if (kind == 0 || kind == 3) {
      g = ps - pt;
    } else if (kind == 1) {
      g = ps * ((ls - lt) - loss);
    } else if (kind == 2) {
      const float m = beta * pt + (1.f - beta) * ps;
      g = (1.f - beta) * ps * ((ls - __logf(fmaxf(m, 1e-30f))) - inner);
    } else {
      const float sg = (ps > pt) ? 1.f : ((ps < pt) ? -1.f : 0.f);
      g = 0.5f * ps * (sg - inner);
    }
    s[i] = __float2bfloat16(g * gs);
  }
}

// ------------------------------------------------------------------------------------------------ merge
struct MergeArgs {
  const void* model[8];
  const void* base;          // may be null (then no task vectors: plain weighted combination)
  float weight[8];
  float threshold[8];        // |tau| below this is dropped (0 keeps everything)
  float density[8];          // DARE keep probability (>= 1 keeps everything)
  int n_models;
  int in_bf16;               // inputs bf16 (1) or fp32 (0)
  int out_bf16;
  int consensus;             // weighted sign consensus instead of a plain weighted sum
  int rescale;               // DARE: divide kept entries by the density
  float lam;
  unsigned long long seed;
  void* out;
  long long n;
};

__device__ __forceinline__ float merge_load(const void* p, long long i, int bf16) {
  return bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]) : static_cast<const float*>(p)[i];
}
__device__ __forceinline__ uint64_t merge_mix(uint64_t z) {
  z += 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

__global__ void merge_fused_kernel(const MergeArgs a) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < a.n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float b = a.base ? merge_load(a.base, i, a.in_bf16) : 0.f;
    float tv[8];
    float votes = 0.f;
#pragma unroll
    for (int m = 0; m < 8; ++m) {
      if (m >= a.n_models) { tv[m] = 0.f; continue; }
      float v = merge_load(a.model[m], i, a.in_bf16) - b;
      if (a.threshold[m] > 0.f && fabsf(v) < a.threshold[m]) v = 0.f;
      if (a.density[m] < 1.f) {
        const uint64_t h = merge_mix(merge_mix(a.seed + static_cast<uint64_t>(m) * 0x632be59bd9b4e019ull) + static_cast<uint64_t>(i));
        const float u = static_cast<float>(h >> 40) * (1.0f / 16777216.0f);
        v = (u < a.density[m]) ? (a.rescale ? v / a.density[m] : v) : 0.f;
      }
      tv[m] = v;
      votes += a.weight[m] * ((v > 0.f) ? 1.f : ((v < 0.f) ? -1.f : 0.f));
    }
    float acc = 0.f;
#pragma unroll
    for (int m = 0; m < 8; ++m) {
      if (m >= a.n_models) continue;
      if (!a.consensus || a.n_models == 1 || tv[m] * votes > 0.f) acc += a.weight[m] * tv[m];
    }
    const float out = b + a.lam * acc;
    if (a.out_bf16) static_cast<__nv_bfloat16*>(a.out)[i] = __float2bfloat16(out);
    else static_cast<float*>(a.out)[i] = out;
  }
}

// dot(a, b), |a|^2, |b|^2 in one pass (SLERP angle); out[3] accumulated atomically
__global__ void dot_norms_kernel(const void* __restrict__ a, const void* __restrict__ b, int bf16, long long n,
                                 float* __restrict__ out) {
  float d = 0.f, na = 0.f, nb = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float x = merge_load(a, i, bf16), y = merge_load(b, i, bf16);
    d += x * y;
    na += x * x;
    nb += y * y;
  }
  for (int o = 16; o > 0; o >>= 1) {
    d += __shfl_xor_sync(0xffffffffu, d, o);
    na += __shfl_xor_sync(0xffffffffu, na, o);
    nb += __shfl_xor_sync(0xffffffffu, nb, o);
  }
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(out, d);
    atomicAdd(out + 1, na);
    atomicAdd(out + 2, nb);
  }
}

}  // namespace pm

using namespace pm;

extern "C" int pm_kd_fwd_bwd(void* student, long long ld, const void* teacher, long long ldt, int rows, int V,
                             float temperature, int kind, float beta, const float* row_scale, float* row_loss,
                             float* loss_sum, int write_grad, cudaStream_t st) {
  if (rows <= 0 || V <= 0 || !(temperature > 0.f) || kind < 0 || kind > 4) return -1;
  kd_fwd_bwd_kernel<<<rows, kKdThreads, 0, st>>>(static_cast<__nv_bfloat16*>(student), ld,
                                                 static_cast<const __nv_bfloat16*>(teacher), ldt, V, 1.f / temperature,
                                                 kind, beta, row_scale, row_loss, loss_sum, write_grad);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int pm_merge_fused(const void* const* models, const void* base, const float* weights,
                              const float* thresholds, const float* densities, int n_models, int in_bf16, int out_bf16,
                              int consensus, int rescale, float lam, unsigned long long seed, void* out, long long n,
                              cudaStream_t st) {
  if (n_models < 1 || n_models > 8) return -1;
  if (n <= 0) return 0;
  MergeArgs a{};
  for (int m = 0; m < n_models; ++m) {
    a.model[m] = models[m];
    a.weight[m] = weights[m];
    a.threshold[m] = thresholds ? thresholds[m] : 0.f;
    a.density[m] = densities ? densities[m] : 1.f;
  }
  a.base = base; a.n_models = n_models; a.in_bf16 = in_bf16; a.out_bf16 = out_bf16; a.consensus = consensus;
  a.rescale = rescale; a.lam = lam; a.seed = seed; a.out = out; a.n = n;
  long long g = (n + 255) / 256;
  if (g > num_sms() * 16) g = num_sms() * 16;
  merge_fused_kernel<<<static_cast<unsigned>(g), 256, 0, st>>>(a);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int pm_dot_norms(const void* a, const void* b, int bf16, long long n, float* out3, cudaStream_t st) {
  if (n <= 0) return 0;
  cudaError_t e = cudaMemsetAsync(out3, 0, 3 * sizeof(float), st);
  if (e != cudaSuccess) return static_cast<int>(e);
  long long g = (n + 255) / 256;
  if (g > num_sms() * 8) g = num_sms() * 8;
  dot_norms_kernel<<<static_cast<unsigned>(g), 256, 0, st>>>(a, b, bf16, n, out3);
  return static_cast<int>(cudaGetLastError());
}
