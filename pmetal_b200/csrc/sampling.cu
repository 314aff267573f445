// On-device token sampling and speculative verification.
//
//   sample_kernel        one CTA per row of logits: penalties (from a per-row token-count table), then top-k, top-p
//                        (nucleus, applied to the top-k survivors) and min-p on the temperature-1 distribution, then an
//                        exact categorical draw from softmax(logit / T) over the survivors by the Gumbel-max trick;
//                        temperature 0 means greedy. Also returns the log-probability of the drawn token under the
//                        filtered, tempered distribution it was drawn from.
//   spec_verify_kernel   one CTA per sequence: walks the K drafted tokens, accepts token i with probability
//                        min(1, p_target/p_draft) (greedy mode: iff it equals the target argmax), on the first
//                        rejection draws from normalize(max(0, p_target - p_draft)), and draws the bonus token from
//                        the last target row when everything was accepted.
//
// Thresholds for top-k / top-p are found exactly with a 4-pass radix select over order-preserving float keys
// (256-bin histograms in shared memory; counts for top-k, probability mass for top-p), so no sort of the
// vocabulary is ever materialised.
//
// Semantics follow the reference sampler (crates/pmetal-models/src/generation.rs:813-1120: repetition, frequency
// and presence penalties, temperature, top-k, top-p, min-p) and verifier
// (crates/pmetal-mlx/src/speculative.rs:343-620: verify_greedy, verify_logits); its Metal kernels only cover
// argmax and small-vocabulary sampling (crates/pmetal-metal/src/kernels/metal/fused_sampler.metal).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include "host_util.cuh"
#include "pmetal_b200.h"

namespace pm {

constexpr int kSampThreads = 1024;

struct SampleParams {
  const void* logits;        // [rows, ld] fp32 or bf16
  int is_bf16;
  long long ld;
  int vocab;
  const int* counts;         // [*, vocab] occurrences of each token so far (may be null)
  const int* count_rows;     // [rows] row of `counts` that belongs to each logits row (null: the same row index)
  const float* temperature;  // per row
  const int* top_k;          // per row, <= 0 disables
  const float* top_p;        // per row, >= 1 disables
  const float* min_p;        // per row, <= 0 disables
  const float* rep_pen;      // per row, 1 disables (may be null together with freq/pres)
  const float* freq_pen;
  const float* pres_pen;
  const unsigned long long* seeds;   // per row
  unsigned long long step;           // mixed into the random stream
  int* out_token;            // [rows]
  float* out_logprob;        // [rows] (may be null)
};

__device__ __forceinline__ uint32_t order_key(float f) {   // larger float -> larger key
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}
// uniform in (0, 1) from (seed, stream, index)
__device__ __forceinline__ float uniform01(uint64_t seed, uint64_t stream, uint64_t idx) {
  const uint64_t h = mix64(mix64(seed ^ (stream * 0xd1342543de82ef95ull)) + idx);
  return (static_cast<float>(h >> 40) + 0.5f) * (1.0f / 16777216.0f);
}
__device__ __forceinline__ float gumbel(float u) { return -__logf(-__logf(u)); }

struct RowView {
  const void* base;
  int is_bf16;
  const int* counts;
  float inv_t, rep, freq, pres;
  bool pen;
  __device__ __forceinline__ float at(int i) const {
    float x = is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(base)[i]) : static_cast<const float*>(base)[i];
    if (pen) {
      const int c = counts[i];
      if (c > 0) {
        x = x > 0.f ? x / rep : x * rep;
        x -= freq * static_cast<float>(c) + pres;
      }
    }
    return x;
  }
};

// block-wide reductions over kSampThreads threads; `red` has 64 floats of shared scratch
__device__ __forceinline__ float block_max(float v, float* red) {
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
__device__ __forceinline__ float block_sum(float v, float* red) {
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
// argmax of (value, index) pairs; ties go to the smaller index
__device__ __forceinline__ void block_argmax(float& v, int& idx, float* redv, int* redi) {
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) { redv[threadIdx.x >> 5] = v; redi[threadIdx.x >> 5] = idx; }
  __syncthreads();
  if (threadIdx.x < 32) {
    v = (threadIdx.x < (blockDim.x >> 5)) ? redv[threadIdx.x] : -INFINITY;
    idx = (threadIdx.x < (blockDim.x >> 5)) ? redi[threadIdx.x] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    if (threadIdx.x == 0) { redv[32] = v; redi[32] = idx; }
  }
  __syncthreads();
  v = redv[32];
  idx = redi[32];
}

// Radix select. Finds the key K such that the weight of {x : key(x) >= K} first reaches `target` when keys are
// taken from the largest down. kMass = false: weight 1 per element (k-th largest); kMass = true: weight
// exp(x - m). Elements with key < floor_key are ignored. Returns the key; *above gets the weight strictly above it.
template <bool kMass>
__device__ uint32_t radix_threshold(const RowView& row, int vocab, float m, float target, uint32_t floor_key,
                                    float* hist /*256*/, float* bcast /*4*/, float* above_out) {
  uint32_t prefix = 0, mask = 0;
  float above = 0.f;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0.f;
    __syncthreads();
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float x = row.at(i);
      const uint32_t k = order_key(x);
      if (k >= floor_key && (k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255], kMass ? __expf(x - m) : 1.f);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float acc = above;
      int b = 255;
      for (; b > 0; --b) {
        if (acc + hist[b] >= target) break;
        acc += hist[b];
      }
      bcast[0] = acc;
      bcast[1] = __int_as_float(b);
    }
    __syncthreads();
    above = bcast[0];
    prefix |= static_cast<uint32_t>(__float_as_int(bcast[1])) << shift;
    mask |= 0xffu << shift;
    __syncthreads();
  }
  *above_out = above;
  return prefix;
}

__global__ void __launch_bounds__(kSampThreads) sample_kernel(const SampleParams p) {
  __shared__ float hist[256];
  __shared__ float red[64];
  __shared__ int redi[64];
  __shared__ float bcast[4];
  const int r = blockIdx.x;
  RowView row;
  row.base = static_cast<const char*>(p.logits) + static_cast<long long>(r) * p.ld * (p.is_bf16 ? 2 : 4);
  row.is_bf16 = p.is_bf16;
  row.counts = p.counts ? p.counts + static_cast<long long>(p.count_rows ? p.count_rows[r] : r) * p.vocab : nullptr;
  const float temp = p.temperature[r];
  const bool greedy = !(temp > 0.f);
  row.inv_t = greedy ? 1.f : 1.f / temp;
  row.rep = p.rep_pen ? p.rep_pen[r] : 1.f;
  row.freq = p.freq_pen ? p.freq_pen[r] : 0.f;
  row.pres = p.pres_pen ? p.pres_pen[r] : 0.f;
  row.pen = row.counts && (row.rep != 1.f || row.freq != 0.f || row.pres != 0.f);

  // pass 1: maximum and its index (this is the greedy answer)
  float mv = -INFINITY;
  int mi = 0x7fffffff;
  for (int i = threadIdx.x; i < p.vocab; i += blockDim.x) {
    const float x = row.at(i);
    if (x > mv) { mv = x; mi = i; }
  }
  block_argmax(mv, mi, red, redi);
  const float m = mv;
  // pass 2: partition function
  float z = 0.f;
  for (int i = threadIdx.x; i < p.vocab; i += blockDim.x) z += __expf(row.at(i) - m);
  z = block_sum(z, red);
  if (greedy) {
    if (threadIdx.x == 0) {
      p.out_token[r] = mi;
      if (p.out_logprob) p.out_logprob[r] = -__logf(z);
    }
    return;
  }
  // thresholds
  uint32_t floor_key = 0;
  float kept_mass = z;
  const int k = p.top_k ? p.top_k[r] : 0;
  if (k > 0 && k < p.vocab) {
    float above;
    floor_key = radix_threshold<false>(row, p.vocab, m, static_cast<float>(k), 0u, hist, bcast, &above);
    float zk = 0.f;
    for (int i = threadIdx.x; i < p.vocab; i += blockDim.x) {
      const float x = row.at(i);
      if (order_key(x) >= floor_key) zk += __expf(x - m);
    }
    kept_mass = block_sum(zk, red);
  }
  const float tp = p.top_p ? p.top_p[r] : 1.f;
  if (tp < 1.f && tp > 0.f) {
    float above;
    const uint32_t kp = radix_threshold<true>(row, p.vocab, m, tp * kept_mass, floor_key, hist, bcast, &above);
    floor_key = max(floor_key, kp);
  }
  const float mp = p.min_p ? p.min_p[r] : 0.f;
  if (mp > 0.f) floor_key = max(floor_key, order_key(m + __logf(mp)));
  // Gumbel-max over the survivors at temperature T, and their tempered partition function for the log-probability
  const unsigned long long seed = p.seeds ? p.seeds[r] : 0ull;
  const float inv_t = row.inv_t;
  float bv = -INFINITY, zt = 0.f;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < p.vocab; i += blockDim.x) {
    const float x = row.at(i);
    if (order_key(x) >= floor_key) {
      const float xt = (x - m) * inv_t;
      zt += __expf(xt);
      const float g = xt + gumbel(uniform01(seed, p.step, static_cast<uint64_t>(i)));
      if (g > bv) { bv = g; bi = i; }
    }
  }
  block_argmax(bv, bi, red, redi);
  zt = block_sum(zt, red);
  if (threadIdx.x == 0) {
    p.out_token[r] = bi;
    if (p.out_logprob) p.out_logprob[r] = (row.at(bi) - m) * inv_t - __logf(zt);
  }
}

// ------------------------------------------------------------------------------------ speculative verification
struct VerifyParams {
  const float* target;   // [n_seq, K+1, vocab] fp32 logits
  const float* draft;    // [n_seq, K, vocab] fp32 logits (null in greedy mode)
  const int* tokens;     // [n_seq, K] drafted tokens
  int K, vocab;
  float temperature;     // <= 0: greedy
  const unsigned long long* seeds;
  unsigned long long step;
  int* n_accepted;       // [n_seq]
  int* next_token;       // [n_seq] correction or bonus token
};

__global__ void __launch_bounds__(kSampThreads) spec_verify_kernel(const VerifyParams p) {
  __shared__ float red[64];
  __shared__ int redi[64];
  const int s = blockIdx.x;
  const bool greedy = !(p.temperature > 0.f);
  const float inv_t = greedy ? 1.f : 1.f / p.temperature;
  const unsigned long long seed = p.seeds ? p.seeds[s] : 0ull;
  const float* trow = p.target + static_cast<long long>(s) * (p.K + 1) * p.vocab;
  const float* drow = p.draft ? p.draft + static_cast<long long>(s) * p.K * p.vocab : nullptr;
  for (int i = 0; i <= p.K; ++i, trow += p.vocab, drow = drow ? drow + p.vocab : nullptr) {
    const bool bonus = i == p.K;
    float tv = -INFINITY;
    int ti = 0x7fffffff;
    for (int j = threadIdx.x; j < p.vocab; j += blockDim.x) {
      const float x = trow[j] * inv_t;
      if (x > tv) { tv = x; ti = j; }
    }
    block_argmax(tv, ti, red, redi);
    const int tok = bonus ? -1 : p.tokens[s * p.K + i];
    if (greedy) {
      if (bonus || ti != tok) {
        if (threadIdx.x == 0) { p.n_accepted[s] = i; p.next_token[s] = ti; }
        return;
      }
      continue;
    }
    float tz = 0.f;
    for (int j = threadIdx.x; j < p.vocab; j += blockDim.x) tz += __expf(trow[j] * inv_t - tv);
    tz = block_sum(tz, red);
    if (bonus) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int j = threadIdx.x; j < p.vocab; j += blockDim.x) {
        const float g = trow[j] * inv_t + gumbel(uniform01(seed, p.step * 64 + 2 * i + 1, static_cast<uint64_t>(j)));
        if (g > bv) { bv = g; bi = j; }
      }
      block_argmax(bv, bi, red, redi);
      if (threadIdx.x == 0) { p.n_accepted[s] = i; p.next_token[s] = bi; }
      return;
    }
    float dv = -INFINITY;
    for (int j = threadIdx.x; j < p.vocab; j += blockDim.x) dv = fmaxf(dv, drow[j] * inv_t);
    dv = block_max(dv, red);
    float dz = 0.f;
    for (int j = threadIdx.x; j < p.vocab; j += blockDim.x) dz += __expf(drow[j] * inv_t - dv);
    dz = block_sum(dz, red);
    const float lt = trow[tok] * inv_t - tv - __logf(tz), ld = drow[tok] * inv_t - dv - __logf(dz);
    const float u = uniform01(seed, p.step * 64 + 2 * i, 0xffffffffull);
    if (__logf(u) < lt - ld) continue;   // accepted with probability min(1, p_t / p_d)
    // rejected: draw from the normalised positive part of (p_t - p_d)
    const float ltz = __logf(tz), ldz = __logf(dz);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int j = threadIdx.x; j < p.vocab; j += blockDim.x) {
      const float pt = __expf(trow[j] * inv_t - tv - ltz), pd = __expf(drow[j] * inv_t - dv - ldz);
      const float res = pt - pd;
      if (res > 0.f) {
        const float g = __logf(res) + gumbel(uniform01(seed, p.step * 64 + 2 * i + 1, static_cast<uint64_t>(j)));
        if (g > bv) { bv = g; bi = j; }
      }
    }
    block_argmax(bv, bi, red, redi);
    if (bi == 0x7fffffff) bi = ti;   // the two distributions coincide numerically
    if (threadIdx.x == 0) { p.n_accepted[s] = i; p.next_token[s] = bi; }
    return;
  }
}

// counts[row, token] += 1 for each newly sampled token (keeps the penalty table current without a host round trip)
__global__ void count_tokens_kernel(int* __restrict__ counts, const int* __restrict__ count_rows,
                                    const int* __restrict__ tokens, int rows, int vocab) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const int t = tokens[r];
  const long long cr = count_rows ? count_rows[r] : r;
  if (t >= 0 && t < vocab) counts[cr * vocab + t] += 1;
}

}  // namespace pm

using namespace pm;

extern "C" int pm_sample(const void* logits, int is_bf16, long long ld, int rows, int vocab, const int* counts,
                         const int* count_rows, const float* temperature, const int* top_k, const float* top_p, const float* min_p,
                         const float* rep_pen, const float* freq_pen, const float* pres_pen,
                         const unsigned long long* seeds, unsigned long long step, int* out_token, float* out_logprob,
                         cudaStream_t st) {
  if (rows <= 0 || vocab <= 0 || !temperature) return -1;
  SampleParams p{logits, is_bf16, ld, vocab, counts, count_rows, temperature, top_k, top_p, min_p, rep_pen, freq_pen, pres_pen,
                 seeds, step, out_token, out_logprob};
  sample_kernel<<<rows, kSampThreads, 0, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int pm_spec_verify(const float* target, const float* draft, const int* tokens, int n_seq, int K, int vocab,
                              float temperature, const unsigned long long* seeds, unsigned long long step,
                              int* n_accepted, int* next_token, cudaStream_t st) {
  if (n_seq <= 0 || K < 0 || vocab <= 0) return -1;
  if (temperature > 0.f && !draft) return -2;
  VerifyParams p{target, draft, tokens, K, vocab, temperature, seeds, step, n_accepted, next_token};
  spec_verify_kernel<<<n_seq, kSampThreads, 0, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int pm_count_tokens(int* counts, const int* count_rows, const int* tokens, int rows, int vocab,
                               cudaStream_t st) {
  if (rows <= 0) return 0;
  count_tokens_kernel<<<(rows + 127) / 128, 128, 0, st>>>(counts, count_rows, tokens, rows, vocab);
  return static_cast<int>(cudaGetLastError());
}
