// Data-parallel gradient reduction fused with scaling, clipping and the AdamW update, over NVLink peer memory.
//
// Every rank keeps its flat fp32 gradient buffer, fp32 parameters and bf16 parameter shadow in
// symmetric (peer-mapped) memory. One launch per rank performs, for the shard of the flat buffer the
// rank owns:
//     g      = sum_p coef_p * grad_p[i]            (P2P loads from every peer: the reduce-scatter,
//                                                   with each rank's clip * 1/accum * 1/N coefficient)
//     m,v,p  = AdamW(g)                            (reference semantics: bias-corrected step, then
//                                                   decoupled decay on the updated parameter)
//     param_q[i], shadow_q[i] = p for every rank q (P2P stores: the all-gather of updated parameters)
// It replaces the reference's flatten -> TCP ring all-reduce(Mean) -> scatter -> optimizer sequence
// (crates/pmetal-distributed/src/ring.rs:48-185, crates/pmetal-trainer/src/distributed_bridge.rs:164-221)
// and its fused Metal AdamW (crates/pmetal-metal/src/kernels/metal/fused_training.metal:82-200).
//
// Cross-rank ordering uses epoch-valued flags in each rank's signal pad:
//   ready[r] : rank r's gradients (and its coefficient) for this epoch are complete
//   done[r]  : rank r has finished reading everybody's gradients and writing everybody's parameters
// All waits are bounded; on expiry the kernel records a status code and returns.
// Plain peer loads/stores only (no multimem), so a rank may leave between steps without faulting peers.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "host_util.cuh"
#include "pmetal_b200.h"

namespace pm {

constexpr int kMaxRanks = 8;
constexpr int kStatusPeerTimeout = 104;

// signal pad layout (uint32 words)
constexpr int kReadyOff = 0;    // [kMaxRanks]
constexpr int kDoneOff = 8;     // [kMaxRanks]
constexpr int kCoefOff = 16;    // [kMaxRanks] float bits
constexpr int kEpochOff = 24;   // local epoch counter
constexpr int kArriveOff = 25;  // local CTA arrival counter
constexpr int kPadWords = 32;

struct DpArgs {
  const float* grads[kMaxRanks];       // peer-mapped flat gradient buffers
  float* params[kMaxRanks];            // peer-mapped flat fp32 parameters
  __nv_bfloat16* shadows[kMaxRanks];   // peer-mapped bf16 shadows (may be null)
  uint32_t* pads[kMaxRanks];           // peer-mapped signal pads
  float* m;
  float* v;
  const float* lr_mult;
  const float* wd;
  const float* gnorm_sq;   // local squared gradient norm (unscaled buffer)
  const float* hp;         // optional device [lr, bc1, bc2]
  long long n;             // total elements (multiple of 1024)
  long long lo, hi;        // owned shard
  int rank, world;
  float lr, beta1, beta2, eps, bc1, bc2, grad_scale, max_norm;
  unsigned long long timeout_ns;
  int* status;
};

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Wait until pad[off + r] >= epoch for every rank r. Threads 0..world-1 of the CTA spin; returns false on timeout.
__device__ __forceinline__ bool wait_all(const uint32_t* pad, int off, int world, uint32_t epoch,
                                         unsigned long long timeout_ns, int* status, int* s_fail) {
  if (threadIdx.x < world) {
    const uint32_t* f = pad + off + threadIdx.x;
    unsigned long long t0 = 0;     // the global timer is slow to read: first looked at after 1024 failed polls
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys(f) - epoch) < 0) {
      if ((++spins & 63u) == 0u && spins >= 1024u) {
        const unsigned long long now = now_ns();
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > timeout_ns) {
          atomicCAS(status, 0, kStatusPeerTimeout);
          *s_fail = 1;
          break;
        }
      }
    }
  }
  __syncthreads();
  return *s_fail == 0;
}

__global__ void __launch_bounds__(256) dp_reduce_adamw_kernel(const DpArgs a) {
  __shared__ int s_fail;
  __shared__ float s_coef[kMaxRanks];
  __shared__ int s_last;
  uint32_t* my_pad = a.pads[a.rank];
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  const uint32_t epoch = my_pad[kEpochOff] + 1u;

  // ---- publish this rank's coefficient and "gradients ready" to every rank
  if (blockIdx.x == 0 && threadIdx.x < a.world) {
    float coef = a.grad_scale / a.world;
    if (a.max_norm > 0.f) {
      const float norm = sqrtf(*a.gnorm_sq) * a.grad_scale;
      coef *= fminf(1.f, a.max_norm / (norm + 1e-6f));
    }
    uint32_t* peer = a.pads[threadIdx.x];
    peer[kCoefOff + a.rank] = __float_as_uint(coef);
    __threadfence_system();
    st_release_sys(peer + kReadyOff + a.rank, epoch);
  }
  // ---- wait for every rank's gradients
  if (!wait_all(my_pad, kReadyOff, a.world, epoch, a.timeout_ns, a.status, &s_fail)) {
    // abandoned step: still count this CTA in, and let the last one close the epoch, so that the pad is in a
    // defined state for the next launch (flags of the failed epoch are then simply too old to match)
    if (threadIdx.x == 0) {
      const uint32_t prev = atomicAdd(my_pad + kArriveOff, 1u);
      if (prev == gridDim.x - 1) {
        my_pad[kArriveOff] = 0u;
        my_pad[kEpochOff] = epoch;
        __threadfence_system();
      }
    }
    return;
  }
  if (threadIdx.x < a.world) s_coef[threadIdx.x] = __uint_as_float(my_pad[kCoefOff + threadIdx.x]);
  __syncthreads();

  float lr = a.lr, bc1 = a.bc1, bc2 = a.bc2;
  if (a.hp) { lr = a.hp[0]; bc1 = a.hp[1]; bc2 = a.hp[2]; }

  // ---- owned shard: reduce, update, broadcast
  for (long long i = a.lo + (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 4; i < a.hi;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
    float4 gp[kMaxRanks];
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (r < a.world) gp[r] = *reinterpret_cast<const float4*>(a.grads[r] + i);
    float g[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (r < a.world) {
        const float c = s_coef[r];
        g[0] += c * gp[r].x; g[1] += c * gp[r].y; g[2] += c * gp[r].z; g[3] += c * gp[r].w;
      }
    const int chunk = static_cast<int>(i >> 10);
    const float lrc = lr * a.lr_mult[chunk];
    const float decay = a.wd[chunk] * lrc;
    float4 m4 = *reinterpret_cast<float4*>(a.m + i);
    float4 v4 = *reinterpret_cast<float4*>(a.v + i);
    float4 p4 = *reinterpret_cast<float4*>(a.params[a.rank] + i);
    float mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w}, pp[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      mm[k] = a.beta1 * mm[k] + (1.f - a.beta1) * g[k];
      vv[k] = a.beta2 * vv[k] + (1.f - a.beta2) * g[k] * g[k];
      pp[k] -= lrc * (mm[k] / bc1) / (sqrtf(vv[k] / bc2) + a.eps);
      pp[k] -= decay * pp[k];
    }
    *reinterpret_cast<float4*>(a.m + i) = make_float4(mm[0], mm[1], mm[2], mm[3]);
    *reinterpret_cast<float4*>(a.v + i) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    const float4 pn = make_float4(pp[0], pp[1], pp[2], pp[3]);
    uint2 sh;
    *reinterpret_cast<__nv_bfloat162*>(&sh.x) = __floats2bfloat162_rn(pp[0], pp[1]);
    *reinterpret_cast<__nv_bfloat162*>(&sh.y) = __floats2bfloat162_rn(pp[2], pp[3]);
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (r < a.world) {
        *reinterpret_cast<float4*>(a.params[r] + i) = pn;
        if (a.shadows[r]) *reinterpret_cast<uint2*>(a.shadows[r] + i) = sh;
      }
  }

  // ---- completion: the last CTA tells every rank this rank is done, waits for all ranks, advances the epoch
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(my_pad + kArriveOff, 1u);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence_system();
  if (threadIdx.x < a.world) st_release_sys(a.pads[threadIdx.x] + kDoneOff + a.rank, epoch);
  const bool ok = wait_all(my_pad, kDoneOff, a.world, epoch, a.timeout_ns, a.status, &s_fail);
  if (threadIdx.x == 0) {
    my_pad[kArriveOff] = 0u;
    my_pad[kEpochOff] = epoch;     // also after a timed-out wait: every rank moves on to the same next epoch
    (void)ok;
    __threadfence_system();
  }
}

}  // namespace pm

using namespace pm;

// ptr arrays hold `world` device addresses each (peer-mapped). shadows may be null.
extern "C" int pm_dp_reduce_adamw(const unsigned long long* grads, const unsigned long long* params,
                                  const unsigned long long* shadows, const unsigned long long* pads, float* m, float* v,
                                  const float* lr_mult, const float* wd, const float* gnorm_sq, const float* hp,
                                  long long n, int rank, int world, float lr, float beta1, float beta2, float eps,
                                  int step, float grad_scale, float max_norm, double timeout_s, int ctas, int* status,
                                  cudaStream_t st) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return -1;
  if (n % 1024) return -2;
  DpArgs a{};
  for (int r = 0; r < world; ++r) {
    a.grads[r] = reinterpret_cast<const float*>(grads[r]);
    a.params[r] = reinterpret_cast<float*>(params[r]);
    a.shadows[r] = shadows ? reinterpret_cast<__nv_bfloat16*>(shadows[r]) : nullptr;
    a.pads[r] = reinterpret_cast<uint32_t*>(pads[r]);
  }
  a.m = m; a.v = v; a.lr_mult = lr_mult; a.wd = wd; a.gnorm_sq = gnorm_sq; a.hp = hp;
  a.n = n;
  const long long chunks = n / 1024;
  const long long per = (chunks + world - 1) / world;
  a.lo = (per * rank < chunks ? per * rank : chunks) * 1024;
  a.hi = (per * (rank + 1) < chunks ? per * (rank + 1) : chunks) * 1024;
  a.rank = rank; a.world = world;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps;
  a.bc1 = 1.f - powf(beta1, static_cast<float>(step));
  a.bc2 = 1.f - powf(beta2, static_cast<float>(step));
  a.grad_scale = grad_scale; a.max_norm = max_norm;
  a.timeout_ns = static_cast<unsigned long long>(timeout_s * 1e9);
  a.status = status;
  if (ctas <= 0) ctas = 64;
  dp_reduce_adamw_kernel<<<ctas, 256, 0, st>>>(a);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int pm_dp_pad_words() { return kPadWords; }
