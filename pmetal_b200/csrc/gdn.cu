// Gated delta rule recurrence (linear-attention layers of the Qwen3-Next hybrids), sequential over tokens with the
// per-head state kept in registers:
//
//     S <- g_t S;   u = beta_t (v_t - k_t S);   S <- S + k_t^T u;   y_t = q_t S          S: [dk, dv] per head
//
// One CTA per (sequence, head); thread t owns column j = t % dv of S for a slice of the dk rows (dk * dv / threads
// values in registers), so the three passes over the state per token (k S, rank-one update, q S) are register FMAs;
// only the per-column partial sums of the row slices cross threads, through shared memory. q and k of a token are
// staged in shared memory by the CTA. Used for decode (T = 1, state in / state out) and for prefill of moderate length;
// the chunk-parallel form for long prefill is models/gdn.py.
//
// Reference: the recurrent step and state update that the reference JIT-compiles as Metal source
// (crates/pmetal-bridge/cpp/bridge_native.cpp:6-139, gdn_metal_step / gdn_metal_state_update) and
// crates/pmetal-mlx/src/kernels/gated_delta.rs.
#include <cuda_runtime.h>
#include <stdint.h>
#include "host_util.cuh"
#include "pmetal_b200.h"

namespace pm {

constexpr int kGdnThreads = 256;

// q, k: [B, T, H, DK] fp32; v: [B, T, H, DV]; g, beta: [B, T, H]; state: [B, H, DK, DV] (in/out); y: [B, T, H, DV].
template <int DK, int DV>
__global__ void __launch_bounds__(kGdnThreads) gdn_scan_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                                               const float* __restrict__ v, const float* __restrict__ g,
                                                               const float* __restrict__ beta, float* __restrict__ state,
                                                               float* __restrict__ y, int T, int H) {
  constexpr int kSlices = kGdnThreads / DV;          // row slices of the state
  constexpr int kRows = DK / kSlices;                // rows per thread
  static_assert(kGdnThreads % DV == 0 && DK % kSlices == 0, "tile shape");
  __shared__ float sq[DK], sk[DK];
  __shared__ float part[kSlices][DV];
  const int b = blockIdx.x / H, h = blockIdx.x % H;
  const int j = threadIdx.x % DV, slice = threadIdx.x / DV, r0 = slice * kRows;
  float S[kRows];
  float* st = state + (static_cast<long long>(b) * H + h) * DK * DV;
#pragma unroll
  for (int i = 0; i < kRows; ++i) S[i] = st[(r0 + i) * DV + j];
  for (int t = 0; t < T; ++t) {
    const long long tok = (static_cast<long long>(b) * T + t) * H + h;
    __syncthreads();                                  // previous token's readers of sq / sk / part are done
    for (int i = threadIdx.x; i < DK; i += kGdnThreads) {
      sq[i] = q[tok * DK + i];
      sk[i] = k[tok * DK + i];
    }
    const float gt = g[tok], bt = beta[tok];
    __syncthreads();
    float pred = 0.f;
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
      S[i] *= gt;
      pred = fmaf(sk[r0 + i], S[i], pred);
    }
    part[slice][j] = pred;
    __syncthreads();
    float full = 0.f;
#pragma unroll
    for (int s = 0; s < kSlices; ++s) full += part[s][j];
    const float u = bt * (v[tok * DV + j] - full);
    float out = 0.f;
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
      S[i] = fmaf(sk[r0 + i], u, S[i]);
      out = fmaf(sq[r0 + i], S[i], out);
    }
    __syncthreads();                                  // everyone has read part[] of the prediction
    part[slice][j] = out;
    __syncthreads();
    if (slice == 0) {
      float yy = 0.f;
#pragma unroll
      for (int s = 0; s < kSlices; ++s) yy += part[s][j];
      y[tok * DV + j] = yy;
    }
  }
#pragma unroll
  for (int i = 0; i < kRows; ++i) st[(r0 + i) * DV + j] = S[i];
}

}  // namespace pm

using namespace pm;

// Returns 0, -1 for an unsupported head shape (supported: dk x dv in {64, 128} x {64, 128}), or a CUDA error code.
extern "C" int pm_gdn_scan(const float* q, const float* k, const float* v, const float* g, const float* beta, float* state,
                           float* y, int B, int T, int H, int dk, int dv, cudaStream_t st) {
  if (B < 1 || T < 1 || H < 1) return -1;
  const dim3 grid(B * H), block(kGdnThreads);
  if (dk == 128 && dv == 128) gdn_scan_kernel<128, 128><<<grid, block, 0, st>>>(q, k, v, g, beta, state, y, T, H);
  else if (dk == 64 && dv == 64) gdn_scan_kernel<64, 64><<<grid, block, 0, st>>>(q, k, v, g, beta, state, y, T, H);
  else if (dk == 128 && dv == 64) gdn_scan_kernel<128, 64><<<grid, block, 0, st>>>(q, k, v, g, beta, state, y, T, H);
  else if (dk == 64 && dv == 128) gdn_scan_kernel<64, 128><<<grid, block, 0, st>>>(q, k, v, g, beta, state, y, T, H);
  else return -1;
  return static_cast<int>(cudaGetLastError());
}
