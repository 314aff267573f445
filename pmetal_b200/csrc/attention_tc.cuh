// Shared definitions of the tcgen05 attention kernels (forward, dQ, dK/dV).
#pragma once
#include "gemm_common.cuh"

namespace pm {

constexpr int kFaThreads = 192;
constexpr int kFaThreads2 = 320;              // TMA warp, MMA warp, two compute warp groups
constexpr int kFaTile = 128;                 // queries per CTA and keys per tile
constexpr int kFaBox = kFaTile * 64 * 2;     // one [128 rows][64 cols] bf16 box: 16 KB
constexpr int kFaTileBytes = 2 * kFaBox;     // [128][128] bf16: 32 KB
constexpr float kFaLog2e = 1.4426950408889634f;

struct FaParams {
  __nv_bfloat16* out;     // forward: O; dQ kernel: dQ; dKV kernel: dK
  __nv_bfloat16* out2;    // dKV kernel: dV
  long long o_stride, o2_stride;
  float* lse;             // [hq][T], natural log
  const float* delta;     // [hq][T] rowsum(dO * O)   (backward)
  const int* seq_start;   // [T]
  int T, hq, hkv;
  float scale;
  int* status;
  // forward kernel only: number of key rows and the causal offset; key j is visible to query i iff
  // seq_start[i] <= j <= i + shift (and j < Tk). Tk = T, shift = 0 is ordinary causal attention; shift >= Tk - 1
  // makes every key visible (a block of ring attention that lies entirely in the past).
  int Tk, shift;
};

// 2^x on the SFU; -inf gives 0
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Store 32 bf16 (packed in pk[16]) of row r into a [128][128] bf16 tile made of two 128B-swizzled
// [128][64] boxes; c = index of the 32-column chunk (0..3). This is the layout tcgen05.mma reads as a
// K-major operand (rows = M/N) and, with the other descriptor, as an MN-major operand (rows = K).
__device__ __forceinline__ void store_row_chunk_sw128(uint32_t tile_addr, int r, int c, const uint32_t (&pk)[16]) {
  const uint32_t row = tile_addr + (c >> 1) * kFaBox + r * 128;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const int chunk = (c & 1) * 4 + g;
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(row + ((chunk ^ (r & 7)) << 4)), "r"(pk[4 * g]),
                 "r"(pk[4 * g + 1]), "r"(pk[4 * g + 2]), "r"(pk[4 * g + 3])
                 : "memory");
  }
}
// descriptors for a [128][128] bf16 tile (two boxes): step s = 16-element slice of the reduction dimension
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile_addr, int s) {
  return make_smem_desc(tile_addr + (s >> 2) * kFaBox + (s & 3) * 32, 16u, 1024u);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile_addr, int s) {
  return make_smem_desc(tile_addr + s * 2048, static_cast<uint32_t>(kFaBox), 1024u);
}


}  // namespace pm
