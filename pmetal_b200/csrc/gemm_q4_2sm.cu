// GEMM against a 4-bit (NF4 / FP4, blocks of 64) weight that is expanded on the way into the tensor cores: no bf16
// copy of the weight is ever written to global memory, in the forward or in the backward pass (QLoRA training; cf. the
// reference's quantised forward / backward, crates/pmetal-lora/src/qlora.rs:287-402, and its dequantising GEMM,
// crates/pmetal-metal/src/kernels/metal4/mpp_quantized.metal).
//
//   forward         D[M, N]  = alpha * ( A[M, K]  * W[N, K]^T + A2[M, K2] * B2[N, K2]^T ) (+ R)      W packed [N, K]
//   input gradient  D[M, Kw] = alpha * ( A[M, Nw] * W[Nw, Kw] + A2[M, K2] * B2[Kw, K2]^T ) (+ R)     same packed W
//
// Same CTA-pair structure as gemm_2sm.cu (256 x 256 tile per pair, tcgen05.mma.cta_group::2, accumulators in TMEM),
// with the B operand produced inside the CTA: the TMA producer brings the packed codes of this CTA's half of the B
// tile (4 KB per 64-wide K block) into a staging ring, eight dequant warps look the codes up in a register-resident code
// book with byte permutes, scale them by the block's absmax (fp32, or 8-bit double-quantised) and store them in the 128-byte-swizzled
// layout the MMA descriptors expect (K-major for the forward pass, MN-major for the input gradient, where the packed
// rows run along the reduction). A generic-to-async proxy fence orders those stores before the MMA reads them.
// The low-rank second product arrives as bf16 through TMA exactly as in the dense kernel.
//
// Per-stage barriers in every CTA of the pair:
//   cfull[s]  <- the codes of the stage have landed (or: this K block needs no expansion)
//   full[s]   <- A tile bytes + one arrive per dequant warp; the partner forwards its completion to the leader
//   empty[s]  <- tcgen05.commit from the leader (to both CTAs)
// Every wait is bounded.
#include "gemm_pair.cuh"
#include "pmetal_b200.h"

namespace pm {

constexpr int kQ4DequantWarps = 8;
constexpr int kQ4Threads = kThreads + 32 * kQ4DequantWarps;       // 448
constexpr int kQ4CodeBytes = kHalfBN * kBK / 2;                    // 4 KB of codes per CTA per K block
constexpr int kQ4StageBytes = kPairStageBytes + kQ4CodeBytes;      // 36 KB

struct Q4Params {
  const float* absmax;         // fp32 scale per block of 64, or null
  const uint8_t* absmax_q;     // 8-bit scale codes (value = code * am_scale + am_offset)
  float am_scale, am_offset;
  int fp4;                     // 0: NF4 code book, 1: FP4
  int w_rows, w_cols;          // shape of the packed weight
  int trans;                   // 0: B[n, k] = W[n, k] (forward); 1: B[n, k] = W[k, n] (input gradient)
};

__constant__ float kQ4Nf4[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                                 -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                                 0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
                                 0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};
__constant__ float kQ4Fp4[16] = {0.0f, 0.0052083333f, 0.6666667f, 1.0f, 0.3333333f, 0.5f, 0.1666667f, 0.25f,
                                 -0.0f, -0.0052083333f, -0.6666667f, -1.0f, -0.3333333f, -0.5f, -0.1666667f, -0.25f};

__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

// Eight 4-bit codes (one 32-bit word of the packed weight; byte b holds element 2b in its high nibble and element 2b+1 in
// its low nibble) -> eight bf16 values times the block scale, as one 16-byte chunk. The 16-entry code book lives in eight
// registers (th: the high bytes of its bf16 values, tl: the low bytes, four entries per register), and a value is looked
// up with byte permutes: one permute per half of the table with the low three bits of the code as selector, a third
// permute in sign-replicating mode that turns bit 3 of every code into a byte mask, and a bitwise select. No shared-
// memory traffic, which this kernel has none to spare of. Table entries and scale are rounded to bf16 and multiplied in
// bf16, so a value can differ from the fp32-multiplied reference by two units in the last place.
__device__ __forceinline__ void q4_expand8(uint32_t w, const uint32_t (&th)[4], const uint32_t (&tl)[4],
                                           __nv_bfloat162 sc2, uint32_t (&out)[4]) {
  const uint32_t ws = w << 4;
#pragma unroll
  for (int half = 0; half < 2; ++half) {                       // nibbles 0..3, then 4..7
    const uint32_t sel = (half ? (w >> 16) : w) & 0x7777u;
    const uint32_t mask = prmt(ws, w, half ? 0xFBEAu : 0xD9C8u);
    const uint32_t ha = prmt(th[0], th[1], sel), hb = prmt(th[2], th[3], sel);
    const uint32_t la = prmt(tl[0], tl[1], sel), lb = prmt(tl[2], tl[3], sel);
    const uint32_t hw = (ha & ~mask) | (hb & mask);
    const uint32_t lw = (la & ~mask) | (lb & mask);
    // nibble i is element i ^ 1: (element 0, element 1) = (nibble 1, nibble 0), low byte first
    uint32_t p0 = prmt(lw, hw, 0x4051u), p1 = prmt(lw, hw, 0x6273u);
    __nv_bfloat162 v0 = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&p0), sc2);
    __nv_bfloat162 v1 = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&p1), sc2);
    out[half * 2] = *reinterpret_cast<uint32_t*>(&v0);
    out[half * 2 + 1] = *reinterpret_cast<uint32_t*>(&v1);
  }
}

__global__ void __launch_bounds__(kQ4Threads, 1)
gemm_q4_2sm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_c,
                   const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_b2,
                   const GemmParams p, const Q4Params q) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int a_bytes = kBM * kBK * 2;
  const int b_bytes = kHalfBN * kBK * 2;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + p.stages * kQ4StageBytes);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* cfull_bar = empty_bar + kMaxStages;
  uint64_t* pfull_bar = cfull_bar + kMaxStages;   // leader only: "the partner's stage is complete"
  uint64_t* tfull_bar = pfull_bar + kMaxStages;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;           // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < p.stages; ++i) {
      mbar_init(&full_bar[i], 1 + kQ4DequantWarps);
      mbar_init(&empty_bar[i], 1);
      mbar_init(&cfull_bar[i], 1);
      mbar_init(&pfull_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 8);
    }
    *abort_flag = 0;
    mbar_init_fence();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_c);
    if (p.nk2) {
      tma_prefetch_desc(&map_a2);
      tma_prefetch_desc(&map_b2);
    }
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int m_tiles = (p.M + 2 * kBM - 1) / (2 * kBM);
  const int n_tiles = (p.N + kPairBN - 1) / kPairBN;
  const int total = m_tiles * n_tiles;
  const int nk = p.nk1 + p.nk2;
  const int first = static_cast<int>(cluster_id_x());
  const int stride = static_cast<int>(num_clusters_x());

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int w = first; w < total && ok; w += stride) {
        const int nb = w % n_tiles, mb = w / n_tiles;
        const int m0 = mb * 2 * kBM + static_cast<int>(rank) * kBM;
        const int n_tile0 = nb * kPairBN;
        const int n0 = n_tile0 + static_cast<int>(rank) * kHalfBN;
        const int a2_off = p.seg_mode == 1 ? seg_of(p, n_tile0) * p.seg_r : 0;
        for (int kb = 0; kb < nk; ++kb, ++it) {
          const int s = it % p.stages;
          const uint32_t ph = (it / p.stages) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, kTimeoutProducer)) { ok = false; break; }
          const uint32_t sa = smem_u32(smem + s * kQ4StageBytes);
          const uint32_t sb = sa + a_bytes;
          const uint32_t sc = sb + b_bytes;
          const uint32_t fb = smem_u32(&full_bar[s]);
          if (kb < p.nk1) {
            mbar_expect_tx(&full_bar[s], a_bytes);
            load_operand_pair_t<true>(sa, &map_a, fb, 0, kBM, m0, kb * kBK);
            mbar_expect_tx(&cfull_bar[s], kQ4CodeBytes);
            if (!q.trans) tma_load_2d_local(sc, &map_c, smem_u32(&cfull_bar[s]), kb * (kBK / 2), n0);
            else tma_load_2d_local(sc, &map_c, smem_u32(&cfull_bar[s]), n0 / 2, kb * kBK);
          } else {
            const int k0 = (kb - p.nk1) * kBK;
            mbar_expect_tx(&full_bar[s], a_bytes + b_bytes);
            load_operand_pair_t<true>(sa, &map_a2, fb, p.a2_mn, kBM, m0, k0 + a2_off);
            load_operand_pair_t<true>(sb, &map_b2, fb, p.b2_mn, kHalfBN, n0, k0);
            mbar_arrive(&cfull_bar[s]);         // nothing to expand in this block
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ partner: forward "stage complete" to the leader
    if (lane == 0 && !leader) {
      uint32_t it = 0;
      bool ok = true;
      for (int w = first; w < total && ok; w += stride) {
        for (int kb = 0; kb < nk; ++kb, ++it) {
          const int s = it % p.stages;
          const uint32_t ph = (it / p.stages) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
          mbar_arrive_cluster(map_to_cta(smem_u32(&pfull_bar[s]), 0));
        }
      }
    }
    // ------------------------------------------------------------------ MMA issuer (leader)
    if (lane == 0 && leader) {
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int w = first; w < total && ok; w += stride) {
        const int buf = acc_it & 1;
        const uint32_t aph = (acc_it >> 1) & 1;
        if (!mbar_wait_cluster(&tempty_bar[buf], aph ^ 1, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * kPairBN;
        uint32_t accumulate = 0;
        for (int kb = 0; kb < nk; ++kb, ++it) {
          const int s = it % p.stages;
          const uint32_t ph = (it / p.stages) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
          if (!mbar_wait_cluster(&pfull_bar[s], ph, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * kQ4StageBytes);
          const uint32_t sb = sa + a_bytes;
          int amn, bmn, nmma;
          if (kb < p.nk1) {
            amn = 0; bmn = q.trans; nmma = 4;
          } else {
            amn = p.a2_mn; bmn = p.b2_mn;
            nmma = min(4, (p.K2 - (kb - p.nk1) * kBK + 15) / 16);
          }
          const uint32_t idesc = make_idesc_bf16_m256(kPairBN, amn, bmn);
          const uint64_t da = make_smem_desc(sa, amn ? 8192u : 16u, 1024u);
          const uint64_t db = make_smem_desc(sb, bmn ? 8192u : 16u, 1024u);
          const uint32_t astep = amn ? 128u : 2u, bstep = bmn ? 128u : 2u;
          for (int j = 0; j < nmma; ++j) {
            umma_f16_pair(d_tmem, da + static_cast<uint64_t>(astep * j), db + static_cast<uint64_t>(bstep * j), idesc,
                          accumulate);
            accumulate = 1;
          }
          umma_commit_pair(map_to_cta(smem_u32(&empty_bar[s]), 0));
          umma_commit_pair(map_to_cta(smem_u32(&empty_bar[s]), 1));
        }
        if (ok) {
          umma_commit_pair(map_to_cta(smem_u32(&tfull_bar[buf]), 0));
          umma_commit_pair(map_to_cta(smem_u32(&tfull_bar[buf]), 1));
        }
        ++acc_it;
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue (warps 2..5 of each CTA)
    const int qd = warp & 3;
    uint32_t acc_it = 0;
    bool ok = true;
    for (int w = first; w < total && ok; w += stride) {
      const int nb = w % n_tiles, mb = w / n_tiles;
      const int buf = acc_it & 1;
      const uint32_t aph = (acc_it >> 1) & 1;
      if (!mbar_wait(&tfull_bar[buf], aph, abort_flag, p.status, kTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after();
      const int row = mb * 2 * kBM + static_cast<int>(rank) * kBM + qd * 32 + lane;
      const bool row_ok = row < p.M;
      for (int c = 0; c < kPairBN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + buf * kPairBN + c * 32 + (static_cast<uint32_t>(qd * 32) << 16), r);
        tmem_ld_wait();
        const int col0 = nb * kPairBN + c * 32;
        if (!row_ok || col0 >= p.n_store) continue;
        epilogue_store_chunk(p, r, row, col0);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[buf]), 0));
      ++acc_it;
    }
  } else {
    // ------------------------------------------------------------------ dequant warps (6..13): one 16-byte code word
    // (32 weights, four 16-byte chunks of bf16) per thread and K block
    const int t = threadIdx.x - kThreads;            // 0..255
    const int blocks_per_row = q.w_cols / 64;
    // where this thread's 16 bytes of codes sit in the staging tile, where its 32 values go in the B tile, and which
    // scale they use: fixed per thread up to the tile / K-block origin
    int row, dst_off;
    if (!q.trans) {          // staging [128 rows][32 B]; B tile row = weight row, 64 k = 128 B
      row = t >> 1;
      dst_off = row * 128 + (t & 1) * 64;
    } else {                 // staging [64 rows][64 B]; two boxes of [64 k][64 mn]
      row = t >> 2;
      dst_off = ((t >> 1) & 1) * 8192 + row * 128 + (t & 1) * 64;
    }
    const int code_off = t * 16;
    uint32_t th[4], tl[4];                           // the code book as bf16, split into high and low bytes
    {
      const float* tab = q.fp4 ? kQ4Fp4 : kQ4Nf4;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        th[j] = tl[j] = 0u;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const uint32_t bits = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(tab[4 * j + e])));
          th[j] |= (bits >> 8) << (8 * e);
          tl[j] |= (bits & 0xFFu) << (8 * e);
        }
      }
    }
    auto scale_of = [&](int w, int kb) -> float {
      if (w >= total || kb >= p.nk1) return 0.f;
      const int n0 = (w % n_tiles) * kPairBN + static_cast<int>(rank) * kHalfBN;
      long long blk;
      if (!q.trans) blk = static_cast<long long>(min(n0 + row, q.w_rows - 1)) * blocks_per_row + kb;
      else blk = static_cast<long long>(min(kb * 64 + row, q.w_rows - 1)) * blocks_per_row +
                 min(n0 / 64 + ((t >> 1) & 1), blocks_per_row - 1);
      return q.absmax ? __ldg(q.absmax + blk) : static_cast<float>(__ldg(q.absmax_q + blk)) * q.am_scale + q.am_offset;
    };
    uint32_t it = 0;
    bool ok = true;
    float scale = scale_of(first, 0);          // the scale of the next K block is always requested one block ahead
    for (int w = first; w < total && ok; w += stride) {
      for (int kb = 0; kb < nk; ++kb, ++it) {
        const int s = it % p.stages;
        const uint32_t ph = (it / p.stages) & 1;
        const bool expand = kb < p.nk1;
        const float next_scale = (kb + 1 < nk) ? scale_of(w, kb + 1) : scale_of(w + stride, 0);
        if (!mbar_wait(&cfull_bar[s], ph, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
        if (expand) {
          uint8_t* sb = smem + s * kQ4StageBytes + a_bytes;
          const uint4 cw = *reinterpret_cast<const uint4*>(sb + b_bytes + code_off);
          const uint32_t words[4] = {cw.x, cw.y, cw.z, cw.w};
          const int c0 = (dst_off >> 4) & 7;           // first chunk index within the 128-byte row
          uint8_t* rowp = sb + (dst_off & ~127);
          const __nv_bfloat162 sc2 = __float2bfloat162_rn(scale);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t o[4];
            q4_expand8(words[i], th, tl, sc2, o);
            const int chunk = (c0 + i) ^ (row & 7);
            *reinterpret_cast<uint4*>(rowp + chunk * 16) = make_uint4(o[0], o[1], o[2], o[3]);
          }
          fence_proxy_async_smem();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_bar[s]);
        scale = next_scale;
      }
    }
  }

  // ------------------------------------------------------------------ tail
  __syncwarp();
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// uint8 tensor map without swizzle: rows of `inner_bytes`, row pitch `ld_bytes`
static int make_map_u8(CUtensorMap* map, const void* ptr, uint64_t inner_bytes, uint64_t rows, uint64_t ld_bytes,
                       uint32_t box_inner, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  cuuint64_t dims[2] = {inner_bytes, rows};
  cuuint64_t strides[1] = {ld_bytes};
  cuuint32_t box[2] = {box_inner, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r) - 1000;
}

}  // namespace pm

using namespace pm;

// A [M, K] bf16 (K-major). codes: packed weight [w_rows, w_cols / 2] bytes, first element of a pair in the high nibble;
// absmax (fp32) or absmax_q (+ am_scale / am_offset) hold one scale per 64 consecutive weights of a row.
//   trans 0: D[M, w_rows] (K = w_cols);  trans 1: D[M, w_cols] (K = w_rows).
// A2 / B2 (bf16, optional) add the low-rank product as in pm_gemm_bf16_2sm; seg_mode 0 or 1. D bf16 (+ R).
// w_cols % 128 == 0 and w_rows % 64 == 0. Returns 0, a negative argument error or a CUDA error code.
extern "C" int pm_gemm_q4_2sm(const void* A, int lda, int a_rows, const void* codes, const float* absmax,
                              const void* absmax_q, float am_scale, float am_offset, int fp4, int w_rows, int w_cols,
                              int trans, const void* A2, int a2_mn, int lda2, int a2_k, const void* B2, int b2_mn, int ldb2,
                              int b2_rows, void* D, int ldd, const void* R, int ldr, int M, int K2, int n_store,
                              float alpha, int seg_mode, const int* seg_end, int seg_r, int max_ctas, int* status,
                              cudaStream_t stream) {
  if (M <= 0 || w_rows <= 0 || w_cols <= 0 || (w_cols % 128) || (w_rows % 64)) return -13;
  if ((ldd % 8) || (reinterpret_cast<uintptr_t>(D) & 15) || (reinterpret_cast<uintptr_t>(codes) & 15)) return -14;
  if (R && ((ldr % 8) || (reinterpret_cast<uintptr_t>(R) & 15))) return -15;
  if (!absmax && !absmax_q) return -16;
  if (seg_mode != 0 && seg_mode != 1) return -17;
  const int N = trans ? w_cols : w_rows, K = trans ? w_rows : w_cols;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.K2 = K2; p.bn = kPairBN;
  p.a_mn = 0; p.b_mn = trans; p.a2_mn = a2_mn; p.b2_mn = b2_mn;
  p.nk1 = K / kBK;
  p.nk2 = K2 > 0 ? (K2 + kBK - 1) / kBK : 0;
  p.splits = 1;
  p.out_mode = 0; p.ldd = ldd; p.ldr = ldr; p.n_store = n_store > 0 ? n_store : N;
  p.alpha = alpha; p.D = D; p.R = R;
  p.seg_mode = seg_mode; p.seg_r = seg_r;
  for (int i = 0; i < 4; ++i) p.seg_end[i] = (seg_mode && seg_end) ? seg_end[i] : 0x7fffffff;
  p.status = status;
  p.kps = 1; p.fwd_full = 1; p.commit_both = 0;
  int stages = (227 * 1024 - 2048) / kQ4StageBytes;
  if (stages > kMaxStages) stages = kMaxStages;
  p.stages = stages;
  p.tmem_cols = 512;
  Q4Params q{};
  q.absmax = absmax; q.absmax_q = static_cast<const uint8_t*>(absmax_q); q.am_scale = am_scale; q.am_offset = am_offset;
  q.fp4 = fp4; q.w_rows = w_rows; q.w_cols = w_cols; q.trans = trans;

  CUtensorMap ma, mc, ma2, mb2;
  int rc;
  if ((rc = operand_map(&ma, A, 0, a_rows, K, lda, kBM))) return rc * 10 - 1;
  if (!trans) rc = make_map_u8(&mc, codes, w_cols / 2, w_rows, w_cols / 2, kBK / 2, kHalfBN);
  else rc = make_map_u8(&mc, codes, w_cols / 2, w_rows, w_cols / 2, kHalfBN / 2, kBK);
  if (rc) return rc * 10 - 2;
  if (K2 > 0) {
    if ((rc = operand_map(&ma2, A2, a2_mn, a_rows, a2_k, lda2, kBM))) return rc * 10 - 3;
    if ((rc = operand_map(&mb2, B2, b2_mn, b2_rows, K2, ldb2, kHalfBN))) return rc * 10 - 4;
  } else {
    ma2 = ma; mb2 = ma;
  }
  const size_t smem = static_cast<size_t>(stages) * kQ4StageBytes + 1024 + 512;
  static DeviceOnce configured;
  if (configured.pending()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_q4_2sm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured.mark();
  }
  const int m_tiles = (M + 2 * kBM - 1) / (2 * kBM), n_tiles = (N + kPairBN - 1) / kPairBN;
  int pairs = m_tiles * n_tiles;
  int cap = (max_ctas > 0 ? max_ctas : num_sms()) / 2;
  if (pairs > cap) pairs = cap;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(kQ4Threads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_q4_2sm_kernel, ma, mc, ma2, mb2, p, q);
  return static_cast<int>(e);
}
