// Pieces shared by the 1-SM and the 2-SM (cta_group::2) tcgen05 GEMM kernels: parameter block,
// LoRA segment lookup, the per-thread epilogue for one 32-column chunk, and tensor-map construction.
#pragma once
#include "common.cuh"

namespace pm {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kThreads = 192;
constexpr int kMaxStages = 8;

struct GemmParams {
  int M, N, K, K2;
  int bn;          // tile width in N: 32, 64, 128 or 256
  int a_mn, b_mn, a2_mn, b2_mn;
  int nk1, nk2;    // number of 64-wide K blocks in the first / second product
  int splits;      // split-K factor (out_mode must be atomic when > 1)
  int stages;
  int out_mode;    // 0: bf16 store, 1: f32 store, 2: f32 atomic add, 3: f32 atomic add, transposed,
                   // 4 / 5: as 2 / 3 with a plain read-add-write (one CTA owns each output tile: needs splits == 1;
                   // the sum is then formed in a fixed order, bit for bit the same on every run)
                   // 6: bf16 store with split-K reduced inside the kernel (1-SM kernel): every split parks its fp32
                   // partial tile in `ws`; the last one to arrive adds them in split order and runs the bf16 epilogue
  int ldd, ldr;
  int n_store;     // columns >= n_store are computed but not written
  float alpha;
  void* D;
  const void* R;
  int seg_mode;    // 0 none; 1: A2 K-offset = seg(n0)*seg_r; 2: B mn-offset = seg(m0)*seg_r; 3: B mn-offset = -seg(k)*seg_r
  int seg_end[4];
  int seg_r;
  int tmem_cols;
  int kps;         // K blocks per pipeline stage (CTA-pair kernel)
  int fwd_full;    // CTA-pair kernel: each CTA counts its own TMA bytes; the partner forwards one arrive per stage
  int commit_both; // CTA-pair kernel: signal both CTAs' barriers with one commit
  int* status;
  float* ws;             // out_mode 6: [tiles][splits][128][bn] fp32 partial tiles
  unsigned* ws_cnt;      // out_mode 6: [tiles][4] arrival counters, zero between launches
};

__device__ __forceinline__ int seg_of(const GemmParams& p, int x) {
  int s = 0;
#pragma unroll
  for (int i = 0; i < 3; ++i) s += (x >= p.seg_end[i]) ? 1 : 0;
  return s;
}


// Write 32 consecutive accumulator columns of one output row (fp32 bits in r) according to out_mode.
__device__ __forceinline__ void epilogue_store_chunk(const GemmParams& p, const uint32_t (&r)[32], int row, int col0) {
    if (p.out_mode == 0 || p.out_mode == 6) {
      __nv_bfloat16* drow = static_cast<__nv_bfloat16*>(p.D) + static_cast<size_t>(row) * p.ldd;
      const __nv_bfloat16* rrow =
          p.R ? static_cast<const __nv_bfloat16*>(p.R) + static_cast<size_t>(row) * p.ldr : nullptr;
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        const int col = col0 + v * 8;
        if (col + 8 <= p.n_store) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[v * 8 + e]) * p.alpha;
          if (rrow) {
            const uint4 rv = *reinterpret_cast<const uint4*>(rrow + col);
            const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              f[2 * e] += bf16_bits_to_float(rw[e] & 0xFFFFu);
              f[2 * e + 1] += bf16_bits_to_float(rw[e] >> 16);
            }
          }
          uint4 o;
          o.x = pack_bf16x2(f[0], f[1]);
          o.y = pack_bf16x2(f[2], f[3]);
          o.z = pack_bf16x2(f[4], f[5]);
          o.w = pack_bf16x2(f[6], f[7]);
          *reinterpret_cast<uint4*>(drow + col) = o;
        } else {
          for (int e = 0; e < 8 && col + e < p.n_store; ++e) {
            float f = __uint_as_float(r[v * 8 + e]) * p.alpha;
            if (rrow) f += __bfloat162float(rrow[col + e]);
            drow[col + e] = __float2bfloat16(f);
          }
        }
      }
    } else if (p.out_mode == 1) {
      float* drow = static_cast<float*>(p.D) + static_cast<size_t>(row) * p.ldd;
#pragma unroll
      for (int e = 0; e < 32; ++e)
        if (col0 + e < p.n_store) drow[col0 + e] = __uint_as_float(r[e]) * p.alpha;
    } else if (p.out_mode == 2) {
      float* drow = static_cast<float*>(p.D) + static_cast<size_t>(row) * p.ldd;
#pragma unroll
      for (int e = 0; e < 32; ++e)
        if (col0 + e < p.n_store) atomicAdd(drow + col0 + e, __uint_as_float(r[e]) * p.alpha);
    } else if (p.out_mode == 3) {
      float* d = static_cast<float*>(p.D);
#pragma unroll
      for (int e = 0; e < 32; ++e)
        if (col0 + e < p.n_store)
          atomicAdd(d + static_cast<size_t>(col0 + e) * p.ldd + row, __uint_as_float(r[e]) * p.alpha);
    } else if (p.out_mode == 4) {
      float* drow = static_cast<float*>(p.D) + static_cast<size_t>(row) * p.ldd;
#pragma unroll
      for (int e = 0; e < 32; ++e)
        if (col0 + e < p.n_store) drow[col0 + e] += __uint_as_float(r[e]) * p.alpha;
    } else {
      float* d = static_cast<float*>(p.D);
#pragma unroll
      for (int e = 0; e < 32; ++e)
        if (col0 + e < p.n_store) d[static_cast<size_t>(col0 + e) * p.ldd + row] += __uint_as_float(r[e]) * p.alpha;
    }
}

// Issue the TMA copies that bring one operand tile (rows x 64 K) into shared memory.
//   K-major : one box [rows][64 k], coordinates (k0, row0)
//   MN-major: rows/64 boxes [64 k][64 mn], coordinates (mn0 + 64 j, k0), 8 KB apart
__device__ __forceinline__ void load_operand(uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int mn_major,
                                             int rows, int row0, int k0) {
  if (!mn_major) {
    tma_load_2d(dst, map, bar, k0, row0);
  } else {
    for (int j = 0; j < rows / 64; ++j) tma_load_2d(dst + j * 8192, map, bar, row0 + 64 * j, k0);
  }
}

// ======================================================================= host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D bf16 tensor map with 128-byte swizzle. inner = contiguous extent (elements).
static inline int make_map(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld_elems,
                    uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld_elems * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r) - 1000;
}

static inline int operand_map(CUtensorMap* map, const void* ptr, int mn_major, int rows_total, int k_total, int ld,
                       int tile_rows) {
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (ld % 8)) return -2;
  if (!mn_major) return make_map(map, ptr, k_total, rows_total, ld, kBK, tile_rows);
  return make_map(map, ptr, rows_total, k_total, ld, 64, kBK);
}



}  // namespace pm
