// Grouped expert GEMMs for mixture-of-experts layers, with expert-parallel dispatch and combine fused in.
//
// Every rank holds E_loc = E / world experts and T_loc tokens. After local routing the (token, slot) rows are sorted
// by expert into `sorted_x` (symmetric memory) with `offsets[E+1]` (symmetric memory as well). Then, per rank:
//
//   ep_prepare_kernel   publishes "my sorted tokens and offsets are ready", waits for every peer's flag (bounded),
//                       reads the peers' offsets and builds the tile list: for every local expert the rows routed to
//                       it by all ranks are concatenated (own rows first) and cut into 128-row tiles, so a tile may
//                       hold rows of several source ranks ("runs"). With few tokens per expert (decode, or many
//                       ranks) this streams each expert's weights through the SMs once instead of once per source.
//   moe_gemm_kernel #1  gate/up projection with the dispatch all-to-all inside: four dedicated warps of every CTA pull
//                       their share of the tiles' token rows out of the *source ranks'* sorted buffers (16-byte
//                       peer loads over NVLink, eight in flight per thread) into a local staging buffer and publish a flag per
//                       tile; the TMA producer waits on a tile's flag before loading it. Every token row crosses
//                       NVLink once (peer memory is not cached in the local L2, so reading remote rows in place would
//                       re-fetch them once per column block). The epilogue applies SwiGLU, writing h locally.
//   moe_gemm_kernel #2  down projection on h; the epilogue stores every output row straight into the *source rank's*
//                       result buffer at the row's sorted position (256-byte row segments, transposed through shared
//                       memory so that a warp's peer stores are contiguous; destination looked up in the tile's
//                       runs) -- this is the combine all-to-all. The launch ends only after every peer has signalled that its pushes are complete,
//                       so the local weighted combine that follows on the stream sees all rows.
//
// With world = 1 the same kernels are the local grouped GEMM. This replaces the reference's per-destination
// send/recv dispatcher (crates/pmetal-distributed/src/expert_parallel/dispatch.rs:66-214) and its grouped-GEMM Metal
// kernels (crates/pmetal-metal/src/kernels/metal/grouped_gemm.metal:125-465, fused_moe.metal).
//
// GEMM core: persistent 128x256x64 tcgen05 tiles over a device-side tile list (warp 0 TMA, warp 1 MMA, warps 2-5
// epilogue, warps 6-9 dispatch stage-in, TMEM double-buffered). Gate/up weights are stored per expert in blocks of 256 rows: 128 gate rows followed
// by the matching 128 up rows, so one accumulator tile holds both halves of 128 outputs.
// All cross-rank waits are bounded and report through the status word; plain peer loads/stores only.
#include "gemm_common.cuh"
#include "pmetal_b200.h"

namespace pm {

constexpr int kEpMaxRanks = 8;
constexpr int kEpBN = 256;
constexpr int kEpStages = 4;
constexpr int kEpThreads = 320;   // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue, warps 6-9 dispatch stage-in
constexpr int kStatusEpPeer = 107;

constexpr int kEpReady = 0;     // [8] rank r's sorted tokens + offsets of this epoch are published
constexpr int kEpPushed = 8;    // [8] rank r has stored all its down-projection rows
constexpr int kEpEpoch = 16;    // local epoch (bumped by ep_prepare_kernel)
constexpr int kEpArrive = 17;   // local CTA arrival counter

struct MoeTile {
  int a_row0;     // first row of the tile in the local staging / hidden buffers (128 rows reserved)
  int rows;       // valid rows (<= 128)
  int expert;     // local expert index (selects the weight rows)
  int run0;       // first entry of this tile in the run list
  int nruns;      // number of runs (<= world)
  int pad[3];
};

struct MoeRun {
  int src;        // rank whose sorted buffer holds the rows (and receives the results)
  int src_row0;   // first row there
  int tile_row0;  // first row inside the tile
  int rows;
};

struct MoeMaps {
  CUtensorMap a;      // local A buffer: staged-in token rows (gate/up) or the hidden rows (down)
  CUtensorMap b;      // stacked weights [E_loc * n_per_expert, K]
};

struct MoeGemmParams {
  const MoeTile* tiles;
  const MoeRun* runs;
  const int* n_tiles;
  int N, K;                 // per-expert output rows of the weight (2*I for gate/up, H for down) and reduction size
  int swiglu;               // 1: out[:, j] = silu(acc[:, j]) * acc[:, j + 128] per 256 block, output width N / 2
  __nv_bfloat16* out[kEpMaxRanks];   // push = 0: out[rank] is the local output; push = 1: every rank's result buffer
  int ldd;
  int push;                 // 1: output rows go to their source ranks' buffers at the rows' sorted positions
  int rank, world;
  int signal_pushed;        // 1: set pushed[rank] on all peers at the end and wait for all peers' flags
  uint32_t* pads[kEpMaxRanks];
  unsigned long long timeout_ns;
  int* status;
  // stage-in (gate/up launch): peers' sorted token buffers, the local staging buffer the A map covers, per-tile flags
  int stage_in;
  const __nv_bfloat16* x_peer[kEpMaxRanks];
  __nv_bfloat16* xin;
  uint32_t* tile_ready;
};

__device__ __forceinline__ uint32_t ep_ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void ep_st_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ bool ep_wait_flag(const uint32_t* flag, uint32_t epoch, unsigned long long timeout_ns,
                                             int* status) {
  unsigned long long t0 = 0;     // the global timer is slow to read: first looked at after 1024 failed polls
  uint32_t spins = 0;
  while (static_cast<int32_t>(ep_ld_acquire(flag) - epoch) < 0) {
    if ((++spins & 31u) == 0u) {
      if (spins >= 1024u) {
        const unsigned long long now = globaltimer_ns();
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > timeout_ns) {
          atomicCAS(status, 0, kStatusEpPeer);
          return false;
        }
      }
      __nanosleep(64);
    }
  }
  return true;
}

// One CTA. offsets[r] points at rank r's [E+1] expert offsets into its sorted token buffer. Writes the tile list and
// the run list; counts_out[0] = number of tiles, counts_out[1] = buffer rows used (128 per tile).
struct EpPtrs {                  // passed by value, so the launch needs no staging copy and can be captured in a graph
  const int* offsets[kEpMaxRanks];
  uint32_t* pads[kEpMaxRanks];
};

constexpr int kEpMaxLocal = 512;     // local experts per rank
constexpr int kStatusEpOverflow = 108;

__global__ void ep_prepare_kernel(const EpPtrs ptrs, int rank, int world, int e_loc, MoeTile* tiles, MoeRun* runs,
                                  int max_tiles, int max_runs, int* counts_out, unsigned long long timeout_ns,
                                  int* status) {
  __shared__ int s_ok;
  __shared__ int s_off[kEpMaxRanks][kEpMaxLocal + 1];
  uint32_t* const* pads = ptrs.pads;
  uint32_t* my_pad = pads[rank];
  const uint32_t epoch = my_pad[kEpEpoch] + 1;
  if (threadIdx.x == 0) {
    s_ok = 1;
    __threadfence_system();
    for (int r = 0; r < world; ++r) ep_st_release(pads[r] + kEpReady + rank, epoch);
  }
  __syncthreads();
  if (threadIdx.x < world) {
    if (!ep_wait_flag(my_pad + kEpReady + threadIdx.x, epoch, timeout_ns, status)) s_ok = 0;
  }
  __syncthreads();
  if (s_ok) {   // all peers' offsets in parallel: a serial scan over peer memory would pay the NVLink latency per load
    for (int i = threadIdx.x; i < world * (e_loc + 1); i += blockDim.x) {
      const int s = i / (e_loc + 1), e = i % (e_loc + 1);
      s_off[s][e] = ptrs.offsets[(rank + s) % world][rank * e_loc + e];
    }
  }
  __syncthreads();
  // one thread per local expert: count its tiles and runs, scan, then write them at the expert's offsets
  __shared__ int s_tiles[kEpMaxLocal], s_runs[kEpMaxLocal];
  auto walk = [&](int e, int n, int nr, bool write) {
    MoeTile cur{};
    int filled = kBM, tiles_e = 0, runs_e = 0;
    for (int s = 0; s < world; ++s) {
      const int src = (rank + s) % world;    // own tokens first
      int lo = s_off[s][e];
      const int hi = s_off[s][e + 1];
      while (lo < hi) {
        if (filled == kBM) {
          if (write && tiles_e > 0) tiles[n + tiles_e - 1] = cur;
          cur = MoeTile{};
          cur.a_row0 = (n + tiles_e) * kBM;
          cur.expert = e;
          cur.run0 = nr + runs_e;
          filled = 0;
          ++tiles_e;
        }
        const int take = min(hi - lo, kBM - filled);
        if (write) runs[nr + runs_e] = MoeRun{src, lo, filled, take};
        ++runs_e;
        cur.rows += take;
        cur.nruns += 1;
        filled += take;
        lo += take;
      }
    }
    if (write && tiles_e > 0) tiles[n + tiles_e - 1] = cur;
    if (!write) {
      s_tiles[e] = tiles_e;
      s_runs[e] = runs_e;
    }
  };
  for (int e = threadIdx.x; e < e_loc; e += blockDim.x) {
    if (s_ok) {
      walk(e, 0, 0, false);
    } else {
      s_tiles[e] = 0;
      s_runs[e] = 0;
    }
  }
  __syncthreads();
  for (int off = 1; off < e_loc; off <<= 1) {       // inclusive scan over the local experts
    int t[2] = {0, 0}, r[2] = {0, 0};
    for (int j = 0, e = threadIdx.x; e < e_loc && j < 2; e += blockDim.x, ++j)
      if (e >= off) {
        t[j] = s_tiles[e - off];
        r[j] = s_runs[e - off];
      }
    __syncthreads();
    for (int j = 0, e = threadIdx.x; e < e_loc && j < 2; e += blockDim.x, ++j) {
      s_tiles[e] += t[j];
      s_runs[e] += r[j];
    }
    __syncthreads();
  }
  const int n_total = s_tiles[e_loc - 1], r_total = s_runs[e_loc - 1];
  const bool overflow = n_total > max_tiles || r_total > max_runs;
  if (!overflow && s_ok)
    for (int e = threadIdx.x; e < e_loc; e += blockDim.x)
      walk(e, e ? s_tiles[e - 1] : 0, e ? s_runs[e - 1] : 0, true);
  __syncthreads();
  if (threadIdx.x == 0) {
    if (overflow) atomicCAS(status, 0, kStatusEpOverflow);
    counts_out[0] = overflow ? 0 : n_total;
    counts_out[1] = n_total * kBM;
    __threadfence();
    my_pad[kEpEpoch] = epoch;
  }
}

__global__ void __launch_bounds__(kEpThreads, 1)
moe_gemm_kernel(const __grid_constant__ MoeMaps maps, const MoeGemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int a_bytes = kBM * kBK * 2, b_bytes = kEpBN * kBK * 2, stage_bytes = a_bytes + b_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kEpStages * stage_bytes);
  uint64_t* empty_bar = full_bar + kEpStages;
  uint64_t* tfull_bar = empty_bar + kEpStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_last = const_cast<int*>(abort_flag) + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t* my_pad = p.pads[p.rank];
  const uint32_t epoch = my_pad[kEpEpoch];   // ep_prepare_kernel already advanced it for this layer call

  if (threadIdx.x == 0) {
    for (int i = 0; i < kEpStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 4);
    }
    *abort_flag = 0;
    *s_last = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int n_blocks = (p.N + kEpBN - 1) / kEpBN;
  const int total = *p.n_tiles * n_blocks;
  const int nk = (p.K + kBK - 1) / kBK;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
        const MoeTile t = p.tiles[w / n_blocks];
        const int nb = w % n_blocks;
        const int b_row = t.expert * p.N + nb * kEpBN;
        if (p.stage_in) {   // the tile's rows must have landed in the staging buffer
          const uint32_t* flag = p.tile_ready + w / n_blocks;
          unsigned long long t0 = 0;     // timer first read after 1024 failed polls (it is slow to read)
          uint32_t spins = 0, v;
          do {
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            if (static_cast<int32_t>(v - epoch) >= 0) break;
            if ((++spins & 31u) == 0u) {
              bool late = false;
              if (spins >= 1024u) {
                const unsigned long long now = globaltimer_ns();
                if (t0 == 0) t0 = now;
                late = now - t0 > p.timeout_ns;
              }
              if (*abort_flag || late) {
                atomicCAS(p.status, 0, kStatusEpPeer);
                *abort_flag = 1;
                ok = false;
              }
              __nanosleep(64);
            }
          } while (ok);
          if (!ok) break;
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kb = 0; kb < nk; ++kb, ++it) {
          const int s = it % kEpStages;
          if (!mbar_wait(&empty_bar[s], ((it / kEpStages) & 1) ^ 1, abort_flag, p.status, kTimeoutProducer)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * stage_bytes;
          mbar_expect_tx(&full_bar[s], stage_bytes);
          tma_load_2d(sa, &maps.a, &full_bar[s], kb * kBK, t.a_row0);
          tma_load_2d(sa + a_bytes, &maps.b, &full_bar[s], kb * kBK, b_row);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(kEpBN, 0, 0);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x, ++acc_it) {
        const int buf = acc_it & 1;
        if (!mbar_wait(&tempty_bar[buf], ((acc_it >> 1) & 1) ^ 1, abort_flag, p.status, kTimeoutMma)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * kEpBN;
        for (int kb = 0; kb < nk; ++kb, ++it) {
          const int s = it % kEpStages;
          if (!mbar_wait(&full_bar[s], (it / kEpStages) & 1, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * stage_bytes);
          const uint64_t da = make_smem_desc(sa, 16u, 1024u), db = make_smem_desc(sa + a_bytes, 16u, 1024u);
          const int nmma = min(4, (p.K - kb * kBK + 15) / 16);
          for (int j = 0; j < nmma; ++j)
            umma_f16(d_tmem, da + static_cast<uint64_t>(2 * j), db + static_cast<uint64_t>(2 * j), idesc,
                     (kb > 0 || j > 0) ? 1u : 0u);
          umma_commit(&empty_bar[s]);
        }
        if (ok) umma_commit(&tfull_bar[buf]);
      }
    }
  } else if (warp >= 6) {
    if (p.stage_in) {
      // ---- dispatch: four dedicated warps copy this CTA's share of the tiles' rows from their source ranks into the
      // staging buffer while the other warps work on tiles that have landed; eight 16-byte loads per thread in flight
      const int t128 = threadIdx.x - 192;
      const int vec_per_row = p.K / 8;
      const int n_t = *p.n_tiles;
      for (int ti = blockIdx.x; ti < n_t; ti += gridDim.x) {
        const MoeTile t = p.tiles[ti];
        for (int ri = 0; ri < t.nruns; ++ri) {
          const MoeRun rn = p.runs[t.run0 + ri];
          const __nv_bfloat16* from = p.x_peer[rn.src] + static_cast<long long>(rn.src_row0) * p.K;
          __nv_bfloat16* to = p.xin + static_cast<long long>(t.a_row0 + rn.tile_row0) * p.K;
          const int n_vec = rn.rows * vec_per_row;
          for (int i0 = t128; i0 < n_vec; i0 += 128 * 8) {
            uint4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
              if (i0 + u * 128 < n_vec) v[u] = reinterpret_cast<const uint4*>(from)[i0 + u * 128];
#pragma unroll
            for (int u = 0; u < 8; ++u)
              if (i0 + u * 128 < n_vec) reinterpret_cast<uint4*>(to)[i0 + u * 128] = v[u];
          }
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (t128 == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.tile_ready + ti), "r"(epoch) : "memory");
      }
    }
  } else {
    const int q = warp & 3;
    uint32_t acc_it = 0;
    for (int w = blockIdx.x; w < total; w += gridDim.x, ++acc_it) {
      const MoeTile t = p.tiles[w / n_blocks];
      const int nb = w % n_blocks;
      const int buf = acc_it & 1;
      if (!mbar_wait(&tfull_bar[buf], (acc_it >> 1) & 1, abort_flag, p.status, kTimeoutEpilogue)) break;
      tc_fence_after();
      const int lrow = q * 32 + lane;
      const bool row_ok = lrow < t.rows;
      __nv_bfloat16* drow = p.out[p.rank] + static_cast<long long>(t.a_row0 + lrow) * p.ldd;
      if (p.push && row_ok) {       // the row's source rank and sorted position there
        for (int ri = 0; ri < t.nruns; ++ri) {
          const MoeRun rn = p.runs[t.run0 + ri];
          if (lrow >= rn.tile_row0 && lrow < rn.tile_row0 + rn.rows) {
            drow = p.out[rn.src] + static_cast<long long>(rn.src_row0 + lrow - rn.tile_row0) * p.ldd;
            break;
          }
        }
      }
      const uint32_t tbase = tmem_base + buf * kEpBN + (static_cast<uint32_t>(q * 32) << 16);
      if (p.swiglu) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t g[32], u[32];
          tmem_ld_32x32b_x32(tbase + c * 32, g);
          tmem_ld_32x32b_x32(tbase + 128 + c * 32, u);
          tmem_ld_wait();
          const int col0 = nb * 128 + c * 32;
          if (!row_ok) continue;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int col = col0 + v * 8;
            if (col + 8 > p.N / 2) continue;
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float gv = __uint_as_float(g[v * 8 + e]);
              f[e] = gv / (1.f + __expf(-gv)) * __uint_as_float(u[v * 8 + e]);
            }
            uint4 o;
            o.x = pack_bf16x2(f[0], f[1]);
            o.y = pack_bf16x2(f[2], f[3]);
            o.z = pack_bf16x2(f[4], f[5]);
            o.w = pack_bf16x2(f[6], f[7]);
            *reinterpret_cast<uint4*>(drow + col) = o;
          }
        }
      } else if (p.push) {
        // Rows leave for their source ranks as 256-byte segments: the warp transposes its 32 x 128 half tile through a
        // swizzled shared-memory buffer and writes two rows per instruction (16 lanes x 16 bytes each); each row's
        // destination comes from the lane that owns the row.
        uint4* stg = reinterpret_cast<uint4*>(smem + kEpStages * stage_bytes + 256) + q * (32 * 16);
        const unsigned long long dptr = row_ok ? reinterpret_cast<unsigned long long>(drow) : 0ull;
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
#pragma unroll 1
          for (int c4 = 0; c4 < 4; ++c4) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(tbase + (half * 4 + c4) * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[v * 8]), __uint_as_float(r[v * 8 + 1]));
              o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
              o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
              o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
              stg[lane * 16 + ((c4 * 4 + v) ^ (lane & 15))] = o;
            }
          }
          __syncwarp();
          const int ch = lane & 15;
          const int col = nb * kEpBN + half * 128 + ch * 8;
#pragma unroll 4
          for (int rr = 0; rr < 16; ++rr) {
            const int row = rr * 2 + (lane >> 4);
            const unsigned long long dp = __shfl_sync(0xffffffffu, dptr, row);
            const uint4 val = stg[row * 16 + (ch ^ (row & 15))];
            if (dp != 0ull && col + 8 <= p.N) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dp) + col) = val;
          }
          __syncwarp();
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < kEpBN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tbase + c * 32, r);
          tmem_ld_wait();
          const int col0 = nb * kEpBN + c * 32;
          if (!row_ok) continue;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int col = col0 + v * 8;
            if (col + 8 > p.N) continue;
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[v * 8]), __uint_as_float(r[v * 8 + 1]));
            o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
            o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
            o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
            *reinterpret_cast<uint4*>(drow + col) = o;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
    }
    if (p.signal_pushed) __threadfence_system();
  }

  __syncwarp();
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (!p.signal_pushed) return;
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(my_pad + kEpArrive, 1u);
    if (prev == gridDim.x - 1) {
      my_pad[kEpArrive] = 0;
      __threadfence_system();
      for (int r = 0; r < p.world; ++r) ep_st_release(p.pads[r] + kEpPushed + p.rank, epoch);
      *s_last = 1;
    }
  }
  __syncthreads();
  // the last CTA keeps the launch alive until every peer's rows have landed in this rank's result buffer
  if (*s_last && threadIdx.x < p.world)
    ep_wait_flag(my_pad + kEpPushed + threadIdx.x, epoch, p.timeout_ns, p.status);
}

}  // namespace pm

using namespace pm;

extern "C" int pm_ep_prepare(const unsigned long long* offset_ptrs, const unsigned long long* pad_ptrs, int rank,
                             int world, int e_loc, void* tiles, void* runs, int max_tiles, int max_runs, int* counts_out,
                             double timeout_s, int* status, cudaStream_t st) {
  if (world < 1 || world > kEpMaxRanks || rank < 0 || rank >= world || e_loc < 1 || e_loc > kEpMaxLocal) return -1;
  EpPtrs ptrs;
  for (int r = 0; r < kEpMaxRanks; ++r) {
    ptrs.offsets[r] = reinterpret_cast<const int*>(offset_ptrs[r < world ? r : rank]);
    ptrs.pads[r] = reinterpret_cast<uint32_t*>(pad_ptrs[r < world ? r : rank]);
  }
  ep_prepare_kernel<<<1, 256, 0, st>>>(ptrs, rank, world, e_loc, static_cast<MoeTile*>(tiles), static_cast<MoeRun*>(runs),
                                       max_tiles, max_runs, counts_out, static_cast<unsigned long long>(timeout_s * 1e9),
                                       status);
  return static_cast<int>(cudaGetLastError());
}

// a: local A buffer [a_rows, K] (row stride lda): the staging buffer of the gate/up launch or the hidden rows of the
// down launch; w: [e_loc * N, K]; out_ptrs[r]: output base of rank r (push = 0 uses out_ptrs[rank] only).
// copy_src_ptrs (gate/up launch): rank r's sorted token buffer [*, K] (row stride K) that tiles are staged in from;
// tile_ready: uint32 [max_tiles], zero-initialised once. Both null for the down projection.
extern "C" int pm_moe_gemm(const void* a, int a_rows, int lda, const void* w, int ldw, int e_loc,
                           const unsigned long long* out_ptrs, int ldd, const void* tiles, const void* runs,
                           const int* n_tiles, int max_tiles, int N, int K, int swiglu, int rank, int world, int push,
                           const unsigned long long* pad_ptrs, const unsigned long long* copy_src_ptrs, void* tile_ready,
                           double timeout_s, int* status, cudaStream_t st) {
  if (world < 1 || world > kEpMaxRanks || rank < 0 || rank >= world) return -1;
  if (N <= 0 || K <= 0 || (N % 8) || (ldd % 8) || (swiglu && (N % 256))) return -2;
  MoeMaps maps;
  MoeGemmParams p{};
  int rc;
  if ((rc = operand_map(&maps.a, a, 0, a_rows, K, lda, kBM))) return rc * 10 - 5;
  for (int r = 0; r < kEpMaxRanks; ++r) {
    const int rr = r < world ? r : rank;
    p.out[r] = reinterpret_cast<__nv_bfloat16*>(out_ptrs[rr]);
    p.pads[r] = reinterpret_cast<uint32_t*>(pad_ptrs[rr]);
  }
  if ((rc = operand_map(&maps.b, w, 0, e_loc * N, K, ldw, kEpBN))) return rc * 10 - 6;
  p.tiles = static_cast<const MoeTile*>(tiles);
  p.runs = static_cast<const MoeRun*>(runs);
  p.n_tiles = n_tiles;
  p.N = N; p.K = K; p.swiglu = swiglu; p.ldd = ldd; p.rank = rank; p.world = world;
  p.push = push;
  p.signal_pushed = push;
  p.stage_in = copy_src_ptrs != nullptr;
  if (p.stage_in) {
    if (!tile_ready || (K % 8)) return -3;
    for (int r = 0; r < kEpMaxRanks; ++r)
      p.x_peer[r] = reinterpret_cast<const __nv_bfloat16*>(copy_src_ptrs[r < world ? r : rank]);
    p.xin = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(a));
    p.tile_ready = static_cast<uint32_t*>(tile_ready);
  }
  p.timeout_ns = static_cast<unsigned long long>(timeout_s * 1e9);
  p.status = status;
  // operand stages, 256 bytes of barriers, 32 KB epilogue transpose buffer (4 warps x 32 rows x 256 B), alignment slack
  const size_t smem = static_cast<size_t>(kEpStages) * (kBM * kBK * 2 + kEpBN * kBK * 2) + 256 + 4 * 32 * 256 + 1024;
  static DeviceOnce configured;
  if (configured.pending()) {
    cudaError_t e = cudaFuncSetAttribute(moe_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured.mark();
  }
  const long long work = static_cast<long long>(max_tiles) * ((N + kEpBN - 1) / kEpBN);
  int grid = num_sms();
  if (work < grid) grid = static_cast<int>(work < 1 ? 1 : work);
  moe_gemm_kernel<<<grid, kEpThreads, smem, st>>>(maps, p);
  return static_cast<int>(cudaGetLastError());
}
