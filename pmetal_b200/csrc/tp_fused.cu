// Tensor-parallel linear layers fused with their collective, over NVLink peer memory (one launch per rank).
//
//   mode 0  all-gather -> GEMM (column-parallel):  Y[M, N_loc] = concat_r(X_r)[M, K] * W_loc[N_loc, K]^T
//           X is sharded by rows across ranks (sequence-parallel activations, M_r = M / world rows each, in
//           symmetric memory). The kernel starts on the tiles of its own shard at once; meanwhile four dedicated
//           warps of every CTA pull the remote shards, 128-row block by block, over NVLink into a local buffer with
//           16-byte peer loads and publish a per-block flag; the TMA producer reaches the remote row blocks last and
//           waits on those flags. Each remote byte crosses NVLink once (reading remote tiles directly would re-fetch
//           a row block once per column tile, since peer memory is not cached in the local L2), and the transfer
//           overlaps the MMAs of the local tiles.
//   mode 1  GEMM -> reduce-scatter (row-parallel): Y_r[M_r, N] = sum_q ( X_q[M, K_loc] * W_q[N, K_loc]^T )[rows of r]
//           Each rank computes all M rows of its partial product; the epilogue pushes every finished tile as bf16
//           straight into the owner's staging slot [parity][source rank] as 256-byte row segments (transposed through
//           shared memory so that a warp's peer stores are contiguous; remote owners first, own rows last); once
//           every rank has signalled, each rank sums the `world` slots of its rows in fixed rank order
//           (deterministic) and writes Y_r.
//
// This replaces the reference's all_to_sharded_forward / sharded_to_all_forward (an all_sum around a local matmul,
// crates/pmetal-distributed/src/tensor_parallel/sharded_linear.rs:41-106).
//
// GEMM core: persistent 128x256x64 tiles, warp 0 = TMA producer, warp 1 = tcgen05.mma issuer (accumulators
// double-buffered in TMEM), warps 2-5 = epilogue, warps 6-9 = stage-in of remote rows (mode 0). Cross-rank ordering
// uses epoch-valued flags in each rank's signal pad (system-scope release/acquire); every wait is bounded and reports
// through the status word. Plain peer loads/stores only: no multimem and no multicast loads.
#include "gemm_common.cuh"
#include "pmetal_b200.h"

namespace pm {

constexpr int kTpMaxRanks = 8;
constexpr int kTpBN = 256;
constexpr int kTpStages = 4;
constexpr int kTpThreads = 320;   // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue, warps 6-9 stage-in (mode 0)
constexpr int kStatusTpPeer = 106;

// signal pad words
constexpr int kTpReady = 0;     // [8] mode 0: rank r's X shard of this epoch is complete
constexpr int kTpDone = 8;      // [8] mode 0: rank r finished reading everyone's shard
constexpr int kTpPushed = 16;   // [8] mode 1: rank r finished pushing its partial tiles
constexpr int kTpEpoch = 24;    // local epoch counter
constexpr int kTpArrive = 25;   // local CTA arrival counter (phase 1)
constexpr int kTpArrive2 = 26;  // local CTA arrival counter (phase 2)

struct TpMaps {
  CUtensorMap a[2];   // mode 0: a[0] = local X shard, a[1] = gathered buffer [M, K]; mode 1: a[0] = local X
  CUtensorMap b;
};

__device__ __forceinline__ uint32_t tp_ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void tp_st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

struct TpParams {
  int mode, rank, world;
  int M, N, K;            // M = total rows (all ranks)
  int rows_per_rank;      // M / world, multiple of 128
  __nv_bfloat16* D;       // mode 0: Y [M, ldd]; mode 1: Y_r [rows_per_rank, ldd]
  int ldd;
  __nv_bfloat16* stage[kTpMaxRanks];   // mode 1: peer-mapped staging, [2][world][rows_per_rank][N] bf16 each
  uint32_t* pads[kTpMaxRanks];
  unsigned long long timeout_ns;
  int* status;
  // mode 0 stage-in: peers' shards (raw pointers, row stride ldx), the local gathered buffer [M, K] that the remote
  // tiles are read from, and one flag per 128-row block of it
  const __nv_bfloat16* x_peer[kTpMaxRanks];
  int ldx;
  __nv_bfloat16* gathered;
  uint32_t* blk_ready;
};

__device__ __forceinline__ uint32_t tp_ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void tp_st_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// bounded wait for *flag >= epoch (wrap-safe); false on expiry
__device__ __forceinline__ bool tp_wait_flag(const uint32_t* flag, uint32_t epoch, unsigned long long timeout_ns,
                                             int* status) {
  unsigned long long t0 = 0;     // the global timer is slow to read: first looked at after 1024 failed polls
  uint32_t spins = 0;
  while (static_cast<int32_t>(tp_ld_acquire(flag) - epoch) < 0) {
    if ((++spins & 31u) == 0u) {
      if (spins >= 1024u) {
        const unsigned long long now = globaltimer_ns();
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > timeout_ns) {
          atomicCAS(status, 0, kStatusTpPeer);
          return false;
        }
      }
      __nanosleep(64);
    }
  }
  return true;
}

// work item -> (rank whose rows these are, row block within that rank, column block)
__device__ __forceinline__ void tp_tile(const TpParams& p, int w, int n_tiles, int tpr, int* owner, int* mb, int* nb) {
  *nb = w % n_tiles;
  const int mseq = w / n_tiles;
  const int s = mseq / tpr;
  *mb = mseq % tpr;
  // mode 0: local shard first, then ring order; mode 1: remote owners first, own rows last
  *owner = (p.mode == 0) ? (p.rank + s) % p.world : (p.rank + 1 + s) % p.world;
}

__global__ void __launch_bounds__(kTpThreads, 1)
tp_gemm_kernel(const __grid_constant__ TpMaps maps, const TpParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int a_bytes = kBM * kBK * 2, b_bytes = kTpBN * kBK * 2, stage_bytes = a_bytes + b_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kTpStages * stage_bytes);
  uint64_t* empty_bar = full_bar + kTpStages;
  uint64_t* tfull_bar = empty_bar + kTpStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_last = const_cast<int*>(abort_flag) + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t* my_pad = p.pads[p.rank];
  const uint32_t epoch = my_pad[kTpEpoch] + 1;   // bumped by the last CTA at the very end of the launch

  if (threadIdx.x == 0) {
    for (int i = 0; i < kTpStages; ++i) {
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
    // mode 0: everything written to the local X shard by earlier kernels of this stream is complete; tell the peers
    if (p.mode == 0 && blockIdx.x == 0) {
      __threadfence_system();
      for (int r = 0; r < p.world; ++r) tp_st_release(p.pads[r] + kTpReady + p.rank, epoch);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tpr = p.rows_per_rank / kBM;
  const int n_tiles = (p.N + kTpBN - 1) / kTpBN;
  const int total = tpr * p.world * n_tiles;
  const int nk = (p.K + kBK - 1) / kBK;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
        int owner, mb, nb;
        tp_tile(p, w, n_tiles, tpr, &owner, &mb, &nb);
        const bool remote = p.mode == 0 && owner != p.rank;
        const CUtensorMap* ma = remote ? &maps.a[1] : &maps.a[0];
        const int m0 = (p.mode == 0) ? (remote ? owner * p.rows_per_rank + mb * kBM : mb * kBM) : (owner * tpr + mb) * kBM;
        if (remote) {   // the row block must have been copied into the gathered buffer (by some CTA's copy warps)
          const uint32_t* flag = p.blk_ready + owner * tpr + mb;
          unsigned long long t0 = 0;     // timer first read after 1024 failed polls (it is slow to read)
          uint32_t spins = 0;
          while (static_cast<int32_t>(tp_ld_acquire_gpu(flag) - epoch) < 0 && ok) {
            if ((++spins & 31u) == 0u) {
              bool late = false;
              if (spins >= 1024u) {
                const unsigned long long now = globaltimer_ns();
                if (t0 == 0) t0 = now;
                late = now - t0 > p.timeout_ns;
              }
              if (*abort_flag || late) {
                atomicCAS(p.status, 0, kStatusTpPeer);
                *abort_flag = 1;
                ok = false;
              }
              __nanosleep(64);
            }
          }
          if (!ok) break;
          // order the flag read (generic proxy) before the TMA reads of the copied rows (async proxy)
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kb = 0; kb < nk; ++kb, ++it) {
          const int s = it % kTpStages;
          if (!mbar_wait(&empty_bar[s], ((it / kTpStages) & 1) ^ 1, abort_flag, p.status, kTimeoutProducer)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * stage_bytes;
          mbar_expect_tx(&full_bar[s], stage_bytes);
          tma_load_2d(sa, ma, &full_bar[s], kb * kBK, m0);
          tma_load_2d(sa + a_bytes, &maps.b, &full_bar[s], kb * kBK, nb * kTpBN);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(kTpBN, 0, 0);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x, ++acc_it) {
        const int buf = acc_it & 1;
        if (!mbar_wait(&tempty_bar[buf], ((acc_it >> 1) & 1) ^ 1, abort_flag, p.status, kTimeoutMma)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * kTpBN;
        for (int kb = 0; kb < nk; ++kb, ++it) {
          const int s = it % kTpStages;
          if (!mbar_wait(&full_bar[s], (it / kTpStages) & 1, abort_flag, p.status, kTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * stage_bytes);
          const uint64_t da = make_smem_desc(sa, 16u, 1024u), db = make_smem_desc(sa + a_bytes, 16u, 1024u);
          const int rem = p.K - kb * kBK;
          const int nmma = min(4, (rem + 15) / 16);
          for (int j = 0; j < nmma; ++j)
            umma_f16(d_tmem, da + static_cast<uint64_t>(2 * j), db + static_cast<uint64_t>(2 * j), idesc,
                     (kb > 0 || j > 0) ? 1u : 0u);
          umma_commit(&empty_bar[s]);
        }
        if (ok) umma_commit(&tfull_bar[buf]);
      }
    }
  } else if (warp >= 6) {
    if (p.mode == 0 && p.world > 1) {
      // ---- stage-in: this CTA's share of the remote row blocks, pulled over NVLink by four dedicated warps while
      // the other warps run the tiles that are already local. Eight 16-byte loads per thread are in flight
      // (16 KB per CTA), enough to cover the link's round trip at full bandwidth.
      const int t128 = threadIdx.x - 192;
      const int vec_per_row = p.K / 8;
      bool copy_ok = true;
      for (int s = 1; s < p.world && copy_ok; ++s) {
        const int src = (p.rank + s) % p.world;
        if (t128 == 0 && !tp_wait_flag(my_pad + kTpReady + src, epoch, p.timeout_ns, p.status)) *abort_flag = 1;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*abort_flag) { copy_ok = false; break; }
        for (int b = 0; b < tpr; ++b) {
          if ((s * tpr + b) % static_cast<int>(gridDim.x) != static_cast<int>(blockIdx.x)) continue;
          const __nv_bfloat16* from = p.x_peer[src] + static_cast<long long>(b) * kBM * p.ldx;
          __nv_bfloat16* to = p.gathered + (static_cast<long long>(src) * p.rows_per_rank + b * kBM) * p.K;
          const int n_vec = kBM * vec_per_row;
          for (int i0 = t128; i0 < n_vec; i0 += 128 * 8) {
            uint4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int i = i0 + u * 128;
              if (i < n_vec) {
                const int r = i / vec_per_row, c = i - r * vec_per_row;
                v[u] = *reinterpret_cast<const uint4*>(from + static_cast<long long>(r) * p.ldx + c * 8);
              }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int i = i0 + u * 128;
              if (i < n_vec) *reinterpret_cast<uint4*>(to + static_cast<long long>(i) * 8) = v[u];
            }
          }
          __threadfence();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (t128 == 0) tp_st_release_gpu(p.blk_ready + src * tpr + b, epoch);
        }
      }
    }
  } else {
    const int q = warp & 3;
    uint32_t acc_it = 0;
    for (int w = blockIdx.x; w < total; w += gridDim.x, ++acc_it) {
      int owner, mb, nb;
      tp_tile(p, w, n_tiles, tpr, &owner, &mb, &nb);
      const int buf = acc_it & 1;
      if (!mbar_wait(&tfull_bar[buf], (acc_it >> 1) & 1, abort_flag, p.status, kTimeoutEpilogue)) break;
      tc_fence_after();
      const int lrow = mb * kBM + q * 32 + lane;     // row within the owner's shard
      if (p.mode == 1) {
        // Peer stores leave as full 256-byte row segments: each warp transposes its 32 x 128 half tile through a
        // swizzled shared-memory buffer (16-byte chunk index xor row, conflict-free both ways) and then writes two
        // rows per instruction, 16 lanes x 16 bytes each. Lane-per-row stores would reach NVLink as 16-byte pieces.
        uint4* stg = reinterpret_cast<uint4*>(smem + kTpStages * stage_bytes + 256) + q * (32 * 16);
        const long long slot0 =
            (static_cast<long long>(epoch & 1) * p.world + p.rank) * p.rows_per_rank + mb * kBM + q * 32;
        __nv_bfloat16* dbase = p.stage[owner] + slot0 * p.N + nb * kTpBN;
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
#pragma unroll 1
          for (int c4 = 0; c4 < 4; ++c4) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(tmem_base + buf * kTpBN + (half * 4 + c4) * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
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
          const int col = nb * kTpBN + half * 128 + ch * 8;
#pragma unroll 4
          for (int rr = 0; rr < 16; ++rr) {
            const int row = rr * 2 + (lane >> 4);
            const uint4 val = stg[row * 16 + (ch ^ (row & 15))];
            if (col + 8 <= p.N) *reinterpret_cast<uint4*>(dbase + static_cast<long long>(row) * p.N + half * 128 + ch * 8) = val;
          }
          __syncwarp();
        }
      } else {
      __nv_bfloat16* drow = p.D + (static_cast<long long>(owner) * p.rows_per_rank + lrow) * p.ldd;
#pragma unroll 1
      for (int c = 0; c < kTpBN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + buf * kTpBN + c * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
        tmem_ld_wait();
        const int col0 = nb * kTpBN + c * 32;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const int col = col0 + v * 8;
          if (col + 8 <= p.N) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[v * 8]), __uint_as_float(r[v * 8 + 1]));
            o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
            o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
            o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
            *reinterpret_cast<uint4*>(drow + col) = o;
          }
        }
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
    }
    if (p.mode == 1) __threadfence_system();   // this thread's peer stores are ordered before the flag below
  }

  // ---------------------------------------------------------------- phase boundary
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
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(my_pad + kTpArrive, 1u);
    if (prev == gridDim.x - 1) {
      // every CTA of this rank has finished its tiles (and, in mode 0, its reads of the peers' shards)
      my_pad[kTpArrive] = 0;
      __threadfence_system();
      const int off = (p.mode == 0) ? kTpDone : kTpPushed;
      for (int r = 0; r < p.world; ++r) tp_st_release(p.pads[r] + off + p.rank, epoch);
      *s_last = 1;
    }
  }
  __syncthreads();

  if (p.mode == 0) {
    // the last CTA keeps the launch alive until every peer has stopped reading this rank's shard, so that whatever
    // runs next on this stream may overwrite it
    if (*s_last && threadIdx.x < p.world) {
      if (!tp_wait_flag(my_pad + kTpDone + threadIdx.x, epoch, p.timeout_ns, p.status)) *abort_flag = 1;
    }
    __syncthreads();
    if (*s_last && threadIdx.x == 0) {
      __threadfence();
      my_pad[kTpEpoch] = epoch;
    }
    return;
  }

  // ---------------------------------------------------------------- mode 1, phase 2: sum the staged partials
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < p.world) {
    if (!tp_wait_flag(my_pad + kTpPushed + threadIdx.x, epoch, p.timeout_ns, p.status)) s_ok = 0;
  }
  __syncthreads();
  if (s_ok) {
    const long long per_slot = static_cast<long long>(p.rows_per_rank) * p.N;
    const __nv_bfloat16* base = p.stage[p.rank] + static_cast<long long>(epoch & 1) * p.world * per_slot;
    const int vec_per_row = p.N / 8;
    const long long n_vec = static_cast<long long>(p.rows_per_rank) * vec_per_row;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_vec;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < p.world; ++r) {
        const uint4 raw = *reinterpret_cast<const uint4*>(base + r * per_slot + i * 8);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h2[e]);
          acc[2 * e] += f.x;
          acc[2 * e + 1] += f.y;
        }
      }
      const long long row = i / vec_per_row;
      const int col = static_cast<int>(i - row * vec_per_row) * 8;
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(p.D + row * p.ldd + col) = o;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(my_pad + kTpArrive2, 1u);
    if (prev == gridDim.x - 1) {
      my_pad[kTpArrive2] = 0;
      __threadfence();
      my_pad[kTpEpoch] = epoch;
    }
  }
}


// ------------------------------------------------------------------------------------------ small all-reduce
// Sum of a bf16 vector over the ranks in one launch per rank, over peer memory: every rank stores its vector into slot
// `rank` of every peer's exchange buffer, the last of its CTAs to finish storing raises a flag on every peer, every CTA
// then waits (bounded) until all ranks' flags for this epoch have arrived in its own pad and sums the `world` slots
// of its share of the vector in fp32. The exchange buffer has two halves used by alternate epochs, so a rank that has
// moved on to the next call cannot overwrite slots a slower peer still reads; the epoch lives in the pad (advanced
// by the last CTA to finish), which keeps the launch replayable from a CUDA graph.
constexpr int kArFlag = 0;       // [2][8] epoch of the data in slot [half][src]
constexpr int kArEpoch = 16;     // local epoch counter
constexpr int kArStored = 17;    // CTAs of this launch that have finished their stores
constexpr int kArDone = 18;      // CTAs of this launch that have finished
constexpr int kStatusArPeer = 108;

struct ArParams {
  __nv_bfloat16* x;
  long long n;
  __nv_bfloat16* bufs[kTpMaxRanks];
  uint32_t* pads[kTpMaxRanks];
  long long slot_elems;
  int rank, world;
  unsigned long long timeout_ns;
  int* status;
};

__global__ void __launch_bounds__(256) peer_allreduce_kernel(const ArParams p) {
  __shared__ int s_fail;
  uint32_t* my_pad = p.pads[p.rank];
  const uint32_t epoch = my_pad[kArEpoch] + 1u;
  const int half = static_cast<int>(epoch & 1u);
  if (threadIdx.x == 0) s_fail = 0;
  const long long n8 = p.n / 8;
  const long long per = (n8 + gridDim.x - 1) / gridDim.x;
  const long long lo = blockIdx.x * per, hi = min(n8, lo + per);
  // ---- scatter this CTA's share of the local vector into slot `rank` of every rank's buffer
  for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const uint4 v = *reinterpret_cast<const uint4*>(p.x + i * 8);
    for (int r = 0; r < p.world; ++r) {
      const int dst = (p.rank + r) % p.world;      // start with the own buffer, then walk the ring
      __nv_bfloat16* slot = p.bufs[dst] + (static_cast<long long>(half) * p.world + p.rank) * p.slot_elems;
      *reinterpret_cast<uint4*>(slot + i * 8) = v;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(my_pad + kArStored, 1u);
    if (prev == gridDim.x - 1) {           // all of this rank's stores are out: tell every rank
      __threadfence_system();
      for (int r = 0; r < p.world; ++r) tp_st_release(p.pads[r] + kArFlag + half * 8 + p.rank, epoch);
    }
  }
  // ---- wait for every rank's slot of this epoch
  if (threadIdx.x < p.world) {
    if (!tp_wait_flag(my_pad + kArFlag + half * 8 + threadIdx.x, epoch, p.timeout_ns, p.status)) s_fail = 1;
  }
  __syncthreads();
  if (!s_fail) {
    const __nv_bfloat16* mine = p.bufs[p.rank] + static_cast<long long>(half) * p.world * p.slot_elems;
    for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < p.world; ++r) {
        const uint4 v = *reinterpret_cast<const uint4*>(mine + r * p.slot_elems + i * 8);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          acc[2 * e] += __uint_as_float(w[e] << 16);
          acc[2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
        }
      }
      uint4 o;
      *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(acc[0], acc[1]);
      *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(acc[2], acc[3]);
      *reinterpret_cast<__nv_bfloat162*>(&o.z) = __floats2bfloat162_rn(acc[4], acc[5]);
      *reinterpret_cast<__nv_bfloat162*>(&o.w) = __floats2bfloat162_rn(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(p.x + i * 8) = o;
    }
  }
  // ---- the last CTA to finish closes the epoch (also after an abandoned wait, so the pad stays consistent)
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(my_pad + kArDone, 1u);
    if (prev == gridDim.x - 1) {
      my_pad[kArStored] = 0u;
      my_pad[kArDone] = 0u;
      my_pad[kArEpoch] = epoch;
      __threadfence_system();
    }
  }
}

}  // namespace pm

using namespace pm;

// mode 0: x_ptrs[r] = rank r's X shard [rows_per_rank, K] (ldx), w = W_loc [N, K] (ldw), out = Y [M, ldd].
// mode 1: x_ptrs[rank] = local X [M, K] (ldx), w = W_loc [N, K], stage_ptrs[r] = rank r's staging buffer,
//         out = Y_r [rows_per_rank, ldd]. K and N are the local extents. mode 0 also takes `gathered` (local bf16
//         [M, K] scratch) and `blk_ready` (uint32 [M / 128], zero-initialised once). Returns 0, a negative argument
//         error, or a CUDA error code.
extern "C" int pm_tp_gemm(int mode, const unsigned long long* x_ptrs, int ldx, const void* w, int ldw, void* out,
                          int ldd, const unsigned long long* stage_ptrs, const unsigned long long* pad_ptrs, int rank,
                          int world, int M, int N, int K, void* gathered, void* blk_ready, double timeout_s, int max_ctas,
                          int* status, cudaStream_t stream) {
  if (mode != 0 && mode != 1) return -1;
  if (world < 1 || world > kTpMaxRanks || rank < 0 || rank >= world) return -2;
  if (M <= 0 || N <= 0 || K <= 0 || M % world || (M / world) % kBM) return -3;
  if ((N % 8) || (ldd % 8) || (reinterpret_cast<uintptr_t>(out) & 15)) return -4;
  TpMaps maps;
  TpParams p{};
  p.mode = mode; p.rank = rank; p.world = world; p.M = M; p.N = N; p.K = K; p.rows_per_rank = M / world;
  p.D = static_cast<__nv_bfloat16*>(out); p.ldd = ldd;
  p.timeout_ns = static_cast<unsigned long long>(timeout_s * 1e9);
  p.status = status;
  int rc;
  for (int r = 0; r < kTpMaxRanks; ++r) {
    const int rr = r < world ? r : rank;
    p.pads[r] = reinterpret_cast<uint32_t*>(pad_ptrs[rr]);
    p.stage[r] = (mode == 1) ? reinterpret_cast<__nv_bfloat16*>(stage_ptrs[rr]) : nullptr;
    p.x_peer[r] = reinterpret_cast<const __nv_bfloat16*>(x_ptrs[rr]);
  }
  p.ldx = ldx;
  p.gathered = static_cast<__nv_bfloat16*>(gathered);
  p.blk_ready = static_cast<uint32_t*>(blk_ready);
  if (mode == 0 && world > 1 && (!gathered || !blk_ready || (K % 8))) return -7;
  if ((rc = operand_map(&maps.a[0], reinterpret_cast<const void*>(x_ptrs[rank]), 0, mode == 0 ? p.rows_per_rank : M, K, ldx,
                        kBM)))
    return rc * 10 - 5;
  maps.a[1] = maps.a[0];
  if (mode == 0 && world > 1 && (rc = operand_map(&maps.a[1], gathered, 0, M, K, K, kBM))) return rc * 10 - 5;
  if ((rc = operand_map(&maps.b, w, 0, N, K, ldw, kTpBN))) return rc * 10 - 6;
  // operand stages, 256 bytes of barriers, 32 KB epilogue transpose buffer (4 warps x 32 rows x 256 B), alignment slack
  const size_t smem = static_cast<size_t>(kTpStages) * (kBM * kBK * 2 + kTpBN * kBK * 2) + 256 + 4 * 32 * 256 + 1024;
  static DeviceOnce configured;
  if (configured.pending()) {
    cudaError_t e = cudaFuncSetAttribute(tp_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured.mark();
  }
  const int total = (M / kBM) * ((N + kTpBN - 1) / kTpBN);
  int grid = total;
  const int cap = max_ctas > 0 ? max_ctas : num_sms();
  if (grid > cap) grid = cap;
  tp_gemm_kernel<<<grid, kTpThreads, smem, stream>>>(maps, p);
  return static_cast<int>(cudaGetLastError());
}

// x: bf16 [n] (n a multiple of 8, at most slot_elems), summed in place over the ranks. bufs[r] / pads[r]: rank r's
// exchange buffer (2 * world * slot_elems bf16) and signal pad (64 uint32, zero-initialised once), peer-mapped.
extern "C" int pm_peer_allreduce(void* x, long long n, const unsigned long long* bufs, const unsigned long long* pads,
                                 long long slot_elems, int rank, int world, double timeout_s, int* status,
                                 cudaStream_t st) {
  if (world < 1 || world > kTpMaxRanks || rank < 0 || rank >= world) return -1;
  if (n <= 0 || (n % 8) || n > slot_elems || (slot_elems % 8)) return -2;
  ArParams p{};
  p.x = static_cast<__nv_bfloat16*>(x);
  p.n = n;
  for (int r = 0; r < kTpMaxRanks; ++r) {
    const int rr = r < world ? r : rank;
    p.bufs[r] = reinterpret_cast<__nv_bfloat16*>(bufs[rr]);
    p.pads[r] = reinterpret_cast<uint32_t*>(pads[rr]);
  }
  p.slot_elems = slot_elems; p.rank = rank; p.world = world;
  p.timeout_ns = static_cast<unsigned long long>(timeout_s * 1e9);
  p.status = status;
  int grid = static_cast<int>((n / 8 + 2047) / 2048);     // about 8 x 16 bytes per thread
  if (grid < 1) grid = 1;
  if (grid > 32) grid = 32;                               // every CTA must be resident: they wait on each other's flag
  peer_allreduce_kernel<<<grid, 256, 0, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}
