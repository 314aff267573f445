// Allocation-free entry point for split-KV paged attention.
//
// This entry point has no counterpart in the reference: the reference gathers its paged cache into a dense
// tensor and calls a library SDPA, so it has neither a split-KV scratch buffer nor a need to avoid allocating
// one. It exists here for callers that must not touch any allocator on the decode path (a serving loop inside
// a CUDA-graph capture, or an embedding host that owns all device memory).
//
// `pm_paged_attn_static` computes exactly what `pm_paged_attn` computes with n_split > 1, but keeps the per-slice
// partials in a file-scope `static __device__` array instead of caller-provided buffers. It performs no
// cudaMalloc / cudaFree and no framework allocation, in set-up or afterwards.
//
// Limits and rules
//   * n_split * total_q * hq  <=  PM_PAGED_STATIC_MAX_ROWS (4096 rows; 2 MiB + 32 KiB of device memory per GPU,
//     reserved when the library's module is loaded). Larger requests are rejected with PM_PAGED_STATIC_E_TOO_LARGE
//     before anything is launched; `pm_paged_attn_static_strerror` turns a code into text.
//   * The first call on a device looks up the scratch array's address (cudaGetSymbolAddress, result checked).
//     Make that first call before any stream capture begins; later calls only enqueue a memset and two kernels and
//     may be captured.
//   * The scratch is one buffer per device. Two calls that overlap in time on the same device (different streams,
//     or different host threads) race on it; serialise them on one stream or with events.
//   * The (max, sum) slots are cleared on every call, so rows that no sequence owns come out as zeros rather than
//     as whatever an earlier call left behind.
#pragma once
#include <cuda_runtime.h>

#define PM_PAGED_STATIC_MAX_ROWS 4096
#define PM_PAGED_STATIC_E_BAD_HEADS (-1)
#define PM_PAGED_STATIC_E_BAD_SPLIT (-2)
#define PM_PAGED_STATIC_E_TOO_LARGE (-3)
#define PM_PAGED_STATIC_E_DEVICE (-4)

#ifdef __cplusplus
extern "C" {
#endif

// q [total_q, hq, 128] bf16; k_cache/v_cache [num_blocks, 64, hkv, 128] bf16; out [total_q, hq, 128] bf16;
// block_table [num_seqs, max_blocks]; seq_lens, q_start, q_lens [num_seqs]. n_split >= 1.
// Returns 0, one of the PM_PAGED_STATIC_E_* codes, or a positive cudaError_t.
int pm_paged_attn_static(const void* q, const void* k_cache, const void* v_cache, void* out, const int* block_table,
                         const int* seq_lens, const int* q_start, const int* q_lens, int num_seqs, int max_blocks,
                         int total_q, int max_q, int hq, int hkv, int n_split, float scale, int window,
                         cudaStream_t stream);

// Largest n_split * total_q * hq this entry point accepts.
int pm_paged_attn_static_max_rows(void);

// Text for a return code of pm_paged_attn_static (static storage; never NULL).
const char* pm_paged_attn_static_strerror(int code);

#ifdef __cplusplus
}
#endif
