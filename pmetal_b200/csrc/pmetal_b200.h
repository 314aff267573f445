// C interface of libpmetal_b200.so: every launcher of the sm_100a kernel library.
//
// All functions take raw device pointers and a CUDA stream, allocate nothing unless their comment says so, and return
// 0 on success, a negative value for an argument or descriptor error, or the CUDA error code of the launch. `status`
// arguments point at a device int that a kernel sets when one of its bounded waits runs out (codes 101-109); the
// caller reads it after synchronising the stream. Pointers and the stream must belong to the current device.
// The no-allocation paged-attention entry point is declared in paged_attn_static.h.
//
// This file is written by pmetal_b200/build.py from the definitions in csrc/*.cu; every source includes it, so a
// declaration that drifts from its definition fails to compile.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---------------------------------------------------------------- attention.cu
// q:[T,hq,128] k:[T,hkv,128] v:[T,hkv,128] with per-token strides; out:[T,hq,128]; lse:[hq,T]
int pm_attn_fwd(const void* q, long long q_stride, const void* k, long long k_stride, const void* v, long long
    v_stride, void* out, long long o_stride, float* lse, const int* seq_start, int T, int hq, int hkv, float scale,
    int window, cudaStream_t st);
// dq:[T,hq,128] dk,dv:[T,hkv,128] (strided). delta:[hq,T] = rowsum(dO*O) computed beforehand.
int pm_attn_bwd(const void* dout, const void* q, long long q_stride, const void* k, long long k_stride, const void*
    v, long long v_stride, long long o_stride, const float* lse, const float* delta, void* dq, long long dq_stride,
    void* dk, long long dk_stride, void* dv, long long dv_stride, const int* seq_start, int T, int hq, int hkv,
    float scale, int window, cudaStream_t st);
int pm_paged_attn_ex(const void* q, const void* k_cache, const void* v_cache, void* out, const int* block_table,
    const int* seq_lens, const int* q_start, const int* q_lens, float* part_o, float* part_ml, int num_seqs, int
    max_blocks, int total_q, int max_q, int hq, int hkv, int n_split, float scale, int window, int sink, const
    float* k_scale, const float* v_scale, cudaStream_t st);
// 4-bit code-book cache: k_cache / v_cache hold two codes per byte [num_blocks, 64, hkv, 64]; a cached value is
// lut16[code] * scale (scales as for the int8 cache). lut16: 16 floats on the host. The query and the output live in
// whatever basis the cached vectors were quantised in (the caller rotates the query and un-rotates the output).
int pm_paged_attn_q4(const void* q, const void* k_cache, const void* v_cache, void* out, const int* block_table,
    const int* seq_lens, const int* q_start, const int* q_lens, float* part_o, float* part_ml, int num_seqs, int
    max_blocks, int total_q, int max_q, int hq, int hkv, int n_split, float scale, int window, int sink, const
    float* k_scale, const float* v_scale, const float* lut16, cudaStream_t st);
int pm_paged_attn(const void* q, const void* k_cache, const void* v_cache, void* out, const int* block_table, const
    int* seq_lens, const int* q_start, const int* q_lens, float* part_o, float* part_ml, int num_seqs, int
    max_blocks, int total_q, int max_q, int hq, int hkv, int n_split, float scale, int window, cudaStream_t st);
int pm_kv_append_q8(const void* k, long long k_stride, const void* v, long long v_stride, void* k_cache, void*
    v_cache, float* k_scale, float* v_scale, const long long* slots, int n_tokens, int hkv, cudaStream_t st);
// sign: 128 floats (+-1) on the device; thr: 15 ascending thresholds on the device.
int pm_kv_append_tq4(const void* k, long long k_stride, const void* v, long long v_stride, void* k_cache, void*
    v_cache, float* k_scale, float* v_scale, const long long* slots, const float* sign, const float* thr, int
    n_tokens, int hkv, cudaStream_t st);
// x, y: [rows / heads, heads, 128] bf16 with token strides x_stride / y_stride (elements); inverse 0: y = H (x sign) / sqrt(d),
// inverse 1: y = (H x) / sqrt(d) * sign.
int pm_tq_rotate(const void* x, long long x_stride, const float* sign, void* y, long long y_stride, long long
    tokens, int heads, int inverse, cudaStream_t st);
int pm_kv_append(const void* k, long long k_stride, const void* v, long long v_stride, void* k_cache, void*
    v_cache, const long long* slots, int n_tokens, int hkv, cudaStream_t st);
int pm_paged_attn_static_max_rows(void);
const char* pm_paged_attn_static_strerror(int code);

// ---------------------------------------------------------------- attention_tc.cu
int pm_attn_fwd_tc_rect(const void* q, long long q_stride, const void* k, long long k_stride, const void* v, long
    long v_stride, void* out, long long o_stride, float* lse, const int* seq_start, int T, int Tk, int shift, int
    hq, int hkv, float scale, int* status, cudaStream_t st);
// Single-softmax-group variant of the same kernel (kept selectable for comparison measurements).
int pm_attn_fwd_tc_rect_v1(const void* q, long long q_stride, const void* k, long long k_stride, const void* v,
    long long v_stride, void* out, long long o_stride, float* lse, const int* seq_start, int T, int Tk, int shift,
    int hq, int hkv, float scale, int* status, cudaStream_t st);
int pm_attn_fwd_tc(const void* q, long long q_stride, const void* k, long long k_stride, const void* v, long long
    v_stride, void* out, long long o_stride, float* lse, const int* seq_start, int T, int hq, int hkv, float scale,
    int* status, cudaStream_t st);

// ---------------------------------------------------------------- attention_tc_bwd.cu
// dout, q: [T, hq*128] (token strides o_stride / q_stride); k, v: [T, hkv*128] (v may be a strided view).
// dq:[T,hq,128], dk:[T,hkv,128], dv:[T,hkv,128] (strided). lse, delta: [hq][T].
int pm_attn_bwd_tc(const void* dout, long long do_stride, const void* q, long long q_stride, const void* k, long
    long k_stride, const void* v, long long v_stride, const float* lse, const float* delta, void* dq, long long
    dq_stride, void* dk, long long dk_stride, void* dv, long long dv_stride, const int* seq_start, int T, int hq,
    int hkv, float scale, int* status, cudaStream_t st);

// ---------------------------------------------------------------- decode_mega.cu
// 1 when one launch can run the step: up to 16 rows, 1 / 2 / 4 query heads per kv head, reduction sizes that are
// multiples of 32, and the staged activations fit in shared memory.
int pm_decode_layers_supported(int M, int H, int hq, int hkv, int I);
// layers: device array of n_layers DmLayer records (10 pointers each). bar: 2 words, counters: M * hkv words, all zero
// at launch (a completed launch leaves the counters zero; the caller clears bar before every launch).
int pm_decode_layers(const void* layers, int n_layers, int M, int H, int hq, int hkv, int I, float eps, float
    scale, void* x, void* h, void* qkv, void* attn, void* act, float* part_o, float* part_ml, unsigned* counters,
    const float* cs, const float* sn, const int* block_table, const int* seq_lens, const long long* slots, int
    max_blocks, int n_split, unsigned* bar, int* status, unsigned long long* trace, cudaStream_t st);

// ---------------------------------------------------------------- dp_fused.cu
// ptr arrays hold `world` device addresses each (peer-mapped). shadows may be null.
int pm_dp_reduce_adamw(const unsigned long long* grads, const unsigned long long* params, const unsigned long long*
    shadows, const unsigned long long* pads, float* m, float* v, const float* lr_mult, const float* wd, const
    float* gnorm_sq, const float* hp, long long n, int rank, int world, float lr, float beta1, float beta2, float
    eps, int step, float grad_scale, float max_norm, double timeout_s, int ctas, int* status, cudaStream_t st);
int pm_dp_pad_words();

// ---------------------------------------------------------------- elementwise.cu
int pm_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd, int T, int H,
    float eps, cudaStream_t st);
int pm_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd, const void* dh_add, void* dx,
    float* dw, int T, int H, cudaStream_t st);
int pm_rope_table(const int* pos, float* cs, float* sn, int T, int half, float theta, float rope_scale,
    cudaStream_t st);
int pm_rope_table_freqs(const int* pos, const float* inv_freq, float* cs, float* sn, int T, int half, float mscale,
    cudaStream_t st);
int pm_qknorm_rope_fwd(const void* qkv, int ld, const void* qw, const void* kw, const float* cs, const float* sn,
    void* q_out, void* k_out, int T, int hq, int hkv, float eps, cudaStream_t st);
int pm_qknorm_rope_cache(const void* qkv, int ld, const void* qw, const void* kw, const float* cs, const float* sn,
    void* q_out, void* k_cache, void* v_cache, const long long* slots, int T, int hq, int hkv, float eps,
    cudaStream_t st);
int pm_qknorm_rope_bwd(const void* dq, const void* dk, const void* qkv, int ld, const void* qw, const void* kw,
    const float* cs, const float* sn, void* dqkv, int T, int hq, int hkv, float eps, cudaStream_t st);
int pm_swiglu_fwd(const void* gu, void* out, long long T, int I, cudaStream_t st);
int pm_swiglu_bwd(const void* dout, const void* gu, void* dgu, long long T, int I, cudaStream_t st);
// act(gate) * up for separate gate / up matrices (row strides in elements, multiples of 8); act: 0 SiLU, 1 GELU-tanh, 2 GELU.
int pm_glu_fwd(const void* gate, const void* up, long long ldg, long long ldu, void* out, long long T, int I, int
    act, cudaStream_t st);
int pm_glu_bwd(const void* dout, const void* gate, const void* up, long long ldg, long long ldu, void* dgate, void*
    dup, long long lddg, long long lddu, long long T, int I, int act, cudaStream_t st);
// row_loss (optional): per-row loss out. row_scale (optional): per-row gradient scale replacing *inv_n.
int pm_ce_fwd_bwd(void* logits, long long ldl, const long long* labels, float* loss_sum, const float* inv_n, float*
    row_loss, const float* row_scale, int n_rows, int V, long long ignore_index, int write_grad, cudaStream_t st);
// Cross entropy plus the z term z_coef * logsumexp(logits)^2 per valid row: z_sum receives the sum of the squared
// normalisers, and the gradient written over the logits is that of (cross entropy + z_coef * z) summed over rows.
int pm_ce_z_fwd_bwd(void* logits, long long ldl, const long long* labels, float* loss_sum, float* z_sum, const
    float* inv_n, int n_rows, int V, long long ignore_index, int write_grad, float z_coef, cudaStream_t st);
// The same with label smoothing (0 <= smooth < 1) and soft-capped logits (softcap > 0: cap * tanh(x / cap)).
int pm_ce_opt_fwd_bwd(void* logits, long long ldl, const long long* labels, float* loss_sum, float* z_sum, const
    float* inv_n, int n_rows, int V, long long ignore_index, int write_grad, float z_coef, float smooth, float
    softcap, cudaStream_t st);
int pm_sumsq(const float* x, long long n, float* out, cudaStream_t st);
int pm_adamw_flat(float* p, const float* g, float* m, float* v, void* shadow, const float* lr_mult, const float*
    wd, const float* gnorm_sq, const float* hp, long long n, float lr, float beta1, float beta2, float eps, int
    step, float grad_scale, float max_norm, cudaStream_t st);
int pm_attn_delta(const void* o, const void* dout, float* delta, int T, int H, cudaStream_t st);
int pm_f32_to_bf16(const float* in, void* out, long long n, cudaStream_t st);
int pm_dequant_4bit(const void* data, const float* absmax, const void* absmax_q, float am_scale, float am_offset,
    void* out, long long n, int block_size, int fp4, cudaStream_t st);

// ---------------------------------------------------------------- gdn.cu
// Returns 0, -1 for an unsupported head shape (supported: dk x dv in {64, 128} x {64, 128}), or a CUDA error code.
int pm_gdn_scan(const float* q, const float* k, const float* v, const float* g, const float* beta, float* state,
    float* y, int B, int T, int H, int dk, int dv, cudaStream_t st);

// ---------------------------------------------------------------- gemm_2sm.cu
// Same contract as pm_gemm_bf16 with the tile fixed at 256 x 256 per CTA pair.
int pm_gemm_bf16_2sm(const void* A, int a_mn, int lda, int a_rows, const void* B, int b_mn, int ldb, int b_rows,
    const void* A2, int a2_mn, int lda2, int a2_k, const void* B2, int b2_mn, int ldb2, int b2_rows, void* D, int
    out_mode, int ldd, const void* R, int ldr, int M, int N, int K, int K2, int n_store, float alpha, int splits,
    int seg_mode, const int* seg_end, int seg_r, int max_ctas, int* status, cudaStream_t stream);

// ---------------------------------------------------------------- gemm_q4_2sm.cu
// A [M, K] bf16 (K-major). codes: packed weight [w_rows, w_cols / 2] bytes, first element of a pair in the high nibble;
// absmax (fp32) or absmax_q (+ am_scale / am_offset) hold one scale per 64 consecutive weights of a row.
//   trans 0: D[M, w_rows] (K = w_cols);  trans 1: D[M, w_cols] (K = w_rows).
// A2 / B2 (bf16, optional) add the low-rank product as in pm_gemm_bf16_2sm; seg_mode 0 or 1. D bf16 (+ R).
// w_cols % 128 == 0 and w_rows % 64 == 0. Returns 0, a negative argument error or a CUDA error code.
int pm_gemm_q4_2sm(const void* A, int lda, int a_rows, const void* codes, const float* absmax, const void*
    absmax_q, float am_scale, float am_offset, int fp4, int w_rows, int w_cols, int trans, const void* A2, int
    a2_mn, int lda2, int a2_k, const void* B2, int b2_mn, int ldb2, int b2_rows, void* D, int ldd, const void* R,
    int ldr, int M, int K2, int n_store, float alpha, int seg_mode, const int* seg_end, int seg_r, int max_ctas,
    int* status, cudaStream_t stream);

// ---------------------------------------------------------------- gemm_tcgen05.cu
// Returns 0 on success, negative on argument / descriptor errors, or the CUDA error code.
//   a_rows/b_rows: extent of the operand along M / N as seen by the tensor map (rows beyond it read as zero).
int pm_gemm_bf16(const void* A, int a_mn, int lda, int a_rows, const void* B, int b_mn, int ldb, int b_rows, const
    void* A2, int a2_mn, int lda2, int a2_k, const void* B2, int b2_mn, int ldb2, int b2_rows, void* D, int
    out_mode, int ldd, const void* R, int ldr, int M, int N, int K, int K2, int n_store, float alpha, int bn, int
    splits, int seg_mode, const int* seg_end, int seg_r, int max_ctas, float* ws, long long ws_floats, unsigned*
    ws_cnt, long long ws_cnt_len, int* status, cudaStream_t stream);

// ---------------------------------------------------------------- gemv.cu
// Returns 0, a negative argument error, or a CUDA error code. K % 8 == 0, row strides % 8 == 0, M <= 16,
// M * cols-per-warp <= 32.
int pm_gemv(const void* x, int ldx, const void* w, int ldw, const void* norm_w, float eps, const void* residual,
    int ldr, void* y, int ldy, int M, int N, int K, int swiglu, float alpha, const void* t, int ldt, const float*
    lora_b, int r, const int* seg_end, cudaStream_t st);
// 4-bit weights: qdata holds N_w * K / 2 bytes (two codes per byte, first element in the high nibble), absmax one fp32
// per qblock elements or absmax_q one byte per block with scale / offset (double quantisation). K % 32 == 0,
// qblock % 32 == 0. Other arguments as pm_gemv.
int pm_gemv_q4(const void* x, int ldx, const void* qdata, const float* absmax, const void* absmax_q, float
    am_scale, float am_offset, int qblock, int fp4, const void* norm_w, float eps, const void* residual, int ldr,
    void* y, int ldy, int M, int N, int K, int swiglu, float alpha, const void* t, int ldt, const float* lora_b,
    int r, const int* seg_end, cudaStream_t st);

// ---------------------------------------------------------------- grouped_gemm.cu
// a, b: the two operands of the mode (see the table at the top); both bf16, row strides lda / ldb in elements.
// off: int32 [E + 1] on the device, multiples of 128, off[E] <= rows_cap. D: bf16 [rows_cap, ldd] (modes 0, 1) or fp32
// [E, N, ldd] (mode 2; experts without rows are left untouched, so clear D first unless accumulating).
int pm_grouped_gemm(int mode, const void* a, int lda, const void* b, int ldb, void* D, int ldd, const int* off, int
    E, int rows_cap, int N, int K, float alpha, int accumulate, int* status, cudaStream_t stream);
// Few rows per expert (see the kernel): x [rows, K] expert-sorted with offsets off [E + 1] (any alignment), w stacked
// [E * N, K] (swiglu 0) or [E * 2N, K] with gate rows above up rows per expert (swiglu 1); y [rows, N] bf16.
// bn (32, 64, 128) is the token tile: experts with more rows take several passes over their weights.
int pm_grouped_gemm_skinny(const void* x, int ldx, int rows, const void* w, int ldw, void* y, int ldy, const int*
    off, int E, int N, int K, int bn, int swiglu, float alpha, int* status, cudaStream_t stream);

// ---------------------------------------------------------------- mhc.cu
// x [T, n, C] bf16; either phi [n C, n^2 + 2n] fp32 (dot products formed here) or raw [T, ld_raw] fp32 = x . phi computed by
// the caller; bias [n^2 + 2n], alpha [3]; n in {2, 4, 8}, C % 8 == 0, iters <= 32.
int pm_mhc_mappings(const void* x, const float* phi, const float* raw, int ld_raw, const float* bias, const float*
    alpha, int T, int n, int C, int iters, float* h_tilde, float* rms_inv, float* h_pre, float* h_post, float*
    h_res, cudaStream_t st);
int pm_mhc_pre(const void* x, const float* h_pre, int T, int n, int C, void* h_in, cudaStream_t st);
int pm_mhc_post_res(const void* x, const void* h_out, const float* h_res, const float* h_post, int T, int n, int C,
    void* x_out, cudaStream_t st);
int pm_mhc_mix_bwd(const void* x, const void* h_out, const void* dh_in, const void* dx_out, const float* h_pre,
    const float* h_post, const float* h_res, int T, int n, int C, void* dx, void* dh_out, float* d_pre, float*
    d_post, float* d_res, cudaStream_t st);
int pm_mhc_constraints_bwd(const float* h_tilde, const float* d_pre, const float* d_post, const float* d_res, int
    T, int n, int iters, float* d_tilde, cudaStream_t st);
// gains [2] fp32, cleared here: largest absolute row sum and column sum of H_res over all tokens
int pm_mhc_amax_gain(const float* h_res, int T, int n, float* gains, cudaStream_t st);
int pm_mhc_expand(const void* x, int T, int n, int C, void* xs, cudaStream_t st);
int pm_mhc_collapse(const void* xs, int T, int n, int C, void* x, cudaStream_t st);

// ---------------------------------------------------------------- moe_gemm.cu
int pm_ep_prepare(const unsigned long long* offset_ptrs, const unsigned long long* pad_ptrs, int rank, int world,
    int e_loc, void* tiles, void* runs, int max_tiles, int max_runs, int* counts_out, double timeout_s, int*
    status, cudaStream_t st);
// a: local A buffer [a_rows, K] (row stride lda): the staging buffer of the gate/up launch or the hidden rows of the
// down launch; w: [e_loc * N, K]; out_ptrs[r]: output base of rank r (push = 0 uses out_ptrs[rank] only).
// copy_src_ptrs (gate/up launch): rank r's sorted token buffer [*, K] (row stride K) that tiles are staged in from;
// tile_ready: uint32 [max_tiles], zero-initialised once. Both null for the down projection.
int pm_moe_gemm(const void* a, int a_rows, int lda, const void* w, int ldw, int e_loc, const unsigned long long*
    out_ptrs, int ldd, const void* tiles, const void* runs, const int* n_tiles, int max_tiles, int N, int K, int
    swiglu, int rank, int world, int push, const unsigned long long* pad_ptrs, const unsigned long long*
    copy_src_ptrs, void* tile_ready, double timeout_s, int* status, cudaStream_t st);

// ---------------------------------------------------------------- moe_quant.cu
// offsets2: optional second destination for the [E + 1] offsets (may be null).
int pm_moe_route2(const void* logits, int is_f32, int T, int E, int k, int renorm, int* topk_idx, float* topk_w,
    int* counts, int* offsets, int* offsets2, int* perm, int* inv, cudaStream_t st);
int pm_moe_route(const void* logits, int is_f32, int T, int E, int k, int renorm, int* topk_idx, float* topk_w,
    int* counts, int* offsets, int* perm, int* inv, cudaStream_t st);
// Routing plus the padded layout of the assignments that belong to experts [e0, e0 + e_loc) (see the kernel).
int pm_moe_route_local(const void* logits, int is_f32, int T, int E, int k, int renorm, int e0, int e_loc, int
    align, int* topk_idx, float* topk_w, int* off, int* dest, int* src, cudaStream_t st);
// off_end points at the device int holding the number of rows in use (off[e_loc]); cap bounds the launch.
int pm_moe_gather_padded(const void* x, const int* src, const int* off_end, int k, void* xs, int cap, int H,
    cudaStream_t st);
int pm_moe_combine_local(const void* z, const int* dest, const float* w, int k, const void* residual, void* y, long
    long T, int H, cudaStream_t st);
int pm_moe_gather(const void* x, const int* perm, int k, void* out, long long n, int H, cudaStream_t st);
int pm_moe_combine2(const void* z, const int* inv, const float* w, int k, const void* residual, void* y, long long
    T, int H, cudaStream_t st);
int pm_moe_combine(const void* z, const int* inv, const float* w, int k, void* y, long long T, int H, cudaStream_t
    st);
int pm_gguf_dequant_bf16(const void* src, void* dst, long long n, int type, cudaStream_t st);
int pm_fp8_quant(const void* x, void* q, float* scales, long long n, cudaStream_t st);
int pm_fp8_dequant(const void* q, const float* scales, void* y, long long n, cudaStream_t st);

// ---------------------------------------------------------------- sampling.cu
int pm_sample(const void* logits, int is_bf16, long long ld, int rows, int vocab, const int* counts, const int*
    count_rows, const float* temperature, const int* top_k, const float* top_p, const float* min_p, const float*
    rep_pen, const float* freq_pen, const float* pres_pen, const unsigned long long* seeds, unsigned long long
    step, int* out_token, float* out_logprob, cudaStream_t st);
int pm_spec_verify(const float* target, const float* draft, const int* tokens, int n_seq, int K, int vocab, float
    temperature, const unsigned long long* seeds, unsigned long long step, int* n_accepted, int* next_token,
    cudaStream_t st);
int pm_count_tokens(int* counts, const int* count_rows, const int* tokens, int rows, int vocab, cudaStream_t st);

// ---------------------------------------------------------------- tp_fused.cu
// mode 0: x_ptrs[r] = rank r's X shard [rows_per_rank, K] (ldx), w = W_loc [N, K] (ldw), out = Y [M, ldd].
// mode 1: x_ptrs[rank] = local X [M, K] (ldx), w = W_loc [N, K], stage_ptrs[r] = rank r's staging buffer,
//         out = Y_r [rows_per_rank, ldd]. K and N are the local extents. mode 0 also takes `gathered` (local bf16
//         [M, K] scratch) and `blk_ready` (uint32 [M / 128], zero-initialised once). Returns 0, a negative argument
//         error, or a CUDA error code.
int pm_tp_gemm(int mode, const unsigned long long* x_ptrs, int ldx, const void* w, int ldw, void* out, int ldd,
    const unsigned long long* stage_ptrs, const unsigned long long* pad_ptrs, int rank, int world, int M, int N,
    int K, void* gathered, void* blk_ready, double timeout_s, int max_ctas, int* status, cudaStream_t stream);
// x: bf16 [n] (n a multiple of 8, at most slot_elems), summed in place over the ranks. bufs[r] / pads[r]: rank r's
// exchange buffer (2 * world * slot_elems bf16) and signal pad (64 uint32, zero-initialised once), peer-mapped.
int pm_peer_allreduce(void* x, long long n, const unsigned long long* bufs, const unsigned long long* pads, long
    long slot_elems, int rank, int world, double timeout_s, int* status, cudaStream_t st);

// ---------------------------------------------------------------- train_aux.cu
int pm_kd_fwd_bwd(void* student, long long ld, const void* teacher, long long ldt, int rows, int V, float
    temperature, int kind, float beta, const float* row_scale, float* row_loss, float* loss_sum, int write_grad,
    cudaStream_t st);
int pm_merge_fused(const void* const* models, const void* base, const float* weights, const float* thresholds,
    const float* densities, int n_models, int in_bf16, int out_bf16, int consensus, int rescale, float lam,
    unsigned long long seed, void* out, long long n, cudaStream_t st);
int pm_dot_norms(const void* a, const void* b, int bf16, long long n, float* out3, cudaStream_t st);

#ifdef __cplusplus
}
#endif
