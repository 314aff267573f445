"""ctypes bindings for the sm_100a kernel library (``pmetal_b200/lib/libpmetal_b200.so``).

The library is plain CUDA C++ with ``extern "C"`` launchers that take raw device
pointers and a stream; tensors are allocated here with PyTorch and every launch
goes to PyTorch's current stream, so the kernels compose with autograd, CUDA graphs
and NCCL streams. Launchers return 0 or an error code, which is raised.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence, Tuple

import torch

_LIB = None
_ERR: Optional[str] = None
_STATUS = {}
LIB_PATH = os.environ.get("PMETAL_NATIVE_LIB") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib", "libpmetal_b200.so")

# The transposed LoRA products read token-major tensors through MN-major tcgen05 descriptors.
# PMETAL_MN_MAJOR=0 routes them through explicit transposes instead.
MN_MAJOR = os.environ.get("PMETAL_MN_MAJOR", "1") == "1"
ATTN_TC = os.environ.get("PMETAL_ATTN_TC", "1") == "1"      # tcgen05 attention kernels
ATTN_FWD_V1 = os.environ.get("PMETAL_ATTN_FWD_V1", "0") == "1"   # single-softmax-group forward (comparison runs)
USE_2SM = os.environ.get("PMETAL_GEMM_2SM", "1") == "1"   # CTA-pair kernel for 256-wide tiles
# Reductions over tokens (LoRA dA / dB, weight gradients) are split across CTAs and summed with fp32 atomics, whose
# order varies from run to run. With PMETAL_DETERMINISTIC=1 every output tile is owned by one CTA and accumulated in a
# fixed order instead (slower for the skinny LoRA products, bitwise reproducible).
DETERMINISTIC = os.environ.get("PMETAL_DETERMINISTIC", "0") == "1"
# PMETAL_TUNA=1: the tile width of plain GEMMs comes from the tuner's cache (utils/tuna.py); a shape seen for the first
# time is timed over the candidate widths once (never during CUDA-graph capture) and the winner is remembered on disk.
TUNA = os.environ.get("PMETAL_TUNA", "0") == "1"
LAUNCHES = 0   # number of kernels launched through this module (bench reporting)

c_void_p, c_int, c_float, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong


def _load():
    global _LIB, _ERR
    if _LIB is not None or _ERR is not None:
        return
    if not os.path.exists(LIB_PATH):
        _ERR = f"{LIB_PATH} not found"
        return
    try:
        _LIB = ctypes.CDLL(LIB_PATH)
    except OSError as e:  # pragma: no cover
        _ERR = str(e)
        return
    for name in dir(_LIB):
        pass
    for fn in ("pm_gemm_bf16", "pm_gemm_bf16_2sm", "pm_rmsnorm_fwd", "pm_rmsnorm_bwd", "pm_rope_table", "pm_qknorm_rope_fwd",
               "pm_qknorm_rope_bwd", "pm_swiglu_fwd", "pm_swiglu_bwd", "pm_ce_fwd_bwd", "pm_sumsq", "pm_adamw_flat",
               "pm_attn_delta", "pm_attn_fwd", "pm_attn_bwd", "pm_f32_to_bf16", "pm_paged_attn", "pm_kv_append", "pm_attn_fwd_tc", "pm_attn_bwd_tc", "pm_dequant_4bit", "pm_sample", "pm_spec_verify", "pm_count_tokens",
               "pm_moe_route", "pm_moe_gather", "pm_moe_combine", "pm_gguf_dequant_bf16", "pm_fp8_quant", "pm_fp8_dequant",
               "pm_kd_fwd_bwd", "pm_merge_fused", "pm_dot_norms", "pm_attn_fwd_tc_rect", "pm_attn_fwd_tc_rect_v1", "pm_gemv",
               "pm_qknorm_rope_cache"):
        getattr(_LIB, fn).restype = c_int


def available() -> bool:
    _load()
    return _LIB is not None and torch.cuda.is_available()


def load_error() -> Optional[str]:
    _load()
    return _ERR


def lib():
    _load()
    if _LIB is None:
        raise RuntimeError(f"native library unavailable: {_ERR}")
    return _LIB


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


_SM_COUNT = {}


def sm_count(device=None) -> int:
    """Number of SMs of the device (grid sizing); 148 when no GPU is present (CPU-side planning and tests)."""
    if not torch.cuda.is_available():
        return 148
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def _chk(rc: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


def status_word(device=None) -> torch.Tensor:
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev not in _STATUS:
        _STATUS[dev] = torch.zeros(1, dtype=torch.int32, device=dev)
    return _STATUS[dev]


def check_status() -> None:
    """Synchronise and raise if any kernel abandoned a bounded wait."""
    for dev, t in _STATUS.items():
        v = int(t.item())
        if v != 0:
            t.zero_()
            raise RuntimeError(f"device-side wait timed out on {dev} (status {v})")


# ------------------------------------------------------------------------------------------- GEMM
def _pick_bn(n: int, seg_sizes: Sequence[int] = (), m: int = 1 << 30) -> int:
    """Widest tile whose boundaries respect the LoRA segments; a ragged last tile is fine (TMA zero-fills).
    A single row block (decode: m <= 128) is bandwidth-bound on the weight read, so narrow tiles are used there to
    spread the columns over as many SMs as possible."""
    segs = seg_sizes[:-1] if len(seg_sizes) > 1 else ()
    widths = (256, 128, 64, 32)
    if m <= 128:
        widths = tuple(b for b in (32, 64, 128, 256) if -(-n // b) <= 4 * sm_count()) or (256,)
        for bn in widths:
            if all(s % bn == 0 for s in segs):
                return bn
    for bn in (256, 128, 64, 32):
        if n >= bn and all(s % bn == 0 for s in segs):
            return bn
    return 32


def tuned_choice(op: str, shape, candidates, default, run):
    """Best of ``candidates`` for ``op`` at ``shape`` according to the tuner's cache; times them on a cache miss."""
    from ..utils.tuna import Tuner, global_tuner
    t = global_tuner()
    key = Tuner.make_key(op, *shape)
    hit = t.lookup(key)
    if hit is not None and hit in list(candidates):
        return hit
    if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
        return default                      # timing needs synchronisation: not inside a capture
    return t.tune(key, list(candidates), run)


def _seg_ends(seg_sizes: Sequence[int]):
    ends, c = [], 0
    for s in seg_sizes:
        c += s
        ends.append(c)
    ends = ends[:-1] + [0x7FFFFFFF] * (5 - len(ends))
    return (c_int * 4)(*ends[:4])


def raw_gemm(A, a_mn, lda, a_rows, B, b_mn, ldb, b_rows, D, out_mode, ldd, M, N, K, *, A2=None, a2_mn=0, lda2=0,
             a2_k=0, B2=None, b2_mn=0, ldb2=0, b2_rows=0, K2=0, R=None, ldr=0, n_store=0, alpha=1.0, bn=128, splits=1,
             seg_mode=0, seg_sizes=(), seg_r=0, max_ctas=0) -> None:
    """One GEMM launch. 256-wide tiles on at least 256 rows go to the CTA-pair (cta_group::2) kernel."""
    segs = _seg_ends(seg_sizes) if seg_mode else None
    if USE_2SM and bn == 256 and M >= 256 and (seg_mode != 2 or all(s % 256 == 0 for s in seg_sizes[:-1])):
        rc = lib().pm_gemm_bf16_2sm(_p(A), c_int(a_mn), c_int(lda), c_int(a_rows), _p(B), c_int(b_mn), c_int(ldb),
                                    c_int(b_rows), _p(A2), c_int(a2_mn), c_int(lda2), c_int(a2_k), _p(B2),
                                    c_int(b2_mn), c_int(ldb2), c_int(b2_rows), _p(D), c_int(out_mode), c_int(ldd),
                                    _p(R), c_int(ldr), c_int(M), c_int(N), c_int(K), c_int(K2), c_int(n_store),
                                    c_float(alpha), c_int(splits), c_int(seg_mode), segs, c_int(seg_r),
                                    c_int(max_ctas), _p(status_word(D.device)), _stream())
        _chk(rc, "pm_gemm_bf16_2sm")
        return
    ws = cnt = None
    if out_mode == 0 and splits == 1 and SPLIT_K and M <= 128 and seg_mode in (0, 1):
        # one row block: the few column tiles leave most SMs idle and each walks all of K by itself; cut K so that the
        # launch covers the machine, partial tiles meeting in a workspace (reduced inside the kernel)
        tiles = -(-N // bn)
        nk = -(-K // 64) + (-(-K2 // 64) if K2 > 0 else 0)
        want = min(nk // 4, sm_count() // tiles)
        if want >= 2:
            per = -(-nk // want)
            want = -(-nk // per)
            got = _splitk_workspace(D.device, tiles * want * 128 * bn, tiles * 4)
            if got is not None and want >= 2:
                ws, cnt = got
                out_mode, splits = 6, want
    rc = lib().pm_gemm_bf16(_p(A), c_int(a_mn), c_int(lda), c_int(a_rows), _p(B), c_int(b_mn), c_int(ldb),
                            c_int(b_rows), _p(A2), c_int(a2_mn), c_int(lda2), c_int(a2_k), _p(B2), c_int(b2_mn),
                            c_int(ldb2), c_int(b2_rows), _p(D), c_int(out_mode), c_int(ldd), _p(R), c_int(ldr),
                            c_int(M), c_int(N), c_int(K), c_int(K2), c_int(n_store), c_float(alpha), c_int(bn),
                            c_int(splits), c_int(seg_mode), segs, c_int(seg_r), c_int(max_ctas), _p(ws),
                            ctypes.c_longlong(ws.numel() if ws is not None else 0), _p(cnt),
                            ctypes.c_longlong(cnt.numel() if cnt is not None else 0), _p(status_word(D.device)), _stream())
    _chk(rc, "pm_gemm_bf16")


SPLIT_K = os.environ.get("PMETAL_GEMM_SPLITK", "1") == "1"
FUSED_Q4 = os.environ.get("PMETAL_FUSED_Q4", "0") == "1"      # opt-in: saves the transient bf16 weight, not time
_SPLITK_WS = {}


def _splitk_workspace(device, floats: int, counters: int):
    """(fp32 partial-tile buffer, zeroed arrival counters) for split-K launches on the current stream of ``device``.
    Launches on one stream run in order and may share a buffer; every stream has its own. Captured launches use a
    buffer of their own that is created ahead of the capture (by the first eager call); a capture that would have to
    create or grow it gets None and runs without the split."""
    capturing = torch.cuda.is_current_stream_capturing()
    dev = device.index if device.index is not None else torch.cuda.current_device()
    keys = [(dev, 0)] if capturing else [(dev, torch.cuda.current_stream(device).cuda_stream), (dev, 0)]
    out = None
    for key in reversed(keys):           # the capture buffer first, so that it always exists before a capture starts
        ent = _SPLITK_WS.get(key)
        if ent is None or ent[0].numel() < floats or ent[1].numel() < counters:
            if capturing:
                return None
            ent = _SPLITK_WS[key] = (torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device),
                                     torch.zeros(max(counters, 4096), dtype=torch.int32, device=device))
        out = ent
    return out


def _t_width(nr: int) -> int:
    return -(-nr // 64) * 64


def gemm(x: torch.Tensor, w: torch.Tensor, alpha: float = 1.0, residual: Optional[torch.Tensor] = None,
         out: Optional[torch.Tensor] = None, pad_n_to: int = 0, bn: int = 0) -> torch.Tensor:
    """[M,K] x [N,K]^T -> [M,N] bf16. ``pad_n_to`` widens the output (extra columns are written as zeros)."""
    M, K = x.shape
    N = w.shape[0]
    Nw = max(N, pad_n_to)
    if out is None:
        out = torch.empty(M, Nw, dtype=torch.bfloat16, device=x.device)

    def run(b):
        raw_gemm(x, 0, x.stride(0), M, w, 0, w.stride(0), N, out, 0, out.stride(0), M, Nw, K, R=residual,
                 ldr=residual.stride(0) if residual is not None else 0, alpha=alpha, bn=b)
    if not bn:
        bn = _pick_bn(Nw, (), M)
        if TUNA:
            bn = tuned_choice("gemm_bn", (M, Nw, K), [b for b in (32, 64, 128, 256) if b <= max(Nw, 32)], bn, run)
    run(bn)
    return out


def gemm_lora(x, w, t, b, seg_sizes, r, residual=None, bn: int = 0) -> torch.Tensor:
    """y = x w^T + sum_seg t[:, seg*r:(seg+1)*r] b_seg^T (+ residual). t already carries the LoRA scale."""
    M, K = x.shape
    N = w.shape[0]
    out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    bn = bn or _pick_bn(N, seg_sizes, M)
    kw = {}
    if t is not None:
        kw = dict(A2=t, a2_mn=0, lda2=t.stride(0), a2_k=t.shape[1], B2=b, b2_mn=0, ldb2=b.stride(0), b2_rows=N, K2=r,
                  seg_mode=1 if len(seg_sizes) > 1 else 0, seg_sizes=seg_sizes, seg_r=r)
    raw_gemm(x, 0, x.stride(0), M, w, 0, w.stride(0), N, out, 0, N, M, N, K, R=residual,
             ldr=residual.stride(0) if residual is not None else 0, bn=bn, **kw)
    return out


def lora_t(x, a, scale: float) -> torch.Tensor:
    """t = scale * x a^T, padded to a multiple of 64 columns (padding is zero)."""
    return gemm(x, a, alpha=scale, pad_n_to=_t_width(a.shape[0]), bn=64)


def lora_dt(dy, b, seg_sizes, r, scale) -> torch.Tensor:
    """dt[:, seg*r:(seg+1)*r] = scale * dy[:, seg] b_seg   ([M, 64-padded]); padding columns are unspecified."""
    M, N = dy.shape
    nseg = len(seg_sizes)
    dt = torch.empty(M, _t_width(nseg * r), dtype=torch.bfloat16, device=dy.device)
    if (MN_MAJOR and nseg * r <= 64 and r % 8 == 0 and all(s % 64 == 0 for s in seg_sizes) and b.is_contiguous()
            and b.shape[1] == r):
        # one launch: b [N, r] is read in place as an MN-major operand; segment s of the reduction lands in output
        # columns [s r, (s + 1) r) because its tile is fetched s r columns left of the origin (zero fill elsewhere)
        raw_gemm(dy, 0, dy.stride(0), M, b, 1, r, r, dt, 0, dt.stride(0), M, 64, N, alpha=scale, bn=64,
                 seg_mode=3, seg_sizes=seg_sizes, seg_r=r)
        return dt
    b_t = b.t().contiguous()                      # [r, N], K-major over N
    n0 = 0
    for i, sz in enumerate(seg_sizes):
        raw_gemm(dy[:, n0:], 0, dy.stride(0), M, b_t[:, n0:], 0, N, r, dt[:, i * r:], 0, dt.stride(0), M, 32, sz,
                 n_store=r, alpha=scale, bn=32)
        n0 += sz
    return dt


def gemm_lora_dx(dy, w, w_t, dt, a) -> torch.Tensor:
    """dx = dy w (+ dt[:, :nr] a).  w:[N,K_in]; w_t:[K_in,N] optional; a:[nr,K_in]."""
    M, N = dy.shape
    kin = w.shape[1]
    out = torch.empty(M, kin, dtype=torch.bfloat16, device=dy.device)
    bn = _pick_bn(kin)
    kw = {}
    if dt is not None:
        nr = a.shape[0]
        if MN_MAJOR:
            kw = dict(A2=dt, a2_mn=0, lda2=dt.stride(0), a2_k=dt.shape[1], B2=a, b2_mn=1, ldb2=a.stride(0),
                      b2_rows=kin, K2=nr)
        else:
            a_t = a.t().contiguous()
            kw = dict(A2=dt, a2_mn=0, lda2=dt.stride(0), a2_k=dt.shape[1], B2=a_t, b2_mn=0, ldb2=nr, b2_rows=kin, K2=nr)
    if w_t is not None:
        raw_gemm(dy, 0, dy.stride(0), M, w_t, 0, w_t.stride(0), kin, out, 0, kin, M, kin, N, bn=bn, **kw)
    elif MN_MAJOR:
        raw_gemm(dy, 0, dy.stride(0), M, w, 1, w.stride(0), kin, out, 0, kin, M, kin, N, bn=max(bn, 64), **kw)
    else:
        wt = w.t().contiguous()
        raw_gemm(dy, 0, dy.stride(0), M, wt, 0, N, kin, out, 0, kin, M, kin, N, bn=bn, **kw)
    return out


def q4_gemm_ok(q, M: int, seg_sizes: Sequence[int] = ()) -> bool:
    """Whether the GEMMs against packed weight ``q`` can expand it on the fly (csrc/gemm_q4_2sm.cu): 4-bit codes in blocks
    of 64 that line up with the rows, enough token rows for 256-row tiles, LoRA segments on tile boundaries."""
    if not FUSED_Q4 or q is None or q.scheme not in ("nf4", "fp4") or q.block_size != 64 or len(q.shape) != 2:
        return False
    n, k = q.shape
    return (M >= 256 and k % 128 == 0 and n % 64 == 0 and q.data.is_cuda
            and all(s % 256 == 0 for s in tuple(seg_sizes)[:-1]))


def _q4_call(x, q, trans: int, out, residual, kw) -> None:
    n, k = q.shape
    segs = _seg_ends(kw.get("seg_sizes", ())) if kw.get("seg_mode", 0) else None
    A2, B2 = kw.get("A2"), kw.get("B2")
    lib().pm_gemm_q4_2sm.restype = c_int
    rc = lib().pm_gemm_q4_2sm(_p(x), c_int(x.stride(0)), c_int(x.shape[0]), _p(q.data), _p(q.absmax), _p(q.absmax_q),
                              c_float(q.absmax_scale), c_float(q.absmax_offset), c_int(int(q.scheme == "fp4")), c_int(n),
                              c_int(k), c_int(trans), _p(A2), c_int(kw.get("a2_mn", 0)), c_int(kw.get("lda2", 0)),
                              c_int(kw.get("a2_k", 0)), _p(B2), c_int(kw.get("b2_mn", 0)), c_int(kw.get("ldb2", 0)),
                              c_int(kw.get("b2_rows", 0)), _p(out), c_int(out.stride(0)), _p(residual),
                              c_int(residual.stride(0) if residual is not None else 0), c_int(x.shape[0]),
                              c_int(kw.get("K2", 0)), c_int(0), c_float(1.0), c_int(kw.get("seg_mode", 0)), segs,
                              c_int(kw.get("seg_r", 0)), c_int(0), _p(status_word(x.device)), _stream())
    _chk(rc, "pm_gemm_q4_2sm")


def gemm_q4_lora(x, q, t, b, seg_sizes, r, residual=None) -> torch.Tensor:
    """y = x W^T + sum_seg t[:, seg] b_seg^T (+ residual) with W given as packed 4-bit codes (expanded inside the GEMM)."""
    M = x.shape[0]
    N = q.shape[0]
    out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    kw = {}
    if t is not None:
        kw = dict(A2=t, a2_mn=0, lda2=t.stride(0), a2_k=t.shape[1], B2=b, b2_mn=0, ldb2=b.stride(0), b2_rows=N, K2=r,
                  seg_mode=1 if len(seg_sizes) > 1 else 0, seg_sizes=seg_sizes, seg_r=r)
    _q4_call(x, q, 0, out, residual, kw)
    return out


def gemm_q4_lora_dx(dy, q, dt, a) -> torch.Tensor:
    """dx = dy W (+ dt[:, :nr] a) with W given as packed 4-bit codes."""
    M = dy.shape[0]
    kin = q.shape[1]
    out = torch.empty(M, kin, dtype=torch.bfloat16, device=dy.device)
    kw = {}
    if dt is not None:
        nr = a.shape[0]
        kw = dict(A2=dt, a2_mn=0, lda2=dt.stride(0), a2_k=dt.shape[1], B2=a, b2_mn=1, ldb2=a.stride(0), b2_rows=kin, K2=nr)
    _q4_call(dy, q, 1, out, None, kw)
    return out


def _splits_for(m_tiles: int, nk: int) -> int:
    """How many ways to cut the reduction of a token-reduction GEMM with ``m_tiles`` output tiles and ``nk`` k-blocks.

    Every (tile, split) pair is one CTA and an SM streams its operands at a fixed rate, so the launch takes
    waves * (k-blocks per split + a fixed cost per CTA) with waves = ceil(pairs / SMs). One pair more than there are SMs
    doubles the time, so the count is chosen by that makespan, not by rounding SMs / tiles up."""
    sms, m_tiles = sm_count(), max(m_tiles, 1)
    best, best_cost = 1, None
    for s in range(1, min(nk, 64) + 1):
        per = -(-nk // s)
        if (s - 1) * per >= nk:              # an empty last split is rejected by the launcher
            continue
        cost = -(-(m_tiles * s) // sms) * (per + 6)
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    return best


def lora_da(dt, x, nr: int, out: torch.Tensor) -> None:
    """out[nr, K_in] (fp32) += dt[:, :nr]^T x  — reduction over tokens, split across CTAs."""
    M, kin = x.shape
    if not MN_MAJOR:
        out.add_(dt[:, :nr].t().float() @ x.float())
        return
    tw = dt.shape[1]
    nk = -(-M // 64)
    det = DETERMINISTIC
    raw_gemm(x, 1, x.stride(0), kin, dt, 1, dt.stride(0), tw, out, 5 if det else 3, out.stride(0), kin, tw, M, n_store=nr,
             bn=64, splits=1 if det else _splits_for(-(-kin // 128), nk))


def lora_db(dy, t, seg_sizes, r: int, out: torch.Tensor) -> None:
    """out[N, r] (fp32) += dy_seg^T t[:, seg*r:(seg+1)*r]."""
    M, N = dy.shape
    if not MN_MAJOR:
        n0 = 0
        for i, sz in enumerate(seg_sizes):
            out[n0:n0 + sz].add_(dy[:, n0:n0 + sz].t().float() @ t[:, i * r:(i + 1) * r].float())
            n0 += sz
        return
    nk = -(-M // 64)
    det = DETERMINISTIC
    raw_gemm(dy, 1, dy.stride(0), N, t, 1, t.stride(0), t.shape[1], out, 4 if det else 2, out.stride(0), N, 64, M,
             n_store=r, bn=64, splits=1 if det else _splits_for(-(-N // 128), nk),
             seg_mode=2 if len(seg_sizes) > 1 else 0, seg_sizes=seg_sizes, seg_r=r)


# ------------------------------------------------------------------------------------------- grouped (expert) GEMM
def grouped_gemm(mode: int, a: torch.Tensor, b: torch.Tensor, off: torch.Tensor, n: int, k: int,
                 out: Optional[torch.Tensor] = None, accumulate: bool = False, alpha: float = 1.0) -> torch.Tensor:
    """Grouped GEMM over expert-sorted rows in the padded layout (``off`` int32 [E+1], multiples of 128; csrc/grouped_gemm.cu).

    mode 0: a = X [R, K], b = W [E, N, K]      -> Y  [R, N] bf16
    mode 1: a = dY [R, N], b = W [E, N, K]     -> dX [R, K] bf16
    mode 2: a = dY [R, N], b = X [R, K]        -> dW [E, N, K] fp32 (experts without rows keep ``out``'s contents)"""
    E = off.numel() - 1
    R = a.shape[0]
    assert R % 128 == 0 and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and off.dtype == torch.int32
    assert a.stride(1) == 1 and b.stride(-1) == 1
    if mode == 0:
        out = out if out is not None else torch.empty(R, n, dtype=torch.bfloat16, device=a.device)
        ldb = b.stride(1)
    elif mode == 1:
        out = out if out is not None else torch.empty(R, k, dtype=torch.bfloat16, device=a.device)
        ldb = b.stride(1)
    else:
        if out is None:
            out = torch.zeros(E, n, k, dtype=torch.float32, device=a.device)
        ldb = b.stride(0)
    lib().pm_grouped_gemm.restype = c_int
    rc = lib().pm_grouped_gemm(c_int(mode), _p(a), c_int(a.stride(0)), _p(b), c_int(ldb), _p(out), c_int(out.stride(-2)),
                               _p(off), c_int(E), c_int(R), c_int(n), c_int(k), c_float(alpha), c_int(int(accumulate)),
                               _p(status_word(a.device)), _stream())
    _chk(rc, "pm_grouped_gemm")
    return out


def grouped_gemm_skinny(x: torch.Tensor, w: torch.Tensor, off: torch.Tensor, swiglu: bool = False,
                        max_rows_per_expert: int = 128) -> torch.Tensor:
    """Expert GEMM for steps that give each expert few rows (csrc/grouped_gemm.cu, swapped operands): ``x`` [R, K]
    expert-sorted with row offsets ``off`` (int32 [E + 1], no alignment), ``w`` [E, N, K], or [E, 2 N, K] with
    ``swiglu`` (gate rows above up rows), in which case the result is silu(x G^T) * (x U^T). Returns [R, N] bf16; rows
    that belong to no expert are left unwritten."""
    E = off.numel() - 1
    R, K = x.shape
    N = w.shape[1] // 2 if swiglu else w.shape[1]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and off.dtype == torch.int32
    assert x.stride(1) == 1 and w.is_contiguous() and w.shape[0] == E and w.shape[2] == K
    bn = 32 if max_rows_per_expert <= 32 else (64 if max_rows_per_expert <= 64 else 128)
    y = torch.empty(R, N, dtype=torch.bfloat16, device=x.device)
    lib().pm_grouped_gemm_skinny.restype = c_int
    rc = lib().pm_grouped_gemm_skinny(_p(x), c_int(x.stride(0)), c_int(R), _p(w), c_int(w.stride(1)), _p(y), c_int(N),
                                      _p(off), c_int(E), c_int(N), c_int(K), c_int(bn), c_int(int(swiglu)),
                                      c_float(1.0), _p(status_word(x.device)), _stream())
    _chk(rc, "pm_grouped_gemm_skinny")
    return y


# ------------------------------------------------------------------------------------------- hyper-connections
def gemm_f32(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """[M, K] x [N, K]^T -> [M, N padded to a multiple of 32] fp32 (extra columns are zero)."""
    M, K = x.shape
    N = w.shape[0]
    bn = 32 if N <= 32 else (64 if N <= 64 else 128)
    Np = -(-N // bn) * bn
    out = torch.zeros(M, Np, dtype=torch.float32, device=x.device)
    raw_gemm(x, 0, x.stride(0), M, w, 0, w.stride(0), N, out, 1, Np, M, Np, K, bn=bn)
    return out


def mhc_mappings(x, raw, bias, alpha, iters: int):
    """x [T, n, C] bf16, raw [T, ld] fp32 = flatten(x) . phi -> (H~ [T, n^2+2n], 1/rms [T], H_pre, H_post, H_res)."""
    T, n, C = x.shape
    out = n * n + 2 * n
    f = lambda *s: torch.empty(*s, dtype=torch.float32, device=x.device)      # noqa: E731
    ht, ri, pre, post, res = f(T, out), f(T), f(T, n), f(T, n), f(T, n, n)
    lib().pm_mhc_mappings.restype = c_int
    _chk(lib().pm_mhc_mappings(_p(x), _p(None), _p(raw), c_int(raw.stride(0)), _p(bias), _p(alpha), c_int(T), c_int(n),
                               c_int(C), c_int(iters), _p(ht), _p(ri), _p(pre), _p(post), _p(res), _stream()),
         "pm_mhc_mappings")
    return ht, ri, pre, post, res


def mhc_pre(x, h_pre):
    T, n, C = x.shape
    out = torch.empty(T, C, dtype=x.dtype, device=x.device)
    lib().pm_mhc_pre.restype = c_int
    _chk(lib().pm_mhc_pre(_p(x), _p(h_pre), c_int(T), c_int(n), c_int(C), _p(out), _stream()), "pm_mhc_pre")
    return out


def mhc_post_res(x, h_out, h_res, h_post):
    T, n, C = x.shape
    out = torch.empty_like(x)
    lib().pm_mhc_post_res.restype = c_int
    _chk(lib().pm_mhc_post_res(_p(x), _p(h_out), _p(h_res), _p(h_post), c_int(T), c_int(n), c_int(C), _p(out), _stream()),
         "pm_mhc_post_res")
    return out


def mhc_mix_bwd(x, h_out, dh_in, dx_out, h_pre, h_post, h_res):
    """Gradients of the two stream applications; either half may be None. Returns (dx, dh_out, dH_pre, dH_post, dH_res)."""
    T, n, C = x.shape
    f = lambda *s: torch.empty(*s, dtype=torch.float32, device=x.device)      # noqa: E731
    dx = torch.empty_like(x)
    dh_out = torch.empty(T, C, dtype=x.dtype, device=x.device) if dx_out is not None else None
    d_pre = f(T, n) if dh_in is not None else None
    d_post, d_res = (f(T, n), f(T, n, n)) if dx_out is not None else (None, None)
    dummy = torch.zeros(n * n, dtype=torch.float32, device=x.device)          # unused halves still need readable gains
    lib().pm_mhc_mix_bwd.restype = c_int
    _chk(lib().pm_mhc_mix_bwd(_p(x), _p(h_out), _p(dh_in), _p(dx_out), _p(h_pre if h_pre is not None else dummy),
                              _p(h_post if h_post is not None else dummy), _p(h_res if h_res is not None else dummy),
                              c_int(T), c_int(n), c_int(C), _p(dx), _p(dh_out), _p(d_pre), _p(d_post), _p(d_res),
                              _stream()), "pm_mhc_mix_bwd")
    return dx, dh_out, d_pre, d_post, d_res


def mhc_constraints_bwd(h_tilde, d_pre, d_post, d_res, n: int, iters: int):
    T = h_tilde.shape[0]
    out = torch.empty_like(h_tilde)
    lib().pm_mhc_constraints_bwd.restype = c_int
    _chk(lib().pm_mhc_constraints_bwd(_p(h_tilde), _p(d_pre), _p(d_post), _p(d_res), c_int(T), c_int(n), c_int(iters),
                                      _p(out), _stream()), "pm_mhc_constraints_bwd")
    return out


def mhc_amax_gain(h_res):
    T, n = h_res.shape[0], h_res.shape[-1]
    g = torch.empty(2, dtype=torch.float32, device=h_res.device)
    lib().pm_mhc_amax_gain.restype = c_int
    _chk(lib().pm_mhc_amax_gain(_p(h_res), c_int(T), c_int(n), _p(g), _stream()), "pm_mhc_amax_gain")
    return g


def mhc_expand(x, n: int):
    T, C = x.shape
    out = torch.empty(T, n, C, dtype=x.dtype, device=x.device)
    lib().pm_mhc_expand.restype = c_int
    _chk(lib().pm_mhc_expand(_p(x), c_int(T), c_int(n), c_int(C), _p(out), _stream()), "pm_mhc_expand")
    return out


def mhc_collapse(xs):
    T, n, C = xs.shape
    out = torch.empty(T, C, dtype=xs.dtype, device=xs.device)
    lib().pm_mhc_collapse.restype = c_int
    _chk(lib().pm_mhc_collapse(_p(xs), c_int(T), c_int(n), c_int(C), _p(out), _stream()), "pm_mhc_collapse")
    return out


# ------------------------------------------------------------------------------------------- norms etc.
def rmsnorm_fwd(x, w, eps: float, residual=None):
    T, H = x.shape
    y = torch.empty_like(x)
    h = torch.empty_like(x) if residual is not None else x
    rstd = torch.empty(T, dtype=torch.float32, device=x.device)
    _chk(lib().pm_rmsnorm_fwd(_p(x), _p(residual), _p(w), _p(y), _p(h if residual is not None else None), _p(rstd),
                              c_int(T), c_int(H), c_float(eps), _stream()), "pm_rmsnorm_fwd")
    return h, y, rstd


def rmsnorm_bwd(dy, h, w, rstd, dh_add=None, want_dw: bool = False):
    T, H = h.shape
    dx = torch.empty_like(h)
    dw = torch.zeros(H, dtype=torch.float32, device=h.device) if want_dw else None
    _chk(lib().pm_rmsnorm_bwd(_p(dy), _p(h), _p(w), _p(rstd), _p(dh_add), _p(dx), _p(dw), c_int(T), c_int(H),
                              _stream()), "pm_rmsnorm_bwd")
    return dx, (dw.to(w.dtype) if dw is not None else None)


def rope_table(positions: torch.Tensor, head_dim: int, theta: float, rope_scale: float = 1.0):
    T = positions.shape[0]
    half = head_dim // 2
    pos = positions if positions.dtype == torch.int32 else positions.to(torch.int32)
    cs = torch.empty(T, half, dtype=torch.float32, device=positions.device)
    sn = torch.empty_like(cs)
    _chk(lib().pm_rope_table(_p(pos), _p(cs), _p(sn), c_int(T), c_int(half), c_float(theta), c_float(rope_scale),
                             _stream()), "pm_rope_table")
    return cs, sn


def rope_table_freqs(positions: torch.Tensor, inv_freq: torch.Tensor, mscale: float = 1.0):
    """cos/sin [T, half] from a host-built frequency vector [half] (fp32, on the device) times `mscale`."""
    T, half = positions.shape[0], inv_freq.shape[0]
    pos = positions if positions.dtype == torch.int32 else positions.to(torch.int32)
    cs = torch.empty(T, half, dtype=torch.float32, device=positions.device)
    sn = torch.empty_like(cs)
    _chk(lib().pm_rope_table_freqs(_p(pos), _p(inv_freq), _p(cs), _p(sn), c_int(T), c_int(half), c_float(mscale),
                                   _stream()), "pm_rope_table_freqs")
    return cs, sn


def qknorm_rope_fwd(qkv, qw, kw, cos, sin, hq: int, hkv: int, eps: float):
    T = qkv.shape[0]
    q = torch.empty(T, hq, 128, dtype=qkv.dtype, device=qkv.device)
    k = torch.empty(T, hkv, 128, dtype=qkv.dtype, device=qkv.device)
    _chk(lib().pm_qknorm_rope_fwd(_p(qkv), c_int(qkv.stride(0)), _p(qw), _p(kw), _p(cos), _p(sin), _p(q), _p(k),
                                  c_int(T), c_int(hq), c_int(hkv), c_float(eps), _stream()), "pm_qknorm_rope_fwd")
    return q, k


def qknorm_rope_cache(qkv, qw, kw, cos, sin, hq: int, hkv: int, eps: float, k_cache, v_cache, slots):
    """Decode: q = rope(norm(q)) returned; rope(norm(k)) and v are written into the paged caches at ``slots``."""
    T = qkv.shape[0]
    q = torch.empty(T, hq, 128, dtype=qkv.dtype, device=qkv.device)
    _chk(lib().pm_qknorm_rope_cache(_p(qkv), c_int(qkv.stride(0)), _p(qw), _p(kw), _p(cos), _p(sin), _p(q), _p(k_cache),
                                    _p(v_cache), _p(slots), c_int(T), c_int(hq), c_int(hkv), c_float(eps), _stream()),
         "pm_qknorm_rope_cache")
    return q


def qknorm_rope_bwd(dq, dk, qkv, qw, kw, cos, sin, hq: int, hkv: int, eps: float, dqkv) -> None:
    T = qkv.shape[0]
    _chk(lib().pm_qknorm_rope_bwd(_p(dq), _p(dk), _p(qkv), c_int(qkv.stride(0)), _p(qw), _p(kw), _p(cos), _p(sin),
                                  _p(dqkv), c_int(T), c_int(hq), c_int(hkv), c_float(eps), _stream()),
         "pm_qknorm_rope_bwd")


def swiglu_fwd(gate_up):
    T, I2 = gate_up.shape
    out = torch.empty(T, I2 // 2, dtype=gate_up.dtype, device=gate_up.device)
    _chk(lib().pm_swiglu_fwd(_p(gate_up), _p(out), c_ll(T), c_int(I2 // 2), _stream()), "pm_swiglu_fwd")
    return out


def swiglu_bwd(dout, gate_up):
    T, I2 = gate_up.shape
    dgu = torch.empty_like(gate_up)
    _chk(lib().pm_swiglu_bwd(_p(dout), _p(gate_up), _p(dgu), c_ll(T), c_int(I2 // 2), _stream()), "pm_swiglu_bwd")
    return dgu


GLU_ACTS = {"silu": 0, "swish": 0, "gelu_tanh": 1, "gelu_pytorch_tanh": 1, "gelu_new": 1, "gelu": 2}


def glu_fwd(gate, up, act: int):
    """act(gate) * up for two [T, I] bf16 matrices whose rows may be strided (views into a fused projection)."""
    T, I = gate.shape
    out = torch.empty(T, I, dtype=gate.dtype, device=gate.device)
    _chk(lib().pm_glu_fwd(_p(gate), _p(up), c_ll(gate.stride(0)), c_ll(up.stride(0)), _p(out), c_ll(T), c_int(I), c_int(act),
                          _stream()), "pm_glu_fwd")
    return out


def glu_bwd(dout, gate, up, act: int):
    T, I = gate.shape
    dg, du = torch.empty(T, I, dtype=gate.dtype, device=gate.device), torch.empty(T, I, dtype=gate.dtype, device=gate.device)
    _chk(lib().pm_glu_bwd(_p(dout), _p(gate), _p(up), c_ll(gate.stride(0)), c_ll(up.stride(0)), _p(dg), _p(du), c_ll(I),
                          c_ll(I), c_ll(T), c_int(I), c_int(act), _stream()), "pm_glu_bwd")
    return dg, du


# ------------------------------------------------------------------------------------------- attention
def attn_fwd(q, k, v, seq_start, scale: float, window: int = 0):
    """Varlen causal attention forward. The tcgen05 kernel handles the common case; sliding windows use the
    mma.sync kernel."""
    T, hq, d = q.shape
    hkv = k.shape[1]
    assert d == 128 and q.stride(2) == 1 and k.stride(2) == 1 and v.stride(2) == 1
    out = torch.empty(T, hq, d, dtype=q.dtype, device=q.device)
    lse = torch.empty(hq, T, dtype=torch.float32, device=q.device)
    if ATTN_TC and window == 0 and q.stride(1) == d and k.stride(1) == d and v.stride(1) == d:
        fn = lib().pm_attn_fwd_tc_rect_v1 if ATTN_FWD_V1 else lib().pm_attn_fwd_tc_rect
        _chk(fn(_p(q), c_ll(q.stride(0)), _p(k), c_ll(k.stride(0)), _p(v), c_ll(v.stride(0)), _p(out),
                c_ll(out.stride(0)), _p(lse), _p(seq_start), c_int(T), c_int(T), c_int(0), c_int(hq), c_int(hkv),
                c_float(scale), _p(status_word(q.device)), _stream()), "pm_attn_fwd_tc")
        return out, lse
    _chk(lib().pm_attn_fwd(_p(q), c_ll(q.stride(0)), _p(k), c_ll(k.stride(0)), _p(v), c_ll(v.stride(0)), _p(out),
                           c_ll(out.stride(0)), _p(lse), _p(seq_start), c_int(T), c_int(hq), c_int(hkv),
                           c_float(scale), c_int(window), _stream()), "pm_attn_fwd")
    return out, lse


def attn_fwd_rect(q, k, v, seq_start, scale: float, shift: int):
    """Attention of Tq queries over Tk keys where key j is visible to query i iff seq_start[i] <= j <= i + shift
    (shift >= Tk - 1: every key). q [Tq, hq, 128], k/v [Tk, hkv, 128] (k/v may live in a peer GPU's memory: the
    kernel's TMA loads read them in place). Returns (out bf16 [Tq, hq, 128], lse fp32 [hq, Tq])."""
    T, hq, d = q.shape
    Tk, hkv = k.shape[0], k.shape[1]
    assert d == 128 and q.stride(1) == d and k.stride(1) == d and v.stride(1) == d
    out = torch.empty(T, hq, d, dtype=q.dtype, device=q.device)
    lse = torch.empty(hq, T, dtype=torch.float32, device=q.device)
    _chk(lib().pm_attn_fwd_tc_rect(_p(q), c_ll(q.stride(0)), _p(k), c_ll(k.stride(0)), _p(v), c_ll(v.stride(0)), _p(out),
                                   c_ll(out.stride(0)), _p(lse), _p(seq_start), c_int(T), c_int(Tk), c_int(shift),
                                   c_int(hq), c_int(hkv), c_float(scale), _p(status_word(q.device)), _stream()),
         "pm_attn_fwd_tc_rect")
    return out, lse


def attn_bwd(dout, q, k, v, o, lse, seq_start, scale: float, window: int = 0, dv_out=None):
    T, hq, d = q.shape
    hkv = k.shape[1]
    delta = torch.empty(hq, T, dtype=torch.float32, device=q.device)
    _chk(lib().pm_attn_delta(_p(o), _p(dout), _p(delta), c_int(T), c_int(hq), _stream()), "pm_attn_delta")
    dq = torch.empty_like(q)
    dk = torch.empty_like(k)
    dv = dv_out if dv_out is not None else torch.empty(T, hkv, d, dtype=q.dtype, device=q.device)
    if ATTN_TC and window == 0 and all(t.stride(1) == d for t in (q, k, v, dout, dv)):
        _chk(lib().pm_attn_bwd_tc(_p(dout), c_ll(dout.stride(0)), _p(q), c_ll(q.stride(0)), _p(k), c_ll(k.stride(0)),
                                  _p(v), c_ll(v.stride(0)), _p(lse), _p(delta), _p(dq), c_ll(dq.stride(0)), _p(dk),
                                  c_ll(dk.stride(0)), _p(dv), c_ll(dv.stride(0)), _p(seq_start), c_int(T), c_int(hq),
                                  c_int(hkv), c_float(scale), _p(status_word(q.device)), _stream()), "pm_attn_bwd_tc")
    else:
        _chk(lib().pm_attn_bwd(_p(dout), _p(q), c_ll(q.stride(0)), _p(k), c_ll(k.stride(0)), _p(v), c_ll(v.stride(0)),
                               c_ll(dout.stride(0)), _p(lse), _p(delta), _p(dq), c_ll(dq.stride(0)), _p(dk),
                               c_ll(dk.stride(0)), _p(dv), c_ll(dv.stride(0)), _p(seq_start), c_int(T), c_int(hq),
                               c_int(hkv), c_float(scale), c_int(window), _stream()), "pm_attn_bwd")
    global LAUNCHES
    LAUNCHES += 1   # pm_attn_bwd launches two kernels
    return (dq, dk) if dv_out is not None else (dq, dk, dv)


# ------------------------------------------------------------------------------------------- loss / optimizer
def gemm_dw(dy: torch.Tensor, x: torch.Tensor, out: torch.Tensor, rows: Optional[int] = None) -> None:
    """out [N, K] (fp32) += dy[:, :N]^T x  — the weight gradient of y = x W^T, reduction over the token rows. Both
    operands are read in place (token index as the reduction dimension); every output tile belongs to one CTA, which
    adds into ``out`` with a plain read-add-write, so the sum is formed in a fixed order."""
    T, K = x.shape
    N = out.shape[0] if rows is None else rows
    assert out.dtype == torch.float32 and out.stride(1) == 1 and dy.stride(1) == 1 and x.stride(1) == 1
    if not MN_MAJOR:
        out[:N].add_(dy[:, :N].t().float() @ x.float())
        return
    bn = 128 if K >= 128 else 64
    raw_gemm(dy, 1, dy.stride(0), N, x, 1, x.stride(0), K, out, 4, out.stride(0), N, K, T, bn=bn)


def linear_ce(hidden, weight, weight_t, labels, ignore_index: int, chunk: int, need_grad: bool, z_coef: float = 0.0,
              w_grad: Optional[torch.Tensor] = None, label_smoothing: float = 0.0, softcap: float = 0.0,
              logit_scale: float = 1.0):
    """Chunked linear + cross-entropy. Logits of one token chunk live in a bf16 scratch buffer, are turned
    into their gradient in place, and feed the input-gradient GEMM; the [T, V] matrix never exists.
    ``z_coef`` adds ``z_coef * logsumexp(logits)^2`` per valid row to the differentiated sum (the second return value
    is the sum of the squared normalisers); ``w_grad`` (fp32 [V, H]) receives the gradient of the head weight;
    ``label_smoothing`` mixes the target with the uniform distribution; ``softcap`` c turns logits into c tanh(x / c);
    ``logit_scale`` multiplies the logits first (inside the GEMM; the gradient picks the factor up on its way back)."""
    T, H = hidden.shape
    V = weight.shape[0]
    labels = labels.contiguous()
    n_valid = (labels != ignore_index).sum()
    # gradient is of the *sum* (the caller divides); d/d(h W^T) = logit_scale * d/d(logits)
    inv_n = torch.full((1,), float(logit_scale), dtype=torch.float32, device=hidden.device)
    loss = torch.zeros(2, dtype=torch.float32, device=hidden.device)  # [cross entropy, squared normalisers]
    dh = torch.empty_like(hidden) if need_grad else None
    chunk = min(chunk, T)
    ldl = -(-V // 8) * 8
    scratch = torch.empty(chunk, ldl, dtype=torch.bfloat16, device=hidden.device)
    bn = _pick_bn(V)
    grads = need_grad or w_grad is not None
    for s in range(0, T, chunk):
        n = min(chunk, T - s)
        h = hidden[s:s + n]
        raw_gemm(h, 0, h.stride(0), n, weight, 0, weight.stride(0), V, scratch, 0, ldl, n, V, H, bn=bn, alpha=logit_scale)
        if label_smoothing > 0.0 or softcap > 0.0:
            _chk(lib().pm_ce_opt_fwd_bwd(_p(scratch), c_ll(ldl), _p(labels[s:s + n]), _p(loss), _p(loss[1:]), _p(inv_n),
                                         c_int(n), c_int(V), c_ll(ignore_index), c_int(1 if grads else 0), c_float(z_coef),
                                         c_float(label_smoothing), c_float(softcap), _stream()), "pm_ce_opt_fwd_bwd")
        else:
            _chk(lib().pm_ce_z_fwd_bwd(_p(scratch), c_ll(ldl), _p(labels[s:s + n]), _p(loss), _p(loss[1:]), _p(inv_n),
                                       c_int(n), c_int(V), c_ll(ignore_index), c_int(1 if grads else 0), c_float(z_coef),
                                       _stream()), "pm_ce_z_fwd_bwd")
        if need_grad:
            d = dh[s:s + n]
            if weight_t is not None:
                raw_gemm(scratch, 0, ldl, n, weight_t, 0, weight_t.stride(0), H, d, 0, d.stride(0), n, H, V,
                         bn=_pick_bn(H))
            elif MN_MAJOR:
                raw_gemm(scratch, 0, ldl, n, weight, 1, weight.stride(0), H, d, 0, d.stride(0), n, H, V,
                         bn=max(64, _pick_bn(H)))
            else:
                wt = weight.t().contiguous()
                raw_gemm(scratch, 0, ldl, n, wt, 0, V, H, d, 0, d.stride(0), n, H, V, bn=_pick_bn(H))
        if w_grad is not None:
            gemm_dw(scratch[:n], h, w_grad, rows=V)
    return loss[0], loss[1], n_valid, dh


def sumsq(x: torch.Tensor, out: torch.Tensor) -> None:
    _chk(lib().pm_sumsq(_p(x), c_ll(x.numel()), _p(out), _stream()), "pm_sumsq")
    global LAUNCHES
    LAUNCHES += 0


def adamw_flat(p, g, m, v, shadow, lr_mult, wd, gnorm_sq, lr, b1, b2, eps, step, grad_scale, max_norm,
               hp=None) -> None:
    """``hp`` (optional device tensor [lr, 1-b1^t, 1-b2^t]) overrides the scalar arguments (CUDA-graph replay)."""
    _chk(lib().pm_adamw_flat(_p(p), _p(g), _p(m), _p(v), _p(shadow), _p(lr_mult), _p(wd), _p(gnorm_sq), _p(hp),
                             c_ll(p.numel()), c_float(lr), c_float(b1), c_float(b2), c_float(eps), c_int(step),
                             c_float(grad_scale), c_float(max_norm or 0.0), _stream()), "pm_adamw_flat")


# ------------------------------------------------------------------------------------------- paged KV
def kv_append(k, v, k_cache, v_cache, slots) -> None:
    """k, v: [n, hkv, 128] (token stride arbitrary) -> cache [num_blocks, 64, hkv, 128] at ``slots``."""
    n, hkv, _ = k.shape
    _chk(lib().pm_kv_append(_p(k), c_ll(k.stride(0)), _p(v), c_ll(v.stride(0)), _p(k_cache), _p(v_cache), _p(slots),
                            c_int(n), c_int(hkv), _stream()), "pm_kv_append")


def kv_append_q8(k, v, k_cache, v_cache, k_scale, v_scale, slots) -> None:
    """bf16 k, v [n, hkv, 128] -> int8 cache [num_blocks, 64, hkv, 128] with fp32 scales [num_blocks, 64, hkv, 2]."""
    n, hkv, d = k.shape
    assert d == 128 and k.dtype == torch.bfloat16 and k.stride(2) == 1 and v.stride(2) == 1 and k.stride(1) == d
    lib().pm_kv_append_q8.restype = c_int
    _chk(lib().pm_kv_append_q8(_p(k), c_ll(k.stride(0)), _p(v), c_ll(v.stride(0)), _p(k_cache), _p(v_cache), _p(k_scale),
                               _p(v_scale), _p(slots), c_int(n), c_int(hkv), _stream()), "pm_kv_append_q8")


def paged_attn(q, k_cache, v_cache, meta, scale: float, window: int = 0, n_split: int = 0, sink: int = 0,
               k_scale=None, v_scale=None, lut=None):
    """q: [total_q, hq, 128]; ``meta`` is a ``BatchMeta``. Long single sequences are split over key blocks.
    With ``k_scale`` / ``v_scale`` the caches are int8, or, with ``lut`` (16 floats), 4-bit codes into that code book;
    ``sink`` keys stay visible in front of a sliding window."""
    total_q, hq, _ = q.shape
    hkv = k_cache.shape[2]
    n_seq = meta.block_table.shape[0]
    if n_split <= 0:
        ctas = n_seq * hkv
        n_blocks = -(-meta.max_kv // 64)
        n_split = max(1, min(n_blocks // 4, 2 * sm_count() // max(ctas, 1), 32)) if ctas < sm_count() else 1
    out = torch.empty_like(q)
    po = pml = None
    if n_split > 1:
        po = torch.empty(n_split, total_q, hq, 128, dtype=torch.float32, device=q.device)
        pml = torch.empty(n_split, total_q, hq, 2, dtype=torch.float32, device=q.device)
    if lut is not None:
        lib().pm_paged_attn_q4.restype = c_int
        arr = (c_float * 16)(*[float(x) for x in lut])
        _chk(lib().pm_paged_attn_q4(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(meta.block_table), _p(meta.seq_lens),
                                    _p(meta.q_start), _p(meta.q_lens), _p(po), _p(pml), c_int(n_seq),
                                    c_int(meta.block_table.shape[1]), c_int(total_q), c_int(meta.max_q), c_int(hq),
                                    c_int(hkv), c_int(n_split), c_float(scale), c_int(window), c_int(sink), _p(k_scale),
                                    _p(v_scale), arr, _stream()), "pm_paged_attn_q4")
        return out
    lib().pm_paged_attn_ex.restype = c_int
    _chk(lib().pm_paged_attn_ex(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(meta.block_table), _p(meta.seq_lens),
                                _p(meta.q_start), _p(meta.q_lens), _p(po), _p(pml), c_int(n_seq),
                                c_int(meta.block_table.shape[1]), c_int(total_q), c_int(meta.max_q), c_int(hq),
                                c_int(hkv), c_int(n_split), c_float(scale), c_int(window), c_int(sink), _p(k_scale),
                                _p(v_scale), _stream()), "pm_paged_attn")
    return out


def kv_append_tq4(k, v, k_cache, v_cache, k_scale, v_scale, slots, sign, thresholds) -> None:
    """bf16 k, v [n, hkv, 128] -> rotated 4-bit cache [num_blocks, 64, hkv, 64] bytes with fp32 scales
    [num_blocks, 64, hkv, 2]; ``sign`` [128] (+-1) and ``thresholds`` [15] are device fp32 tensors."""
    n, hkv, d = k.shape
    assert d == 128 and k.dtype == torch.bfloat16 and k.stride(2) == 1 and v.stride(2) == 1 and k.stride(1) == d
    lib().pm_kv_append_tq4.restype = c_int
    _chk(lib().pm_kv_append_tq4(_p(k), c_ll(k.stride(0)), _p(v), c_ll(v.stride(0)), _p(k_cache), _p(v_cache),
                                _p(k_scale), _p(v_scale), _p(slots), _p(sign), _p(thresholds), c_int(n), c_int(hkv),
                                _stream()), "pm_kv_append_tq4")


def tq_rotate(x, sign, inverse: bool = False):
    """Signed Walsh-Hadamard rotation of every 128-vector of x [T, h, 128] (bf16): forward H(x sign)/sqrt(d), inverse
    (H x)/sqrt(d) sign."""
    T, h, d = x.shape
    assert d == 128 and x.stride(2) == 1 and x.stride(1) == d
    out = torch.empty(T, h, d, dtype=x.dtype, device=x.device)
    lib().pm_tq_rotate.restype = c_int
    _chk(lib().pm_tq_rotate(_p(x), c_ll(x.stride(0)), _p(sign), _p(out), c_ll(out.stride(0)), c_ll(T), c_int(h),
                            c_int(int(inverse)), _stream()), "pm_tq_rotate")
    return out


# ------------------------------------------------------------------------------------------- QLoRA
def dequant_4bit(q) -> torch.Tensor:
    """``QuantizedTensor`` (nf4/fp4) -> bf16 tensor of its shape."""
    n = 1
    for d in q.shape:
        n *= d
    out = torch.empty(q.shape, dtype=torch.bfloat16, device=q.data.device)
    _chk(lib().pm_dequant_4bit(_p(q.data), _p(q.absmax), _p(q.absmax_q), c_float(q.absmax_scale),
                               c_float(q.absmax_offset), _p(out), c_ll(n), c_int(q.block_size),
                               c_int(1 if q.scheme == "fp4" else 0), _stream()), "pm_dequant_4bit")
    return out


def token_nll(hidden, weight, tokens, chunk: int = 4096, row_scale=None, weight_t=None):
    """Per-token negative log-likelihood of ``tokens`` under softmax(hidden @ weight^T), chunked over tokens.

    With ``row_scale`` (per-token upstream gradient of the NLL) it also returns d/d hidden; logits of a chunk
    exist only in a transient bf16 buffer. Tokens equal to -100 give 0."""
    T, H = hidden.shape
    V = weight.shape[0]
    tokens = tokens.contiguous()
    nll = torch.empty(T, dtype=torch.float32, device=hidden.device)
    dh = torch.empty_like(hidden) if row_scale is not None else None
    chunk = min(chunk, T)
    ldl = -(-V // 8) * 8
    scratch = torch.empty(chunk, ldl, dtype=torch.bfloat16, device=hidden.device)
    bn = _pick_bn(V)
    for s in range(0, T, chunk):
        n = min(chunk, T - s)
        h = hidden[s:s + n]
        raw_gemm(h, 0, h.stride(0), n, weight, 0, weight.stride(0), V, scratch, 0, ldl, n, V, H, bn=bn)
        _chk(lib().pm_ce_fwd_bwd(_p(scratch), c_ll(ldl), _p(tokens[s:s + n]), _p(None), _p(None), _p(nll[s:s + n]),
                                 _p(row_scale[s:s + n] if row_scale is not None else None), c_int(n), c_int(V),
                                 c_ll(-100), c_int(1 if row_scale is not None else 0), _stream()), "pm_ce_fwd_bwd")
        if row_scale is not None:
            d = dh[s:s + n]
            if weight_t is not None:
                raw_gemm(scratch, 0, ldl, n, weight_t, 0, weight_t.stride(0), H, d, 0, d.stride(0), n, H, V,
                         bn=_pick_bn(H))
            else:
                raw_gemm(scratch, 0, ldl, n, weight, 1, weight.stride(0), H, d, 0, d.stride(0), n, H, V,
                         bn=max(64, _pick_bn(H)))
    return nll, dh


# ------------------------------------------------------------------------------------------- sampling
c_ull = ctypes.c_ulonglong


def sample(logits, temperature, top_k=None, top_p=None, min_p=None, counts=None, rep_pen=None, freq_pen=None,
           pres_pen=None, seeds=None, step: int = 0, want_logprob: bool = True, count_rows=None):
    """logits [rows, V] fp32 or bf16 (row stride arbitrary); per-row parameter tensors on the device.
    ``counts`` [*, V] int32 holds token occurrences; logits row r uses counts row ``count_rows[r]`` (int32, default r).
    Returns (tokens int32 [rows], logprobs fp32 [rows] or None)."""
    rows, V = logits.shape
    assert logits.stride(1) == 1 and logits.dtype in (torch.float32, torch.bfloat16)
    tok = torch.empty(rows, dtype=torch.int32, device=logits.device)
    lp = torch.empty(rows, dtype=torch.float32, device=logits.device) if want_logprob else None
    _chk(lib().pm_sample(_p(logits), c_int(int(logits.dtype == torch.bfloat16)), c_ll(logits.stride(0)), c_int(rows),
                         c_int(V), _p(counts), _p(count_rows), _p(temperature), _p(top_k), _p(top_p), _p(min_p), _p(rep_pen),
                         _p(freq_pen), _p(pres_pen), _p(seeds), c_ull(step), _p(tok), _p(lp), _stream()), "pm_sample")
    return tok, lp


def spec_verify(target_logits, draft_logits, draft_tokens, temperature: float = 0.0, seeds=None, step: int = 0):
    """target_logits [n, K+1, V] fp32, draft_logits [n, K, V] fp32 (None for greedy), draft_tokens [n, K] int32.
    Returns (n_accepted int32 [n], next_token int32 [n])."""
    n, k1, V = target_logits.shape
    K = k1 - 1
    assert target_logits.is_contiguous() and target_logits.dtype == torch.float32
    if draft_logits is not None:
        assert draft_logits.is_contiguous() and draft_logits.dtype == torch.float32
    acc = torch.empty(n, dtype=torch.int32, device=target_logits.device)
    nxt = torch.empty(n, dtype=torch.int32, device=target_logits.device)
    _chk(lib().pm_spec_verify(_p(target_logits), _p(draft_logits), _p(draft_tokens.contiguous()), c_int(n), c_int(K),
                              c_int(V), c_float(temperature), _p(seeds), c_ull(step), _p(acc), _p(nxt), _stream()),
         "pm_spec_verify")
    return acc, nxt


def count_tokens(counts, tokens, count_rows=None) -> None:
    """counts[count_rows[r] (default r), tokens[r]] += 1 for every row r."""
    _chk(lib().pm_count_tokens(_p(counts), _p(count_rows), _p(tokens), c_int(tokens.numel()), c_int(counts.shape[1]),
                               _stream()), "pm_count_tokens")


# ------------------------------------------------------------------------------------------- MoE routing
def moe_route(router_logits, k: int, renorm: bool = True, offsets_out=None):
    """router_logits [T, E] (bf16 or fp32). Returns dict(topk_idx [T,k], topk_w [T,k], counts [E], offsets [E+1],
    perm [T*k] (sorted position -> token*k+slot), inv [T*k] (token*k+slot -> sorted position))."""
    T, E = router_logits.shape
    dev = router_logits.device
    x = router_logits.contiguous()
    if x.dtype not in (torch.float32, torch.bfloat16):
        x = x.float()
    out = dict(topk_idx=torch.empty(T, k, dtype=torch.int32, device=dev), topk_w=torch.empty(T, k, dtype=torch.float32, device=dev),
               counts=torch.empty(E, dtype=torch.int32, device=dev), offsets=torch.empty(E + 1, dtype=torch.int32, device=dev),
               perm=torch.empty(T * k, dtype=torch.int32, device=dev), inv=torch.empty(T * k, dtype=torch.int32, device=dev))
    _chk(lib().pm_moe_route2(_p(x), c_int(int(x.dtype == torch.float32)), c_int(T), c_int(E), c_int(k), c_int(int(renorm)),
                             _p(out["topk_idx"]), _p(out["topk_w"]), _p(out["counts"]), _p(out["offsets"]),
                             _p(offsets_out), _p(out["perm"]), _p(out["inv"]), _stream()), "pm_moe_route2")
    return out


def moe_gather(x, perm, k: int):
    n, H = perm.numel(), x.shape[1]
    out = torch.empty(n, H, dtype=torch.bfloat16, device=x.device)
    _chk(lib().pm_moe_gather(_p(x.contiguous()), _p(perm), c_int(k), _p(out), c_ll(n), c_int(H), _stream()), "pm_moe_gather")
    return out


def moe_combine(z, inv, w, k: int, residual=None):
    """y[t] = sum_j w[t, j] * z[inv[t * k + j]] (+ residual[t]); residual is a contiguous bf16 [T, H] tensor."""
    T, H = inv.numel() // k, z.shape[1]
    y = torch.empty(T, H, dtype=torch.bfloat16, device=z.device)
    _chk(lib().pm_moe_combine2(_p(z.contiguous()), _p(inv), _p(w.contiguous()), c_int(k), _p(residual), _p(y), c_ll(T),
                               c_int(H), _stream()), "pm_moe_combine2")
    return y


# ------------------------------------------------------------------------------------------- GGUF / FP8
def gguf_dequant_bf16(raw, ggml_type: int, shape):
    """raw: uint8 device tensor of GGUF blocks (Q4_0=2, Q8_0=8, Q4_K=12, Q6_K=14) -> bf16 tensor of ``shape``."""
    n = 1
    for d in shape:
        n *= d
    out = torch.empty(shape, dtype=torch.bfloat16, device=raw.device)
    _chk(lib().pm_gguf_dequant_bf16(_p(raw), _p(out), c_ll(n), c_int(int(ggml_type)), _stream()), "pm_gguf_dequant_bf16")
    return out


def fp8_quant(x):
    """bf16 tensor (numel % 128 == 0) -> (uint8 E4M3 codes of the same shape, fp32 scales per 128 elements)."""
    x = x.contiguous()
    n = x.numel()
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    sc = torch.empty(n // 128, dtype=torch.float32, device=x.device)
    _chk(lib().pm_fp8_quant(_p(x), _p(q), _p(sc), c_ll(n), _stream()), "pm_fp8_quant")
    return q, sc


def fp8_dequant(q, scales):
    y = torch.empty(q.shape, dtype=torch.bfloat16, device=q.device)
    _chk(lib().pm_fp8_dequant(_p(q), _p(scales), _p(y), c_ll(q.numel()), _stream()), "pm_fp8_dequant")
    return y


# ------------------------------------------------------------------------------------------- distillation / merge
KD_KINDS = {"kl": 0, "forward_kl": 0, "reverse_kl": 1, "js": 2, "jsd": 2, "soft_ce": 3, "tvd": 4}


def kd_fwd_bwd(student_logits, teacher_logits, temperature: float, kind: str = "kl", beta: float = 0.5, row_scale=None,
               write_grad: bool = True):
    """student_logits [rows, V] bf16 is overwritten with the gradient (times row_scale); returns per-row losses."""
    rows, V = student_logits.shape
    assert student_logits.dtype == torch.bfloat16 and teacher_logits.dtype == torch.bfloat16
    assert student_logits.stride(1) == 1 and teacher_logits.stride(1) == 1
    row_loss = torch.empty(rows, dtype=torch.float32, device=student_logits.device)
    _chk(lib().pm_kd_fwd_bwd(_p(student_logits), c_ll(student_logits.stride(0)), _p(teacher_logits),
                             c_ll(teacher_logits.stride(0)), c_int(rows), c_int(V), c_float(temperature),
                             c_int(KD_KINDS[kind]), c_float(beta), _p(row_scale), _p(row_loss), _p(None),
                             c_int(int(write_grad)), _stream()), "pm_kd_fwd_bwd")
    return row_loss


def merge_fused(models, base, weights, thresholds=None, densities=None, consensus=False, rescale=True, lam=1.0, seed=0,
                out_dtype=torch.float32):
    """Fused task-vector merge of up to 8 same-shaped tensors (all bf16 or all fp32)."""
    m0 = models[0]
    bf = m0.dtype == torch.bfloat16
    ms = [m.contiguous() for m in models]
    assert all(m.dtype == m0.dtype and m.shape == m0.shape for m in ms)
    b = base.contiguous().to(m0.dtype) if base is not None else None
    out = torch.empty(m0.shape, dtype=out_dtype, device=m0.device)
    ptrs = (c_void_p * len(ms))(*[m.data_ptr() for m in ms])
    fa = lambda v: (c_float * len(ms))(*[float(x) for x in v]) if v is not None else None     # noqa: E731
    _chk(lib().pm_merge_fused(ptrs, _p(b), fa(weights), fa(thresholds), fa(densities), c_int(len(ms)), c_int(int(bf)),
                              c_int(int(out_dtype == torch.bfloat16)), c_int(int(consensus)), c_int(int(rescale)),
                              c_float(lam), c_ull(seed), _p(out), c_ll(m0.numel()), _stream()), "pm_merge_fused")
    return out


def dot_norms(a, b):
    out = torch.empty(3, dtype=torch.float32, device=a.device)
    _chk(lib().pm_dot_norms(_p(a.contiguous()), _p(b.contiguous()), c_int(int(a.dtype == torch.bfloat16)), c_ll(a.numel()),
                            _p(out), _stream()), "pm_dot_norms")
    return out


# ------------------------------------------------------------------------------------------- decode mat-vec
def gemv(x, w, norm_w=None, eps: float = 1e-6, residual=None, swiglu: bool = False, alpha: float = 1.0, t=None,
         lora_b=None, r: int = 0, seg_sizes: Sequence[int] = ()):
    """x [M <= 16, K] bf16, w [N_w, K] bf16 -> [M, N] bf16 (N = N_w / 2 with ``swiglu``). Optional fused RMSNorm of x,
    residual add, SwiGLU over (gate rows, up rows) and LoRA term t . lora_b^T (t carries the scale)."""
    M, K = x.shape
    Nw = w.shape[0]
    N = Nw // 2 if swiglu else Nw
    y = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    ends = _seg_ends(seg_sizes) if len(seg_sizes) > 1 else (c_int * 4)(*([0x7FFFFFFF] * 4))
    _chk(lib().pm_gemv(_p(x), c_int(x.stride(0)), _p(w), c_int(w.stride(0)), _p(norm_w), c_float(eps), _p(residual),
                       c_int(residual.stride(0) if residual is not None else 0), _p(y), c_int(N), c_int(M), c_int(N),
                       c_int(K), c_int(int(swiglu)), c_float(alpha), _p(t), c_int(t.stride(0) if t is not None else 0),
                       _p(lora_b), c_int(r), ends, _stream()), "pm_gemv")
    return y


def gemv_q4(x, q, norm_w=None, eps: float = 1e-6, residual=None, swiglu: bool = False, alpha: float = 1.0, t=None,
            lora_b=None, r: int = 0, seg_sizes: Sequence[int] = ()):
    """As ``gemv`` with the weight given as a 4-bit ``QuantizedTensor`` (nf4 / fp4) of shape [N_w, K]: the codes are
    expanded to bf16 inside the kernel, so a decode step streams a quarter of the bytes."""
    M, K = x.shape
    Nw = q.shape[0]
    N = Nw // 2 if swiglu else Nw
    y = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    ends = _seg_ends(seg_sizes) if len(seg_sizes) > 1 else (c_int * 4)(*([0x7FFFFFFF] * 4))
    _chk(lib().pm_gemv_q4(_p(x), c_int(x.stride(0)), _p(q.data), _p(q.absmax), _p(q.absmax_q), c_float(q.absmax_scale),
                          c_float(q.absmax_offset), c_int(q.block_size), c_int(1 if q.scheme == "fp4" else 0), _p(norm_w),
                          c_float(eps), _p(residual), c_int(residual.stride(0) if residual is not None else 0), _p(y),
                          c_int(N), c_int(M), c_int(N), c_int(K), c_int(int(swiglu)), c_float(alpha), _p(t),
                          c_int(t.stride(0) if t is not None else 0), _p(lora_b), c_int(r), ends, _stream()), "pm_gemv_q4")
    return y


def gdn_scan(q, k, v, g, beta, state=None):
    """Gated delta rule over a token sequence (csrc/gdn.cu). q, k [B, T, H, dk], v [B, T, H, dv], g, beta [B, T, H], all
    fp32; ``state`` [B, H, dk, dv] fp32 or None (zeros). Returns (y [B, T, H, dv], final state)."""
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    f = lambda t: t.float().contiguous()
    q, k, v, g, beta = f(q), f(k), f(v), f(g), f(beta)
    st = torch.zeros(B, H, dk, dv, dtype=torch.float32, device=q.device) if state is None else state.float().contiguous().clone()
    y = torch.empty(B, T, H, dv, dtype=torch.float32, device=q.device)
    _chk(lib().pm_gdn_scan(_p(q), _p(k), _p(v), _p(g), _p(beta), _p(st), _p(y), c_int(B), c_int(T), c_int(H), c_int(dk),
                           c_int(dv), _stream()), "pm_gdn_scan")
    return y, st


def gdn_scan_supported(dk: int, dv: int) -> bool:
    return dk in (64, 128) and dv in (64, 128)


# ------------------------------------------------------------------------------------------- whole-step decode kernel
def decode_layers_supported(M: int, H: int, hq: int, hkv: int, I: int) -> bool:
    return bool(lib().pm_decode_layers_supported(c_int(M), c_int(H), c_int(hq), c_int(hkv), c_int(I)))


def decode_layers(table, n_layers: int, x, scratch: dict, cos, sin, meta, hq: int, hkv: int, I: int, eps: float,
                  scale: float):
    """All decoder layers of one decode step in a single cooperative launch (csrc/decode_mega.cu). ``table`` is the
    int64 device tensor of per-layer pointers, ``x`` [M, H] bf16 is updated in place, ``scratch`` holds the work
    buffers made by ``decode_scratch``."""
    M, H = x.shape
    scratch["bar"].zero_()
    _chk(lib().pm_decode_layers(_p(table), c_int(n_layers), c_int(M), c_int(H), c_int(hq), c_int(hkv), c_int(I),
                                c_float(eps), c_float(scale), _p(x), _p(scratch["h"]), _p(scratch["qkv"]),
                                _p(scratch["attn"]), _p(scratch["act"]), _p(scratch["part_o"]), _p(scratch["part_ml"]),
                                _p(scratch["counters"]), _p(cos), _p(sin), _p(meta.block_table), _p(meta.seq_lens),
                                _p(meta.slots), c_int(meta.block_table.shape[1]), c_int(scratch["n_split"]),
                                _p(scratch["bar"]), _p(status_word(x.device)), _p(scratch.get("trace")), _stream()),
         "pm_decode_layers")
    return x


def decode_splits(M: int, hkv: int, max_kv: int) -> int:
    """CTAs per (row, kv head) in the attention phase: fill the grid, at least 64 keys per CTA, at most 16."""
    return max(1, min(sm_count() // max(M * hkv, 1), 16, max(max_kv // 64, 1)))


def decode_scratch(M: int, H: int, hq: int, hkv: int, I: int, n_split: int, device) -> dict:
    bf = dict(dtype=torch.bfloat16, device=device)
    return dict(h=torch.empty(M, H, **bf), qkv=torch.empty(M, (hq + 2 * hkv) * 128, **bf), attn=torch.empty(M, hq * 128, **bf),
                act=torch.empty(M, I, **bf), part_o=torch.empty(n_split, M, hq, 128, dtype=torch.float32, device=device),
                part_ml=torch.empty(n_split, M, hq, 2, dtype=torch.float32, device=device),
                counters=torch.zeros(M * hkv, dtype=torch.int32, device=device),
                bar=torch.zeros(2, dtype=torch.int32, device=device), n_split=n_split)
