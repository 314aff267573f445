"""Differentiable operators used by the models.

Each function runs the hand-written sm_100a kernel (``ops.native``) when its inputs
live on a CUDA device and falls back to the PyTorch statement in ``ops.reference``
on CPU. A CUDA tensor with the native library missing raises instead of silently
taking the slow path, unless ``PMETAL_ALLOW_TORCH_FALLBACK=1`` is set.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from . import reference as ref

_FORCE_REF = os.environ.get("PMETAL_FORCE_REFERENCE", "0") == "1"


def _native():
    from . import native
    return native


class force_reference:
    """Context manager: run every op through the PyTorch reference path (tests, debugging)."""

    def __enter__(self):
        global _FORCE_REF
        self._old = _FORCE_REF
        _FORCE_REF = True

    def __exit__(self, *a):
        global _FORCE_REF
        _FORCE_REF = self._old


def set_force_reference(on: bool = True) -> None:
    """Process-wide switch to the PyTorch reference operators (``--no-fused`` / ``--no-flash-attention``). The environment
    variable is set as well so that child processes follow."""
    global _FORCE_REF
    _FORCE_REF = bool(on)
    os.environ["PMETAL_FORCE_REFERENCE"] = "1" if on else "0"


def native_enabled(t: torch.Tensor) -> bool:
    """CUDA tensor, native library loaded and the reference path not forced (any dtype)."""
    return (not _FORCE_REF) and t.is_cuda and _native().available()


PAD_SMALL_HEADS = os.environ.get("PMETAL_PAD_SMALL_HEADS", "1") == "1"


def use_native(t: torch.Tensor) -> bool:
    if _FORCE_REF or not t.is_cuda:
        return False
    nat = _native()
    if nat.available():
        return t.dtype == torch.bfloat16
    if os.environ.get("PMETAL_ALLOW_TORCH_FALLBACK", "0") == "1":
        return False
    raise RuntimeError("pmetal_b200 native CUDA library is not built/loaded; run __graft_entry__.build() "
                       f"({nat.load_error()})")


# --------------------------------------------------------------------------- RMSNorm (+ residual add)
class _RmsNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, residual):
        nat = _native()
        h, y, rstd = nat.rmsnorm_fwd(x, weight, eps, residual)
        ctx.save_for_backward(h, weight, rstd)
        ctx.has_res = residual is not None
        ctx.w_grad = weight.requires_grad
        ctx.mark_non_differentiable(rstd)
        ctx.set_materialize_grads(False)     # an unused output must not cost a zero-filled [T, H] gradient
        return y, h

    @staticmethod
    def backward(ctx, dy, dh):
        h, weight, rstd = ctx.saved_tensors
        nat = _native()
        if dy is None:                       # only the pass-through output was used
            return dh, None, None, (dh if ctx.has_res else None)
        dx, dw = nat.rmsnorm_bwd(dy.contiguous(), h, weight, rstd, dh, ctx.w_grad)
        return dx, dw, None, (dx if ctx.has_res else None)


def add_rms_norm(x: torch.Tensor, residual: Optional[torch.Tensor], weight: torch.Tensor, eps: float):
    """h = x + residual (or x); returns (rms_norm(h)·w, h).

    Callers that also feed the un-normalised stream onward (the residual branch of a pre-norm block) should use the
    returned ``h`` for it: both gradients then meet inside the norm's backward kernel instead of in a separate add."""
    if use_native(x):
        y, h = _RmsNormFn.apply(x, weight, eps, residual)
        return y, h
    h = x if residual is None else x + residual
    return ref.rms_norm(h, weight, eps), h


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return add_rms_norm(x, None, weight, eps)[0]


# --------------------------------------------------------------------------- SwiGLU
class _SwigluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        ctx.save_for_backward(gate_up)
        return _native().swiglu_fwd(gate_up)

    @staticmethod
    def backward(ctx, dout):
        (gate_up,) = ctx.saved_tensors
        return _native().swiglu_bwd(dout.contiguous(), gate_up)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    if use_native(gate_up):
        return _SwigluFn.apply(gate_up)
    return ref.swiglu(gate_up)


class _GluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up, act):
        ctx.save_for_backward(gate, up)
        ctx.act = act
        return _native().glu_fwd(gate, up, act)

    @staticmethod
    def backward(ctx, dout):
        gate, up = ctx.saved_tensors
        dg, du = _native().glu_bwd(dout.contiguous(), gate, up, ctx.act)
        return dg, du, None


def glu(gate: torch.Tensor, up: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """``act(gate) * up`` for separate gate / up activations [..., I]: SwiGLU (``silu``), GeGLU (``gelu_tanh``) or exact
    GELU gating. One kernel forward and one backward on a GPU (crates/pmetal-bridge/cpp/bridge_compiled.cpp:35-118:
    fused_swiglu / fused_geglu_tanh); the PyTorch operators elsewhere."""
    code = _native().GLU_ACTS.get(act) if gate.is_cuda else None
    if (code is not None and use_native(gate) and up.dtype == gate.dtype and gate.shape == up.shape and gate.shape[-1] % 8 == 0
            and gate.stride(-1) == 1 and up.stride(-1) == 1):
        g2, u2 = gate.reshape(-1, gate.shape[-1]), up.reshape(-1, up.shape[-1])
        if g2.stride(0) % 8 == 0 and u2.stride(0) % 8 == 0:
            return _GluFn.apply(g2, u2, code).view(gate.shape)
    if act in ("silu", "swish"):
        return F.silu(gate) * up
    if act in ("gelu_tanh", "gelu_pytorch_tanh", "gelu_new"):
        return F.gelu(gate, approximate="tanh") * up
    if act == "gelu":
        return F.gelu(gate) * up
    raise ValueError(f"unknown gated activation {act!r}")


# --------------------------------------------------------------------------- attention block
def rope_table(positions: torch.Tensor, head_dim: int, theta: float, rope_scale: float = 1.0):
    """cos/sin [T, head_dim/2] in fp32 for the positions of this batch (shared by every layer)."""
    if positions.is_cuda and not _FORCE_REF and _native().available():
        return _native().rope_table(positions, head_dim, theta, rope_scale)
    return ref.rope_cos_sin(positions, head_dim, theta, rope_scale)


def rope_table_scheduled(positions: torch.Tensor, inv_freq: torch.Tensor, mscale: float = 1.0):
    """cos/sin [T, half] for a precomputed frequency schedule (llama3, yarn, NTK, longrope) and its attention factor."""
    if positions.is_cuda and not _FORCE_REF and _native().available():
        return _native().rope_table_freqs(positions, inv_freq, mscale)
    ang = positions.float()[:, None] * inv_freq.to(positions.device)[None, :]
    return ang.cos() * mscale, ang.sin() * mscale


class _AttnBlockFn(torch.autograd.Function):
    """fused projection [T,(hq+2hkv)*d] -> per-head RMSNorm(q,k) -> RoPE -> varlen causal attention -> [T,hq*d].

    Backward writes dv straight into the v slice of the fused gradient, so the
    gradient of the fused projection is assembled without a zero-fill or a concat.
    """

    @staticmethod
    def forward(ctx, qkv, qw, kw, cos, sin, seq_start, hq, hkv, d, eps, scale, window):
        nat = _native()
        q, k = nat.qknorm_rope_fwd(qkv, qw, kw, cos, sin, hq, hkv, eps)
        T = qkv.shape[0]
        v = qkv[:, (hq + hkv) * d:].view(T, hkv, d)
        o, lse = nat.attn_fwd(q, k, v, seq_start, scale, window)
        ctx.save_for_backward(qkv, qw, kw, cos, sin, seq_start, q, k, o, lse)
        ctx.cfg = (hq, hkv, d, eps, scale, window)
        return o.view(T, hq * d)

    @staticmethod
    def backward(ctx, do):
        qkv, qw, kw, cos, sin, seq_start, q, k, o, lse = ctx.saved_tensors
        hq, hkv, d, eps, scale, window = ctx.cfg
        nat = _native()
        T = qkv.shape[0]
        dqkv = torch.empty_like(qkv)
        v = qkv[:, (hq + hkv) * d:].view(T, hkv, d)
        dv = dqkv[:, (hq + hkv) * d:].view(T, hkv, d)
        dq, dk = nat.attn_bwd(do.contiguous().view(T, hq, d), q, k, v, o, lse, seq_start, scale, window, dv)
        nat.qknorm_rope_bwd(dq, dk, qkv, qw, kw, cos, sin, hq, hkv, eps, dqkv)
        dqw = dkw = None
        if qw is not None and (ctx.needs_input_grad[1] or ctx.needs_input_grad[2]):
            # gradient of the per-head norm weights: un-rotate the gradient, multiply by the normalised activations
            def norm_weight_grad(g, raw):
                g = ref.apply_rope(g, cos, -sin).float()
                x = raw.float()
                xhat = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
                return (g * xhat).sum((0, 1))
            dqw = norm_weight_grad(dq, qkv[:, :hq * d].view(T, hq, d)).to(qw.dtype)
            dkw = norm_weight_grad(dk, qkv[:, hq * d:(hq + hkv) * d].view(T, hkv, d)).to(kw.dtype)
        return (dqkv, dqw, dkw) + (None,) * 9


class _AttnCoreFn(torch.autograd.Function):
    """Varlen causal attention on already normalised / rotated q, k and v [T, h, 128] (the tcgen05 kernels)."""

    @staticmethod
    def forward(ctx, q, k, v, seq_start, scale, window):
        nat = _native()
        o, lse = nat.attn_fwd(q, k, v, seq_start, scale, window)
        ctx.save_for_backward(q, k, v, o, lse, seq_start)
        ctx.cfg = (scale, window)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, seq_start = ctx.saved_tensors
        scale, window = ctx.cfg
        dq, dk, dv = _native().attn_bwd(do.contiguous(), q, k, v, o, lse, seq_start, scale, window)
        return dq, dk, dv, None, None, None


def _attention_padded_heads(qkv, q_weight, k_weight, cos, sin, seq_start, hq, hkv, d, eps, scale, window):
    """Head sizes below 128 (64, 80, 96, ...) on the 128-wide kernels: QK-norm and RoPE at the true width, then q, k and
    v are zero-padded to 128 channels (zeros add nothing to q.k, and the padded output channels are dropped)."""
    T = qkv.shape[0]
    q = qkv[:, :hq * d].view(T, hq, d)
    k = qkv[:, hq * d:(hq + hkv) * d].view(T, hkv, d)
    v = qkv[:, (hq + hkv) * d:].view(T, hkv, d)
    if q_weight is not None:
        q, k = ref.rms_norm(q, q_weight, eps), ref.rms_norm(k, k_weight, eps)
    q, k = ref.apply_rope(q, cos, sin), ref.apply_rope(k, cos, sin)
    pad = (0, 128 - d)
    qp, kp, vp = (F.pad(t, pad).contiguous() for t in (q, k, v))
    o = _AttnCoreFn.apply(qp, kp, vp, seq_start, scale, window)
    return o[..., :d].reshape(T, hq * d)


def attention_block(qkv: torch.Tensor, q_weight, k_weight, cos: torch.Tensor, sin: torch.Tensor,
                    cu_seqlens: torch.Tensor, seq_start: Optional[torch.Tensor], hq: int, hkv: int, d: int,
                    eps: float, scale: Optional[float] = None, window: int = 0, softcap: float = 0.0) -> torch.Tensor:
    """Packed-sequence self-attention on a fused q|k|v projection. Returns [T, hq*d]."""
    T = qkv.shape[0]
    scale = scale if scale is not None else d ** -0.5
    if use_native(qkv) and d == 128 and softcap == 0.0:
        if seq_start is None:
            seq_start = ref.seq_starts_from_cu(cu_seqlens, T)
        return _AttnBlockFn.apply(qkv, q_weight, k_weight, cos, sin, seq_start, hq, hkv, d, eps, scale, window)
    if use_native(qkv) and d < 128 and d % 8 == 0 and softcap == 0.0 and PAD_SMALL_HEADS:
        if seq_start is None:
            seq_start = ref.seq_starts_from_cu(cu_seqlens, T)
        return _attention_padded_heads(qkv, q_weight, k_weight, cos, sin, seq_start, hq, hkv, d, eps, scale, window)
    q = qkv[:, :hq * d].view(T, hq, d)
    k = qkv[:, hq * d:(hq + hkv) * d].view(T, hkv, d)
    v = qkv[:, (hq + hkv) * d:].view(T, hkv, d)
    if q_weight is not None:
        q, k = ref.rms_norm(q, q_weight, eps), ref.rms_norm(k, k_weight, eps)
    q, k = ref.apply_rope(q, cos, sin), ref.apply_rope(k, cos, sin)
    return ref.varlen_attention(q, k, v, cu_seqlens, scale, True, window, softcap).reshape(T, hq * d)


# --------------------------------------------------------------------------- trainable parameters with bf16 shadows
class _ShadowFn(torch.autograd.Function):
    """The bf16 shadow of an fp32 master parameter as a differentiable stand-in: kernels read the shadow, the gradient
    flows to the master."""

    @staticmethod
    def forward(ctx, master, shadow):
        return shadow.view_as(shadow)

    @staticmethod
    def backward(ctx, g):
        return g.to(torch.float32), None


def live(p: torch.Tensor) -> torch.Tensor:
    """What the native kernels should read for parameter ``p``: its bf16 shadow (kept in step by the optimiser) when it
    trains in fp32 on the GPU, else ``p`` itself."""
    sh = getattr(p, "shadow", None)
    if sh is None or not p.requires_grad or not native_enabled(sh):
        return p
    return _ShadowFn.apply(p, sh)


class _DenseLinearFn(torch.autograd.Function):
    """y = x W^T (+ residual) with a trainable W: forward and input gradient read the bf16 shadow on the tcgen05 GEMM, the
    weight gradient dY^T X is accumulated straight into the master's fp32 ``.grad`` (fixed summation order)."""

    @staticmethod
    def forward(ctx, x, master, shadow, residual):
        nat = _native()
        x2 = x.reshape(-1, x.shape[-1])
        y = nat.gemm(x2, shadow, residual=residual.reshape(-1, shadow.shape[0]) if residual is not None else None)
        ctx.save_for_backward(x2, shadow)
        ctx.master = master
        ctx.has_res = residual is not None
        ctx.shape = x.shape
        return y.view(*x.shape[:-1], shadow.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, shadow = ctx.saved_tensors
        nat = _native()
        dy2 = dy.reshape(-1, shadow.shape[0]).contiguous()
        dx = nat.gemm_lora_dx(dy2, shadow, None, None, None).view(ctx.shape) if ctx.needs_input_grad[0] else None
        m = ctx.master
        if m.grad is None:
            m.grad = torch.zeros_like(m, dtype=torch.float32)
        nat.gemm_dw(dy2, x2, m.grad)
        return dx, None, None, (dy if ctx.has_res else None)


def dense_linear(x: torch.Tensor, master: torch.Tensor, shadow: torch.Tensor, residual: Optional[torch.Tensor] = None):
    return _DenseLinearFn.apply(x, master, shadow, residual)


# --------------------------------------------------------------------------- fused base + LoRA linear
class _LoraLinearFn(torch.autograd.Function):
    """y = x W^T + sum_seg s (x A_seg^T) B_seg^T over a row-stacked group of projections (+ residual).

    ``a32``/``b32`` are the fp32 parameters (autograd edges); ``a``/``b`` their bf16 compute copies,
    ``a`` stacked [n_seg*r, K] and ``b`` stacked [N, r]. Factor gradients are accumulated in fp32
    straight into ``.grad`` when that buffer already exists (the flat optimizer pre-binds it).
    """

    @staticmethod
    def forward(ctx, x, w, w_t, a32, b32, a, b, seg_sizes, r, scale, residual, qweight=None):
        nat = _native()
        fused_q = qweight is not None and nat.q4_gemm_ok(qweight, x.shape[0], seg_sizes)
        if qweight is not None and not fused_q:
            # QLoRA off the fused shapes: dequantise into a transient buffer; only the packed weight is kept
            from ..lora.qlora import dequantize_weight
            w, w_t = dequantize_weight(qweight), None
        t = nat.lora_t(x, a, scale) if a is not None else None    # [M, 64-padded] = s x A^T
        if fused_q:       # the GEMM expands the 4-bit codes on their way into the tensor cores
            y = nat.gemm_q4_lora(x, qweight, t, b, seg_sizes, r, residual)
        else:
            y = nat.gemm_lora(x, w, t, b, seg_sizes, r, residual)
        ctx.fused_q = fused_q
        ctx.save_for_backward(x, None if qweight is not None else w, w_t, a, b, t)
        ctx.params = (a32, b32)
        ctx.qweight = qweight
        ctx.cfg = (seg_sizes, r, scale, residual is not None)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, w_t, a, b, t = ctx.saved_tensors
        a32, b32 = ctx.params
        seg_sizes, r, scale, has_res = ctx.cfg
        nat = _native()
        fused_q = ctx.fused_q and _native().MN_MAJOR
        if ctx.qweight is not None and not fused_q:
            from ..lora.qlora import dequantize_weight
            w = dequantize_weight(ctx.qweight)
        dy = dy.contiguous()
        da = db = dx = None
        if a is not None:
            dt = nat.lora_dt(dy, b, seg_sizes, r, scale)          # [M, 64-padded] = s dY_seg B_seg
            if ctx.needs_input_grad[0]:
                dx = nat.gemm_q4_lora_dx(dy, ctx.qweight, dt, a) if fused_q else nat.gemm_lora_dx(dy, w, w_t, dt, a)

            def target(p32):
                g = p32.grad
                if g is not None and g.dtype == torch.float32 and g.is_contiguous():
                    return g, None
                z = torch.zeros(p32.shape, dtype=torch.float32, device=p32.device)
                return z, z
            ga, da = target(a32)
            gb, db = target(b32)
            nat.lora_da(dt, x, a.shape[0], ga)
            nat.lora_db(dy, t, seg_sizes, r, gb)
        elif ctx.needs_input_grad[0]:
            dx = nat.gemm_q4_lora_dx(dy, ctx.qweight, None, None) if fused_q else nat.gemm_lora_dx(dy, w, w_t, None, None)
        return dx, None, None, da, db, None, None, None, None, None, (dy if has_res else None), None


def lora_linear(x: torch.Tensor, w: torch.Tensor, w_t: Optional[torch.Tensor], a: Optional[torch.Tensor],
                b: Optional[torch.Tensor], seg_sizes: Sequence[int], r: int, scale: float,
                residual: Optional[torch.Tensor] = None, a_c: Optional[torch.Tensor] = None,
                b_c: Optional[torch.Tensor] = None, qweight=None) -> torch.Tensor:
    if use_native(x):
        if a is not None:
            a_c = a_c if a_c is not None else a.detach().to(torch.bfloat16)
            b_c = b_c if b_c is not None else b.detach().to(torch.bfloat16)
        return _LoraLinearFn.apply(x, w, w_t, a, b, a_c, b_c, tuple(seg_sizes), r, scale, residual, qweight)
    if qweight is not None:
        from ..lora.nf4 import dequantize
        w = dequantize(qweight, x.dtype)
    y = F.linear(x, w)
    if a is not None:
        outs, n0 = [], 0
        for i, n in enumerate(seg_sizes):
            t = F.linear(x, a[i * r:(i + 1) * r].to(x.dtype))
            outs.append(scale * F.linear(t, b[n0:n0 + n].to(x.dtype)))
            n0 += n
        y = y + torch.cat(outs, dim=-1)
    if residual is not None:
        y = y + residual
    return y


# --------------------------------------------------------------------------- linear + cross-entropy
class _LinearCeFn(torch.autograd.Function):
    """Σ over valid rows of (cross entropy + z_coef · logsumexp²), with the gradients formed in the forward pass: the
    one for the hidden states is saved, the one for a trainable head weight is accumulated chunk by chunk into an fp32
    buffer and added to the master's ``.grad`` in backward (scaled by the incoming gradient)."""

    @staticmethod
    def forward(ctx, hidden, weight, weight_t, labels, ignore_index, chunk, z_coef, master, smoothing=0.0, softcap=0.0,
                logit_scale=1.0):
        w_grad = None
        if master is not None:
            w_grad = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
        ce, z, n_valid, dh = _native().linear_ce(hidden, weight, weight_t, labels, ignore_index, chunk,
                                                 hidden.requires_grad, z_coef, w_grad, smoothing, softcap, logit_scale)
        ctx.save_for_backward(dh, w_grad)
        ctx.master = master
        ctx.mark_non_differentiable(n_valid)
        total = ce + z_coef * z if z_coef else ce.clone()
        ce_out, z_out = ce.detach().clone(), z.detach().clone()
        ctx.mark_non_differentiable(ce_out, z_out)
        return total, n_valid, ce_out, z_out

    @staticmethod
    def backward(ctx, dloss, _dn, _dce, _dz):
        dh, w_grad = ctx.saved_tensors
        if w_grad is not None:
            m = ctx.master
            if m.grad is None:
                m.grad = torch.zeros_like(m, dtype=torch.float32)
            m.grad.addcmul_(w_grad, dloss.to(torch.float32))
        return ((dh * dloss.to(dh.dtype)) if dh is not None else None,) + (None,) * 10


def _head_pair(weight: torch.Tensor):
    """(tensor the kernels read, fp32 master that receives the gradient or None) for a head weight that may be a
    trainable fp32 master with a bf16 shadow."""
    sh = getattr(weight, "shadow", None)
    if weight.requires_grad and sh is not None and native_enabled(sh):
        return sh, weight
    return weight, None


def linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100,
                         chunk: int = 4096, weight_t: Optional[torch.Tensor] = None, softcap: float = 0.0,
                         label_smoothing: float = 0.0, logit_scale: float = 1.0):
    """Returns (Σ loss over valid tokens, number of valid tokens). A frozen head, or a trainable fp32 head with a bf16
    shadow (full-parameter training), runs the chunked kernels; anything else the reference path. ``softcap`` c replaces
    the logits by c tanh(x / c); ``label_smoothing`` e mixes the one-hot target with e / V; ``logit_scale`` multiplies the
    logits before either."""
    w, master = _head_pair(weight)
    if use_native(hidden) and (master is not None or not weight.requires_grad):
        return _LinearCeFn.apply(hidden, w, weight_t if master is None else None, labels, ignore_index, chunk, 0.0, master,
                                 float(label_smoothing), float(softcap), float(logit_scale))[:2]
    return ref.linear_cross_entropy(hidden, weight, labels, ignore_index, chunk, softcap, label_smoothing, logit_scale)


def linear_cross_entropy_z(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, z_coef: float,
                           ignore_index: int = -100, chunk: int = 4096):
    """Cross entropy with the z regulariser of pre-training: returns (mean over valid tokens of ce + z_coef·lse²,
    mean ce, mean lse²); the last two are for logging only."""
    w, master = _head_pair(weight)
    if use_native(hidden) and (master is not None or not weight.requires_grad):
        total, n, ce, z = _LinearCeFn.apply(hidden, w, None, labels, ignore_index, chunk, float(z_coef), master)
        d = n.clamp(min=1).to(total.dtype)
        return total / d, ce / d, z / d
    V = weight.shape[0]
    valid = labels != ignore_index
    ce_sum = hidden.new_zeros((), dtype=torch.float32)
    z_sum = hidden.new_zeros((), dtype=torch.float32)
    for a in range(0, hidden.shape[0], chunk):
        lg = (hidden[a:a + chunk] @ weight.t().to(hidden.dtype)).float()
        m = valid[a:a + chunk]
        lse = torch.logsumexp(lg, -1)
        tgt = labels[a:a + chunk].clamp(0, V - 1)
        ce_sum = ce_sum + ((lse - lg.gather(-1, tgt[:, None]).squeeze(-1)) * m).sum()
        z_sum = z_sum + ((lse ** 2) * m).sum()
    d = valid.sum().clamp(min=1).to(torch.float32)
    return (ce_sum + z_coef * z_sum) / d, (ce_sum / d).detach(), (z_sum / d).detach()


def causal_lm_loss(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100,
                   weight_t: Optional[torch.Tensor] = None, softcap: float = 0.0, label_smoothing: float = 0.0) -> torch.Tensor:
    """Mean over non-ignored tokens; ``labels`` must already be shifted/aligned with ``hidden``."""
    s, n = linear_cross_entropy(hidden, weight, labels, ignore_index, weight_t=weight_t, softcap=softcap,
                                label_smoothing=label_smoothing)
    return s / n.clamp(min=1).to(s.dtype)


# --------------------------------------------------------------------------- grouped expert MLP
GROUP_ALIGN = 128      # row alignment of every expert's slab in the padded sorted layout (one GEMM tile)


def padded_expert_layout(idx: torch.Tensor, num_experts: int, align: int = GROUP_ALIGN):
    """Where each (token, slot) assignment goes when rows are sorted by expert with every expert's slab padded to a
    multiple of ``align`` rows. Returns (dest [T*k] int64: row of assignment i in the padded buffer, off int32 [E+1],
    rows_cap: static capacity of the buffer). Everything stays on the device; ``rows_cap`` depends on shapes only."""
    flat = idx.reshape(-1)
    n = flat.numel()
    counts = torch.bincount(flat, minlength=num_experts)
    padded = (counts + (align - 1)) // align * align
    off = torch.zeros(num_experts + 1, dtype=torch.int64, device=idx.device)
    off[1:] = torch.cumsum(padded, 0)
    start = torch.zeros(num_experts + 1, dtype=torch.int64, device=idx.device)
    start[1:] = torch.cumsum(counts, 0)
    order = torch.argsort(flat, stable=True)
    rank = torch.empty_like(order)
    rank[order] = torch.arange(n, device=idx.device) - start[flat[order]]
    dest = off[flat] + rank
    rows_cap = -(-(n + num_experts * (align - 1)) // align) * align
    return dest, off.to(torch.int32), rows_cap


class _GroupedLinearFn(torch.autograd.Function):
    """y[r] = x[r] W_e(r)^T over rows grouped by expert in the padded layout; tcgen05 grouped GEMMs forward and backward."""

    @staticmethod
    def forward(ctx, x, w, off):
        nat = _native()
        E, N, K = w.shape
        ctx.save_for_backward(x, w, off)
        return nat.grouped_gemm(0, x, w, off, N, K)

    @staticmethod
    def backward(ctx, dy):
        x, w, off = ctx.saved_tensors
        nat = _native()
        E, N, K = w.shape
        dy = dy.contiguous()
        dx = nat.grouped_gemm(1, dy, w, off, N, K) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            dw = nat.grouped_gemm(2, dy, x, off, N, K).to(w.dtype)
        return dx, dw, None


def grouped_linear(x: torch.Tensor, w: torch.Tensor, off: torch.Tensor) -> torch.Tensor:
    """x [R, K] rows grouped by expert (padded layout, ``off`` int32 [E+1]); w [E, N, K]. Returns [R, N]."""
    if use_native(x) and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and w.shape[2] % 8 == 0:
        return _GroupedLinearFn.apply(x, w.contiguous() if not w.is_contiguous() else w, off)
    out = torch.zeros(x.shape[0], w.shape[1], dtype=x.dtype, device=x.device)
    o = off.tolist()
    for e in range(w.shape[0]):
        if o[e + 1] > o[e]:
            out[o[e]:o[e + 1]] = F.linear(x[o[e]:o[e + 1]], w[e])
    return out


def grouped_mlp(xs: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, offsets: torch.Tensor) -> torch.Tensor:
    """Rows of ``xs`` are grouped by expert (``offsets`` [E+1], unpadded); returns down_e(swiglu(gate_up_e(x))) per row.
    Plain per-expert loop: the oracle of the grouped kernels and the CPU path."""
    out = torch.empty(xs.shape[0], down.shape[1], dtype=xs.dtype, device=xs.device)
    off = offsets.tolist()
    for e in range(gate_up.shape[0]):
        s, t = off[e], off[e + 1]
        if t > s:
            out[s:t] = F.linear(ref.swiglu(F.linear(xs[s:t], gate_up[e])), down[e])
    return out


def moe_experts(x: torch.Tensor, w: torch.Tensor, idx: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    """Mixture-of-experts feed-forward for routed tokens: x [T, H], routing weights w [T, k] and expert ids idx [T, k].
    On the native path tokens are scattered into the padded expert-sorted layout and both projections (and their
    gradients) run as grouped tcgen05 GEMMs with no host synchronisation; elsewhere a per-expert loop."""
    T, k = idx.shape
    E = gate_up.shape[0]
    if use_native(x) and gate_up.dtype == torch.bfloat16:
        dest, off, cap = padded_expert_layout(idx, E)
        tok = torch.arange(T, device=x.device).repeat_interleave(k)
        xs = torch.zeros(cap, x.shape[1], dtype=x.dtype, device=x.device).index_copy(0, dest, x[tok])
        act = swiglu(grouped_linear(xs, gate_up, off))
        ys = grouped_linear(act, down, off)[dest]
        ys = ys * w.reshape(-1).to(ys.dtype)[:, None]
        return torch.zeros_like(x).index_add(0, tok, ys)
    flat = idx.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=E)
    offsets = torch.zeros(E + 1, dtype=torch.int64, device=idx.device)
    offsets[1:] = torch.cumsum(counts, 0)
    tok = order // k
    ys = grouped_mlp(x[tok], gate_up, down, offsets)
    ys = ys * w.reshape(-1)[order].to(ys.dtype)[:, None]
    out = torch.zeros_like(x)
    out.index_add_(0, tok, ys)
    return out


# --------------------------------------------------------------------------- per-token log-probabilities
class _TokenLogpFn(torch.autograd.Function):
    """log p(token_t | hidden_t) for a frozen output head; the backward recomputes each logits chunk."""

    @staticmethod
    def forward(ctx, hidden, weight, weight_t, tokens, chunk):
        nll, _ = _native().token_nll(hidden, weight, tokens, chunk)
        ctx.save_for_backward(hidden, weight, weight_t, tokens)
        ctx.chunk = chunk
        return -nll

    @staticmethod
    def backward(ctx, dlogp):
        hidden, weight, weight_t, tokens = ctx.saved_tensors
        # d/dh of (-nll) with upstream dlogp  ==  d/dh of nll scaled by -dlogp
        _, dh = _native().token_nll(hidden, weight, tokens, ctx.chunk, (-dlogp).float().contiguous(), weight_t)
        return dh, None, None, None, None


def token_logprobs(hidden: torch.Tensor, weight: torch.Tensor, tokens: torch.Tensor, chunk: int = 4096,
                   weight_t: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Selective log-softmax: log-probability of ``tokens`` [T] under the head applied to ``hidden`` [T, H].
    (reference: crates/pmetal-trainer/src/logprob_utils.rs)"""
    if use_native(hidden) and not weight.requires_grad:
        return _TokenLogpFn.apply(hidden, weight, weight_t, tokens, chunk)
    out = []
    for s in range(0, hidden.shape[0], chunk):
        lg = F.linear(hidden[s:s + chunk], weight).float()
        t = tokens[s:s + chunk]
        lp = torch.log_softmax(lg, -1).gather(-1, t.clamp(min=0)[:, None])[:, 0]
        out.append(torch.where(t >= 0, lp, torch.zeros_like(lp)))
    return torch.cat(out)
