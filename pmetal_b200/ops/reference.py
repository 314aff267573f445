"""Plain-PyTorch statements of every fused operator.

These are the numerical oracle for the CUDA kernels (tests compare each kernel to
the function of the same name evaluated in fp32) and the execution path on CPU.
The math restates the reference's Metal shaders: RMSNorm
(crates/pmetal-metal/src/kernels/metal/fused_norm_lora.metal), half-split RoPE with
explicit positions (fused_rope.metal), SwiGLU (fused_swiglu.metal), fused LoRA
(fused_lora.metal:128-497), varlen attention (flash_attention.metal:1093-1130),
chunked linear+cross-entropy (fused_cross_entropy.metal:64-881) and AdamW
(crates/pmetal-bridge/src/optimizer.rs:215-337).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * weight.float()).to(x.dtype)


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float, scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables [T, head_dim/2] for integer positions (fp32)."""
    half = head_dim // 2
    inv = theta ** (-torch.arange(0, half, dtype=torch.float32, device=positions.device) / half)
    ang = positions.float()[:, None] * (inv[None, :] / scale)
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-split ("non-traditional") rotary embedding on [T, H, D]."""
    half = x.shape[-1] // 2
    xf = x.float()
    x1, x2 = xf[..., :half], xf[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


def qk_norm_rope(q: torch.Tensor, k: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                 positions: torch.Tensor, theta: float, eps: float = 1e-6, rope_scale: float = 1.0):
    """Per-head RMSNorm on q and k (Qwen3) followed by RoPE. q:[T,Hq,D] k:[T,Hkv,D]."""
    if q_weight is not None:
        q = rms_norm(q, q_weight, eps)
        k = rms_norm(k, k_weight, eps)
    cos, sin = rope_cos_sin(positions, q.shape[-1], theta, rope_scale)
    return apply_rope(q, cos, sin), apply_rope(k, cos, sin)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """[T, 2I] with gate in the first half, up in the second → silu(gate) * up."""
    g, u = gate_up.chunk(2, dim=-1)
    return (F.silu(g.float()) * u.float()).to(gate_up.dtype)


def lora_linear(x: torch.Tensor, weight: torch.Tensor, lora_a: Optional[torch.Tensor], lora_b: Optional[torch.Tensor],
                scale: float, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x Wᵀ + scale · (x Aᵀ) Bᵀ  (crates/pmetal-lora/src/lora.rs:429-465)."""
    y = F.linear(x, weight, bias)
    if lora_a is not None:
        t = F.linear(x, lora_a.to(x.dtype))
        y = y + scale * F.linear(t, lora_b.to(x.dtype))
    return y


def seq_starts_from_cu(cu_seqlens: torch.Tensor, total: int) -> torch.Tensor:
    """For every token the index of the first token of its document. int32 [total]."""
    cu = cu_seqlens.to(torch.int64)
    idx = torch.arange(total, device=cu.device)
    doc = torch.searchsorted(cu[1:].contiguous(), idx, right=True)
    return cu[doc].to(torch.int32)


def varlen_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor, scale: float,
                     causal: bool = True, window: int = 0, softcap: float = 0.0) -> torch.Tensor:
    """Block-diagonal (per-document) causal attention with GQA. q:[T,Hq,D], k,v:[T,Hkv,D] → [T,Hq,D]."""
    T, hq, d = q.shape
    hkv = k.shape[1]
    rep = hq // hkv
    out = torch.empty_like(q)
    cu = cu_seqlens.tolist()
    for s, e in zip(cu[:-1], cu[1:]):
        if e <= s:
            continue
        qq = q[s:e].transpose(0, 1).float()                      # [Hq, L, D]
        kk = k[s:e].transpose(0, 1).float().repeat_interleave(rep, 0)
        vv = v[s:e].transpose(0, 1).float().repeat_interleave(rep, 0)
        sc = torch.matmul(qq, kk.transpose(1, 2)) * scale
        if softcap > 0:
            sc = softcap * torch.tanh(sc / softcap)
        L = e - s
        i = torch.arange(L, device=q.device)
        mask = torch.ones(L, L, dtype=torch.bool, device=q.device)
        if causal:
            mask &= i[None, :] <= i[:, None]
        if window > 0:
            mask &= i[None, :] > i[:, None] - window
        sc = sc.masked_fill(~mask, float("-inf"))
        out[s:e] = torch.matmul(sc.softmax(-1), vv).transpose(0, 1).to(q.dtype)
    return out


def linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100,
                         chunk: int = 4096, softcap: float = 0.0,
                         label_smoothing: float = 0.0, logit_scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Σ over valid tokens of (logsumexp(h Wᵀ) − (h Wᵀ)[label]) and the valid-token count; with ``label_smoothing`` e
    the target is (1 − e) one-hot + e / V.

    ``labels`` are already aligned with ``hidden`` (the caller did the causal shift).
    Token-chunked so the [T, V] logits never exist at once.
    """
    total = hidden.new_zeros((), dtype=torch.float32)
    valid = labels != ignore_index
    for s in range(0, hidden.shape[0], chunk):
        h = hidden[s:s + chunk]
        lab = labels[s:s + chunk]
        logits = F.linear(h, weight.to(h.dtype)).float()
        if logit_scale != 1.0:
            logits = logits * logit_scale
        if softcap > 0:
            logits = softcap * torch.tanh(logits / softcap)
        total = total + F.cross_entropy(logits, lab, ignore_index=ignore_index, reduction="sum",
                                        label_smoothing=label_smoothing)
    return total, valid.sum()


def adamw_step(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, step: int, lr: float,
               beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8, weight_decay: float = 0.01) -> None:
    """Bias-corrected Adam step, then decoupled decay on the *updated* parameter
    (optimizer.rs:295-336): p ← p − lr·m̂/(√v̂+eps);  p ← p − wd·lr·p."""
    g = g.float()
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    mh = m / (1 - beta1 ** step) if step > 0 else m          # step <= 0: no bias correction
    vh = v / (1 - beta2 ** step) if step > 0 else v
    p.sub_(lr * mh / (vh.sqrt() + eps))
    if weight_decay != 0.0:
        p.sub_(weight_decay * lr * p)


def global_grad_norm(grads) -> torch.Tensor:
    return torch.sqrt(sum((g.float() ** 2).sum() for g in grads))
