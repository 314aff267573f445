"""Distillation losses.

Token-level losses take student and teacher logits ``[..., V]`` and a temperature; all return a scalar mean over
tokens (optionally masked) multiplied by T^2 as usual for soft targets. Set follows crates/pmetal-distill/src/losses/*.rs:
forward / reverse KL, Jensen-Shannon, skewed JSD, soft cross-entropy, total variation, hinge and logistic ranking on the
teacher's top-k, MSE on logits, GKD (generalised JSD with beta), MiniLLM (reverse KL with teacher-mixed sampling weight),
universal-logit (cross-vocabulary: compare sorted probability profiles), hidden-state MSE / cosine / L1, and
attention transfer. On CUDA the KL-family goes through the fused chunked kernel (``fused_kd_loss``)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F


def _masked_mean(per_tok: torch.Tensor, mask: Optional[torch.Tensor]) -> torch.Tensor:
    if mask is None:
        return per_tok.mean()
    m = mask.to(per_tok.dtype)
    return (per_tok * m).sum() / m.sum().clamp(min=1)


def _lsm(x, T):
    return F.log_softmax(x.float() / T, dim=-1)


def kl_divergence(student, teacher, T: float = 2.0, mask=None, reverse: bool = False):
    ls, lt = _lsm(student, T), _lsm(teacher, T)
    per = (ls.exp() * (ls - lt)).sum(-1) if reverse else (lt.exp() * (lt - ls)).sum(-1)
    return _masked_mean(per, mask) * T * T


def jensen_shannon(student, teacher, T: float = 2.0, mask=None, beta: float = 0.5):
    """Generalised JSD: beta KL(p_t || m) + (1 - beta) KL(p_s || m), m = beta p_t + (1 - beta) p_s."""
    ls, lt = _lsm(student, T), _lsm(teacher, T)
    ps, pt = ls.exp(), lt.exp()
    lm = torch.log((beta * pt + (1 - beta) * ps).clamp(min=1e-30))
    per = beta * (pt * (lt - lm)).sum(-1) + (1 - beta) * (ps * (ls - lm)).sum(-1)
    return _masked_mean(per, mask) * T * T


def skewed_jsd(student, teacher, T: float = 2.0, mask=None, alpha: float = 0.1):
    """Skew divergence pair: KL(p_t || a p_t + (1-a) p_s) and its mirror, averaged."""
    ls, lt = _lsm(student, T), _lsm(teacher, T)
    ps, pt = ls.exp(), lt.exp()
    m1 = torch.log((alpha * pt + (1 - alpha) * ps).clamp(min=1e-30))
    m2 = torch.log((alpha * ps + (1 - alpha) * pt).clamp(min=1e-30))
    per = 0.5 * (pt * (lt - m1)).sum(-1) + 0.5 * (ps * (ls - m2)).sum(-1)
    return _masked_mean(per, mask) * T * T


def soft_cross_entropy(student, teacher, T: float = 2.0, mask=None):
    per = -(_lsm(teacher, T).exp() * _lsm(student, T)).sum(-1)
    return _masked_mean(per, mask) * T * T


def total_variation(student, teacher, T: float = 1.0, mask=None):
    per = 0.5 * (_lsm(teacher, T).exp() - _lsm(student, T).exp()).abs().sum(-1)
    return _masked_mean(per, mask)


def logit_mse(student, teacher, mask=None):
    return _masked_mean(((student.float() - teacher.float()) ** 2).mean(-1), mask)


def _topk_pairs(student, teacher, T, k):
    pt = _lsm(teacher, T).exp()
    k = min(k, pt.shape[-1])
    tv, ti = pt.topk(k, dim=-1)
    return tv, ti


def hinge_ranking(student, teacher, T: float = 1.0, mask=None, top_k: int = 32):
    """For teacher-ordered pairs (i before j) of the teacher's top-k: relu((p_t[i]-p_t[j]) - (p_s[i]-p_s[j]))."""
    tv, ti = _topk_pairs(student, teacher, T, top_k)
    sv = _lsm(student, T).exp().gather(-1, ti)
    tm = tv.unsqueeze(-1) - tv.unsqueeze(-2)
    sm = sv.unsqueeze(-1) - sv.unsqueeze(-2)
    valid = (tm > 0).to(tm.dtype)
    per = (F.relu(tm - sm) * valid).sum((-1, -2)) / valid.sum((-1, -2)).clamp(min=1)
    return _masked_mean(per, mask)


def logistic_ranking(student, teacher, T: float = 1.0, mask=None, top_k: int = 32):
    """softplus(-(s[i] - s[j])) over pairs the teacher ranks i above j (student scores are scaled logits)."""
    tv, ti = _topk_pairs(student, teacher, T, top_k)
    sv = (student.float() / T).gather(-1, ti)
    tm = tv.unsqueeze(-1) - tv.unsqueeze(-2)
    sm = sv.unsqueeze(-1) - sv.unsqueeze(-2)
    valid = (tm > 0).to(tm.dtype)
    per = (F.softplus(-sm) * valid).sum((-1, -2)) / valid.sum((-1, -2)).clamp(min=1)
    return _masked_mean(per, mask)


def gkd(student, teacher, T: float = 1.0, mask=None, beta: float = 0.5):
    """GKD: beta = 0 forward KL, beta = 1 reverse KL, in between the generalised JSD."""
    if beta <= 0:
        return kl_divergence(student, teacher, T, mask)
    if beta >= 1:
        return kl_divergence(student, teacher, T, mask, reverse=True)
    return jensen_shannon(student, teacher, T, mask, beta=1 - beta)


def minillm(student, teacher, T: float = 1.0, mask=None, teacher_mix: float = 0.2):
    """Reverse KL against a teacher-mixed student (stabilised MiniLLM objective)."""
    ls, lt = _lsm(student, T), _lsm(teacher, T)
    mix = torch.log((teacher_mix * lt.exp() + (1 - teacher_mix) * ls.exp()).clamp(min=1e-30)).detach()
    per = (mix.exp() * (ls - lt)).sum(-1)
    return _masked_mean(per, mask) * T * T


def universal_logit(student, teacher, T: float = 1.0, mask=None, top_k: Optional[int] = None):
    """Cross-vocabulary distillation: compare the sorted (descending) probability profiles, zero-padded to a common
    length, with an L1 distance."""
    ps = _lsm(student, T).exp().sort(-1, descending=True).values
    pt = _lsm(teacher, T).exp().sort(-1, descending=True).values
    if top_k:
        ps, pt = ps[..., :top_k], pt[..., :top_k]
    n = max(ps.shape[-1], pt.shape[-1])
    ps = F.pad(ps, (0, n - ps.shape[-1]))
    pt = F.pad(pt, (0, n - pt.shape[-1]))
    return _masked_mean((ps - pt).abs().sum(-1), mask)


def hidden_state_loss(student_h, teacher_h, kind: str = "mse", proj: Optional[torch.Tensor] = None, mask=None):
    """``proj`` [H_t, H_s] maps student hidden states to the teacher width when they differ."""
    s = student_h.float()
    if proj is not None:
        s = s @ proj.float().t()
    t = teacher_h.float()
    if kind == "mse":
        per = ((s - t) ** 2).mean(-1)
    elif kind == "l1":
        per = (s - t).abs().mean(-1)
    elif kind == "cosine":
        per = 1 - F.cosine_similarity(s, t, dim=-1)
    else:
        raise ValueError(kind)
    return _masked_mean(per, mask)


def attention_transfer(student_attn, teacher_attn):
    """MSE between head-averaged attention maps [B, H, T, T] (head counts may differ)."""
    return ((student_attn.float().mean(1) - teacher_attn.float().mean(1)) ** 2).mean()


def reasoning_mask(tokens: torch.Tensor, start_token: int, end_token: int) -> torch.Tensor:
    """1.0 for tokens strictly inside a ``start_token … end_token`` span (the markers themselves count as outside the
    span start and as its last position respectively: inclusive running counts of both markers are subtracted and
    clamped, crates/pmetal-distill/src/reasoning.rs:235-256)."""
    inside = (tokens == start_token).cumsum(-1) - (tokens == end_token).cumsum(-1)
    return inside.clamp(0, 1).float()


def rationale_kl(student, teacher, T: float = 2.0, mask=None, reasoning_weight: float = 1.0,
                 token_weights: Optional[torch.Tensor] = None):
    """Entropy-weighted forward KL (rationale-based distillation, crates/pmetal-distill/src/reasoning.rs:178-226): token i
    gets weight ``1 + reasoning_weight * H_i / max_j H_j`` with H the teacher's entropy at temperature T, times optional
    external weights (a reasoning-span mask, or a per-sample correctness signal for outcome supervision); the loss is
    the weighted mean of the per-token KL. No T^2 factor, as in the reference."""
    ls, lt = _lsm(student, T), _lsm(teacher, T)
    pt = lt.exp()
    kl = (pt * (lt - ls)).sum(-1)
    ent = -(pt * lt).sum(-1)
    w = 1.0 + reasoning_weight * ent / ent.max().clamp(min=1e-6)
    if token_weights is not None:
        w = w * token_weights.to(w.dtype)
    if mask is not None:
        w = w * mask.to(w.dtype)
    return (kl * w).sum() / w.sum().clamp(min=1e-6)


LOSSES = {"kl": kl_divergence, "forward_kl": kl_divergence, "rationale": rationale_kl,
          "reverse_kl": lambda s, t, T=2.0, mask=None: kl_divergence(s, t, T, mask, reverse=True),
          "js": jensen_shannon, "jsd": jensen_shannon, "skewed_jsd": skewed_jsd, "soft_ce": soft_cross_entropy,
          "tvd": total_variation, "hinge_ranking": hinge_ranking, "logistic_ranking": logistic_ranking, "gkd": gkd,
          "minillm": minillm, "universal_logit": universal_logit,
          "mse": lambda s, t, T=1.0, mask=None: logit_mse(s, t, mask)}


# ------------------------------------------------------------------------------------------- fused chunked KD
class _FusedKdFn(torch.autograd.Function):
    """loss = mean over unmasked tokens of D(softmax(h_t W_t^T / T), softmax(h_s W_s^T / T)) * T^2, computed chunk by
    chunk: logits of a chunk exist only transiently and the kernel turns the student logits into their gradient in
    place, which is multiplied straight back through the student head."""

    @staticmethod
    def forward(ctx, h_s, w_s, h_t, w_t, mask, T, kind, beta, chunk):
        from ..ops import native
        n = h_s.shape[0]
        m = mask.float() if mask is not None else torch.ones(n, device=h_s.device)
        denom = m.sum().clamp(min=1)
        scale = (m / denom * (T * T)).contiguous()
        loss = torch.zeros((), device=h_s.device)
        dh = torch.empty_like(h_s)
        need_dw = w_s.requires_grad
        dw = torch.zeros_like(w_s, dtype=torch.float32) if need_dw else None
        for a in range(0, n, chunk):
            b = min(n, a + chunk)
            ls = (h_s[a:b] @ w_s.t()).contiguous()
            lt = (h_t[a:b] @ w_t.t()).contiguous()
            rl = native.kd_fwd_bwd(ls, lt, T, kind, beta, row_scale=scale[a:b])
            loss = loss + (rl * scale[a:b]).sum()
            dh[a:b] = ls @ w_s
            if need_dw:
                dw += (ls.t() @ h_s[a:b]).float()
        ctx.save_for_backward(dh, dw)
        return loss

    @staticmethod
    def backward(ctx, g):
        dh, dw = ctx.saved_tensors
        return (dh * g.to(dh.dtype), None if dw is None else (dw * g).to(dh.dtype), None, None, None, None, None, None,
                None)


def fused_kd_loss(h_student, w_student, h_teacher, w_teacher, mask=None, T: float = 2.0, kind: str = "kl",
                  beta: float = 0.5, chunk: int = 2048):
    """Hidden states [n, H] (bf16) and output heads [V, H]; falls back to the dense formula off-GPU."""
    from ..ops import functional as ops
    if ops.use_native(h_student) and h_student.dtype == torch.bfloat16:
        return _FusedKdFn.apply(h_student, w_student, h_teacher.detach(), w_teacher.detach(), mask, T, kind, beta, chunk)
    s = h_student.float() @ w_student.float().t()
    t = h_teacher.float() @ w_teacher.float().t()
    fn = {"kl": kl_divergence, "forward_kl": kl_divergence, "soft_ce": soft_cross_entropy, "tvd": total_variation}.get(kind)
    if kind == "reverse_kl":
        return kl_divergence(s, t, T, mask, reverse=True)
    if kind in ("js", "jsd"):
        return jensen_shannon(s, t, T, mask, beta)
    if kind == "tvd":
        return total_variation(s, t, T, mask) * T * T
    return fn(s, t, T, mask)
