"""Model-merge methods on tensors.

Every function takes the same-named tensor from each model (and the base model's where a method works on
task vectors ``tau_i = theta_i - theta_base``) and returns the merged tensor in fp32. Method set and
parameters follow crates/pmetal-merge/src/methods/*.rs: linear, slerp, multislerp, task_arithmetic, ties
(magnitude sparsify + weighted sign consensus), dare_linear / dare_ties (random drop with 1/density rescale),
della / della_linear (magnitude-ranked drop probabilities), breadcrumbs (drop the top and bottom
magnitude tails), model_stock, nearswap, passthrough, ram, souper, fisher, regmean. All math is elementwise
or reduction-only and runs on whichever device holds the tensors (CUDA for large checkpoints).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch


@dataclass
class MergeParameters:
    weight: float = 1.0
    density: float = 1.0
    lambda_: float = 1.0
    t: float = 0.5
    rescale: bool = True
    epsilon: float = 0.1          # della: spread of drop probabilities around (1 - density)
    seed: Optional[int] = 42
    extra: Dict[str, float] = field(default_factory=dict)


def sparsify_by_magnitude(t: torch.Tensor, density: float) -> torch.Tensor:
    """Keep the largest-|x| fraction ``density`` (threshold = k-th smallest magnitude, ties kept)."""
    if density >= 1.0:
        return t
    if density <= 0.0:
        return torch.zeros_like(t)
    flat = t.reshape(-1).abs()
    n = flat.numel()
    k = min(int(math.ceil((1.0 - density) * n)), n - 1)
    thr = torch.kthvalue(flat.float(), k + 1).values
    return t * (t.abs() >= thr)


def sign_consensus(tensors: Sequence[torch.Tensor], weights: Sequence[float]) -> torch.Tensor:
    """Sum of weight_m * tensor_m over the models whose sign agrees with the weighted majority sign."""
    if len(tensors) == 1:
        return tensors[0] * weights[0]
    votes = sum(torch.sign(t) * w for t, w in zip(tensors, weights))
    maj = torch.sign(votes)
    out = torch.zeros_like(tensors[0])
    for t, w in zip(tensors, weights):
        out += (t * w) * ((torch.sign(t) * maj) > 0)
    return out


def _weighted_sum(ts, ws):
    out = torch.zeros_like(ts[0])
    for t, w in zip(ts, ws):
        out += t * w
    return out


def _f(ts):
    return [t.float() for t in ts]


def linear(tensors, weights, normalize: bool = True) -> torch.Tensor:
    ts = _f(tensors)
    s = sum(weights)
    ws = [w / s for w in weights] if (normalize and abs(s) > 1e-12) else list(weights)
    return _weighted_sum(ts, ws)


def slerp(a: torch.Tensor, b: torch.Tensor, t: float, eps: float = 1e-8) -> torch.Tensor:
    a, b = a.float(), b.float()
    na, nb = a.norm(), b.norm()
    if na < eps or nb < eps:
        return (1 - t) * a + t * b
    cos = torch.clamp((a * b).sum() / (na * nb), -1.0, 1.0)
    omega = torch.acos(cos)
    so = torch.sin(omega)
    if so.abs() < 1e-6:
        return (1 - t) * a + t * b
    return (torch.sin((1 - t) * omega) / so) * a + (torch.sin(t * omega) / so) * b


def multislerp(tensors, weights, base: Optional[torch.Tensor] = None, eps: float = 1e-8) -> torch.Tensor:
    """Spherical weighted mean: normalise, average, re-normalise, restore the weighted mean norm."""
    ts = _f(tensors)
    if base is not None:
        ts = [t - base.float() for t in ts]
    s = sum(weights)
    ws = [w / s for w in weights]
    norms = [t.norm() for t in ts]
    unit = [t / n.clamp(min=eps) for t, n in zip(ts, norms)]
    mean = _weighted_sum(unit, ws)
    out = mean / mean.norm().clamp(min=eps) * sum(n * w for n, w in zip(norms, ws))
    return out + base.float() if base is not None else out


def task_arithmetic(tensors, base, weights, lam: float = 1.0) -> torch.Tensor:
    b = base.float()
    return b + lam * _weighted_sum([t.float() - b for t in tensors], weights)


def ties(tensors, base, weights, densities, lam: float = 1.0) -> torch.Tensor:
    b = base.float()
    tvs = [sparsify_by_magnitude(t.float() - b, d) for t, d in zip(tensors, densities)]
    return b + lam * sign_consensus(tvs, weights)


def _dare_mask(shape, density: float, gen, device) -> torch.Tensor:
    if density >= 1.0:
        return torch.ones(shape, device=device)
    return (torch.rand(shape, generator=gen, device=device) < density).float()


def dare(tensors, base, weights, densities, lam: float = 1.0, rescale: bool = True, consensus: bool = False,
         seed: Optional[int] = 42) -> torch.Tensor:
    b = base.float()
    gen = torch.Generator(device=b.device)
    if seed is not None:
        gen.manual_seed(seed)
    tvs = []
    for t, d in zip(tensors, densities):
        tv = (t.float() - b) * _dare_mask(b.shape, d, gen, b.device)
        if rescale and 0.0 < d < 1.0:
            tv = tv / d
        tvs.append(tv)
    merged = sign_consensus(tvs, weights) if consensus else _weighted_sum(tvs, weights)
    return b + lam * merged


def della(tensors, base, weights, densities, lam: float = 1.0, epsilon: float = 0.1, consensus: bool = True,
          seed: Optional[int] = 42) -> torch.Tensor:
    """Magnitude-aware stochastic pruning: within each row, elements ranked by |tau| get keep-probabilities
    spread linearly over [density - eps, density + eps] (largest magnitude -> highest), kept values rescaled by 1/p."""
    b = base.float()
    gen = torch.Generator(device=b.device)
    if seed is not None:
        gen.manual_seed(seed)
    tvs = []
    for t, d in zip(tensors, densities):
        tv = t.float() - b
        if d >= 1.0:
            tvs.append(tv)
            continue
        rows = tv.reshape(-1, tv.shape[-1]) if tv.dim() > 1 else tv.reshape(1, -1)
        n = rows.shape[1]
        rank = rows.abs().argsort(dim=1).argsort(dim=1).float()               # 0 = smallest magnitude
        eps = min(epsilon, d, 1.0 - d)
        p = (d - eps) + (2 * eps) * (rank / max(n - 1, 1))
        keep = torch.rand(rows.shape, generator=gen, device=b.device) < p
        tvs.append((rows * keep / p.clamp(min=1e-6)).reshape(tv.shape))
    merged = sign_consensus(tvs, weights) if consensus else _weighted_sum(tvs, weights)
    return b + lam * merged


def breadcrumbs(tensors, base, weights, lam: float = 1.0, top_p: float = 0.99, bottom_p: float = 0.10,
                consensus: bool = False) -> torch.Tensor:
    """Drop the ``bottom_p`` smallest-magnitude and the (1 - top_p) largest-magnitude entries of each task vector."""
    b = base.float()
    tvs = []
    for t in tensors:
        tv = t.float() - b
        a = tv.abs().reshape(-1)
        n = a.numel()
        lo = torch.kthvalue(a, max(int(bottom_p * n), 1)).values if bottom_p > 0 else a.new_tensor(-1.0)
        hi = torch.kthvalue(a, min(max(int(math.ceil(top_p * n)), 1), n)).values if top_p < 1 else a.new_tensor(float("inf"))
        tvs.append(tv * ((tv.abs() > lo) & (tv.abs() <= hi)))
    merged = sign_consensus(tvs, weights) if consensus else _weighted_sum(tvs, weights)
    return b + lam * merged


def model_stock(tensors, base) -> torch.Tensor:
    """Interpolate between the fine-tuned average and the base with t = N cos / (1 + (N-1) cos), cos = mean pairwise
    cosine of the task vectors."""
    b = base.float()
    if not tensors:
        return b
    tvs = [t.float() - b for t in tensors]
    n = len(tvs)
    if n == 1:
        return b + tvs[0]
    cs = []
    for i in range(n):
        for j in range(i + 1, n):
            d = tvs[i].norm() * tvs[j].norm()
            cs.append(((tvs[i] * tvs[j]).sum() / d.clamp(min=1e-12)).clamp(-1, 1))
    cos = torch.stack(cs).mean()
    t = (n * cos / (1 + (n - 1) * cos)).clamp(0.0, 1.0)
    return b + t * (sum(tvs) / n)


def nearswap(tensors, base, lam: float = 1.0) -> torch.Tensor:
    """Per element take the model value closest to the base."""
    b = base.float()
    if len(tensors) == 1:
        return b + lam * (tensors[0].float() - b)
    st = torch.stack(_f(tensors))
    idx = (st - b).abs().argmin(dim=0, keepdim=True)
    sel = st.gather(0, idx)[0]
    return b + lam * (sel - b)


def passthrough(tensors) -> torch.Tensor:
    return tensors[0].float()


def ram(tensors, base, weights) -> torch.Tensor:
    """Magnitude-renormalised task arithmetic: the merged task vector is rescaled to the weighted mean norm."""
    b = base.float()
    tvs = [t.float() - b for t in tensors]
    merged = _weighted_sum(tvs, weights)
    target = sum(tv.norm() * w for tv, w in zip(tvs, weights)) / max(sum(weights), 1e-12)
    return b + merged * (target / merged.norm().clamp(min=1e-12))


def souper(tensors, weights=None) -> torch.Tensor:
    """Uniform (or weighted) model soup."""
    return linear(tensors, weights or [1.0] * len(tensors), True)


def fisher(tensors, fishers, eps: float = 1e-8) -> torch.Tensor:
    """Fisher-weighted average: sum_i F_i theta_i / sum_i F_i (diagonal Fisher estimates per model)."""
    num = sum(f.float() * t.float() for f, t in zip(fishers, tensors))
    return num / (sum(f.float() for f in fishers) + eps)


def regmean(tensors, grams, alpha: float = 0.9) -> torch.Tensor:
    """RegMean for linear weights [out, in]: W = (sum_i W_i G_i)(sum_i G_i)^-1 with off-diagonals of the
    Gram matrices G_i = X_i^T X_i shrunk by ``alpha``."""
    gs = []
    for g in grams:
        g = g.double()
        d = torch.diag(torch.diag(g))
        gs.append(alpha * g + (1 - alpha) * d)
    num = sum(t.double() @ g for t, g in zip(tensors, gs))
    return (num @ torch.linalg.pinv(sum(gs))).float()


METHODS = ("linear", "slerp", "multislerp", "task_arithmetic", "ties", "dare_ties", "dare_linear", "della",
           "della_linear", "breadcrumbs", "model_stock", "nearswap", "passthrough", "ram", "souper", "fisher", "regmean")
REQUIRES_BASE = {"task_arithmetic", "ties", "dare_ties", "dare_linear", "della", "della_linear", "breadcrumbs",
                 "model_stock", "nearswap", "ram"}


def merge_tensor(method: str, tensors: List[torch.Tensor], base: Optional[torch.Tensor], params: List[MergeParameters],
                 g: MergeParameters, aux: Optional[dict] = None) -> torch.Tensor:
    if method in REQUIRES_BASE and base is None:
        raise ValueError(f"merge method {method} needs a base model")
    ws = [p.weight for p in params]
    ds = [p.density for p in params]
    if method == "linear":
        return linear(tensors, ws)
    if method == "slerp":
        if len(tensors) != 2:
            raise ValueError("slerp merges exactly two models")
        return slerp(tensors[0], tensors[1], g.t)
    if method == "multislerp":
        return multislerp(tensors, ws, base)
    if method == "task_arithmetic":
        return task_arithmetic(tensors, base, ws, g.lambda_)
    if method == "ties":
        return ties(tensors, base, ws, ds, g.lambda_)
    if method in ("dare_ties", "dare_linear"):
        return dare(tensors, base, ws, ds, g.lambda_, g.rescale, method == "dare_ties", g.seed)
    if method in ("della", "della_linear"):
        return della(tensors, base, ws, ds, g.lambda_, g.epsilon, method == "della", g.seed)
    if method == "breadcrumbs":
        return breadcrumbs(tensors, base, ws, g.lambda_)
    if method == "model_stock":
        return model_stock(tensors, base)
    if method == "nearswap":
        return nearswap(tensors, base, g.lambda_)
    if method == "passthrough":
        return passthrough(tensors)
    if method == "ram":
        return ram(tensors, base, ws)
    if method == "souper":
        return souper(tensors, ws)
    if method == "fisher":
        return fisher(tensors, (aux or {})["fishers"])
    if method == "regmean":
        return regmean(tensors, (aux or {})["grams"])
    raise ValueError(f"unknown merge method {method!r}")
