"""Manifold-constrained hyper-connections (crates/pmetal-mhc/src/{layer,mappings,sinkhorn,params}.rs and its eight Metal
kernels: compute_mappings, apply_constraints, apply_pre/post_res_mapping, sinkhorn_backward, expand/collapse_streams).

The residual stream is widened to ``n`` parallel streams. Each layer reads a mixture of streams (``pre`` mapping, a
softmax over streams), writes its output back with ``post`` weights, and mixes the streams with a residual matrix that
is projected onto doubly-stochastic matrices by Sinkhorn-Knopp normalisation so that the mixing preserves the mean
signal (its rows and columns sum to one). All maps are tiny (n <= 8), so this is plain differentiable PyTorch."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


def sinkhorn_knopp(logits: torch.Tensor, iters: int = 20, eps: float = 1e-8) -> torch.Tensor:
    """exp(logits) alternately row- and column-normalised -> approximately doubly stochastic [..., n, n]."""
    m = torch.exp(logits - logits.amax(dim=(-1, -2), keepdim=True))
    for _ in range(iters):
        m = m / (m.sum(-1, keepdim=True) + eps)
        m = m / (m.sum(-2, keepdim=True) + eps)
    return m


def expand_streams(x: torch.Tensor, n: int) -> torch.Tensor:
    """[T, H] -> [T, n, H] (every stream starts as a copy)."""
    return x.unsqueeze(-2).expand(*x.shape[:-1], n, x.shape[-1]).contiguous()


def collapse_streams(xs: torch.Tensor) -> torch.Tensor:
    return xs.mean(-2)


class MhcLayer(nn.Module):
    def __init__(self, n_streams: int = 4, sinkhorn_iters: int = 20, dynamic: bool = False, hidden: int = 0):
        super().__init__()
        self.n, self.iters = n_streams, sinkhorn_iters
        self.pre_logits = nn.Parameter(torch.zeros(n_streams))
        self.post_logits = nn.Parameter(torch.zeros(n_streams))
        self.res_logits = nn.Parameter(torch.eye(n_streams) * 4.0)        # starts near the identity mixing
        self.dynamic = nn.Linear(hidden, 2 * n_streams, bias=False) if dynamic and hidden else None
        if self.dynamic is not None:
            nn.init.zeros_(self.dynamic.weight)

    def mappings(self, xs: torch.Tensor):
        pre, post = self.pre_logits, self.post_logits
        if self.dynamic is not None:
            d = self.dynamic(F.rms_norm(xs.mean(-2), (xs.shape[-1],)))
            pre, post = pre + d[..., : self.n], post + d[..., self.n:]
        return F.softmax(pre, -1), torch.sigmoid(post) * 2, sinkhorn_knopp(self.res_logits, self.iters)

    def forward(self, xs: torch.Tensor, fn) -> torch.Tensor:
        """xs [T, n, H]; ``fn`` maps [T, H] -> [T, H] (the wrapped attention or MLP block without its residual)."""
        pre, post, res = self.mappings(xs)
        if pre.dim() == 1:
            inp = torch.einsum("n,tnh->th", pre, xs)
            mixed = torch.einsum("mn,tnh->tmh", res, xs)
            return mixed + post[None, :, None] * fn(inp)[:, None, :]
        inp = torch.einsum("tn,tnh->th", pre, xs)
        mixed = torch.einsum("mn,tnh->tmh", res, xs)
        return mixed + post[:, :, None] * fn(inp)[:, None, :]
