"""Manifold-constrained hyper-connections (crates/pmetal-mhc/src/{layer,mappings,sinkhorn,params}.rs and its eight Metal
kernels: compute_mappings, apply_constraints, apply_pre/post_res_mapping, sinkhorn_backward, compute_amax_gain,
expand/collapse_streams).

The residual stream is widened to ``n`` parallel streams. Each layer reads a mixture of streams (``pre`` mapping),
writes its output back with ``post`` weights, and mixes the streams with a residual matrix that is projected onto
doubly-stochastic matrices by Sinkhorn-Knopp normalisation so that the mixing preserves the mean signal (its rows and
columns sum to one).

Two forms:
* ``MhcLayer`` — static mappings (one set of logits per layer, optionally shifted by a small projection of the mean stream).
* ``MhcDynamicLayer`` — the per-token form of the paper: ``H~ = alpha_g (RMSNorm(flatten(x)) phi) + b`` gives, for every
  token, ``H_pre = sigmoid``, ``H_post = 2 sigmoid`` and ``H_res = Sinkhorn`` of its three parts. On a GPU the projection
  runs on the tcgen05 GEMM and everything else on the kernels of ``csrc/mhc.cu`` (one pass over the streams per
  application, forward and backward); elsewhere the same arithmetic runs in PyTorch, which is also the test oracle."""
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
    if _native_ok(x) and x.dim() == 2:
        from ..ops import native as nat
        return nat.mhc_expand(x.contiguous(), n)
    return x.unsqueeze(-2).expand(*x.shape[:-1], n, x.shape[-1]).contiguous()


def collapse_streams(xs: torch.Tensor) -> torch.Tensor:
    if _native_ok(xs) and xs.dim() == 3 and not xs.requires_grad:
        from ..ops import native as nat
        return nat.mhc_collapse(xs.contiguous())
    return xs.mean(-2)


def _native_ok(x: torch.Tensor) -> bool:
    from ..ops import functional as ops
    return x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and ops.use_native(x)


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


# ------------------------------------------------------------------------------------------- per-token mappings
def mappings_reference(x: torch.Tensor, phi: torch.Tensor, bias: torch.Tensor, alpha: torch.Tensor, iters: int,
                       eps: float = 1e-6):
    """x [T, n, C] -> (H_pre [T, n], H_post [T, n], H_res [T, n, n]) in fp32."""
    T, n, C = x.shape
    flat = x.reshape(T, n * C).float()
    xn = flat * torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + eps)
    raw = xn @ phi.float()
    gate = torch.cat([alpha[0].expand(n), alpha[1].expand(n), alpha[2].expand(n * n)]).float()
    ht = raw * gate + bias.float()
    return (torch.sigmoid(ht[:, :n]), 2 * torch.sigmoid(ht[:, n:2 * n]),
            sinkhorn_knopp(ht[:, 2 * n:].reshape(T, n, n), iters))


class _MappingsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, phi, bias, alpha, iters):
        from ..ops import native as nat
        T, n, C = x.shape
        out = n * n + 2 * n
        flat = x.reshape(T, n * C)
        phi_t = phi.detach().t().contiguous().to(torch.bfloat16)              # [out, nC]: K-major operand
        raw = nat.gemm_f32(flat, phi_t)                                       # [T, >= out] fp32 on the tensor cores
        ht, ri, pre, post, res = nat.mhc_mappings(x, raw, bias.detach().float(), alpha.detach().float(), iters)
        ctx.save_for_backward(x, phi, alpha, ht, ri, raw)
        ctx.iters = iters
        ctx.mark_non_differentiable(ht)
        return pre, post, res, ht

    @staticmethod
    def backward(ctx, d_pre, d_post, d_res, _):
        from ..ops import native as nat
        x, phi, alpha, ht, ri, raw = ctx.saved_tensors
        T, n, C = x.shape
        out = n * n + 2 * n
        z = lambda t, shape: t.contiguous().float() if t is not None else torch.zeros(shape, device=x.device)   # noqa: E731
        d_ht = nat.mhc_constraints_bwd(ht, z(d_pre, (T, n)), z(d_post, (T, n)), z(d_res, (T, n, n)), n, ctx.iters)
        gate = torch.cat([alpha[0].expand(n), alpha[1].expand(n), alpha[2].expand(n * n)]).float()
        rawn = raw[:, :out] * ri[:, None]                                     # (RMSNorm(x) . phi)
        d_bias = d_ht.sum(0)
        g = d_ht * rawn
        d_alpha = torch.stack([g[:, :n].sum(), g[:, n:2 * n].sum(), g[:, 2 * n:].sum()])
        d_rawn = d_ht * gate                                                  # [T, out]
        flat = x.reshape(T, n * C)
        xn = flat.float() * ri[:, None]
        d_phi = xn.t() @ d_rawn                                               # [nC, out]
        d_xn = d_rawn @ phi.float().t()                                       # [T, nC]
        d_flat = ri[:, None] * (d_xn - xn * (d_xn * xn).mean(-1, keepdim=True))
        return d_flat.reshape(T, n, C).to(x.dtype), d_phi.to(phi.dtype), d_bias.to(phi.dtype), d_alpha.to(alpha.dtype), None


class _PreFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, h_pre):
        from ..ops import native as nat
        ctx.save_for_backward(x, h_pre)
        return nat.mhc_pre(x, h_pre)

    @staticmethod
    def backward(ctx, dh_in):
        from ..ops import native as nat
        x, h_pre = ctx.saved_tensors
        dx, _, d_pre, _, _ = nat.mhc_mix_bwd(x, None, dh_in.contiguous(), None, h_pre, None, None)
        return dx, d_pre


class _PostResFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, h_out, h_res, h_post):
        from ..ops import native as nat
        ctx.save_for_backward(x, h_out, h_res, h_post)
        return nat.mhc_post_res(x, h_out, h_res, h_post)

    @staticmethod
    def backward(ctx, dx_out):
        from ..ops import native as nat
        x, h_out, h_res, h_post = ctx.saved_tensors
        dx, dh_out, _, d_post, d_res = nat.mhc_mix_bwd(x, h_out, None, dx_out.contiguous(), None, h_post, h_res)
        return dx, dh_out, d_res, d_post


def apply_pre(x: torch.Tensor, h_pre: torch.Tensor) -> torch.Tensor:
    """h_in[t] = sum_n H_pre[t, n] x[t, n]."""
    if _native_ok(x) and x.shape[1] in (2, 4, 8):
        return _PreFn.apply(x.contiguous(), h_pre.contiguous().float())
    return torch.einsum("tn,tnc->tc", h_pre.to(x.dtype), x)


def apply_post_res(x: torch.Tensor, h_out: torch.Tensor, h_res: torch.Tensor, h_post: torch.Tensor) -> torch.Tensor:
    """x_out[t, m] = sum_n H_res[t, m, n] x[t, n] + H_post[t, m] h_out[t]."""
    if _native_ok(x) and x.shape[1] in (2, 4, 8):
        return _PostResFn.apply(x.contiguous(), h_out.contiguous(), h_res.contiguous().float(), h_post.contiguous().float())
    return torch.einsum("tmn,tnc->tmc", h_res.to(x.dtype), x) + h_post.to(x.dtype)[:, :, None] * h_out[:, None, :]


def compute_mappings(x: torch.Tensor, phi: torch.Tensor, bias: torch.Tensor, alpha: torch.Tensor, iters: int = 20):
    if _native_ok(x) and x.shape[1] in (2, 4, 8) and iters <= 32:
        pre, post, res, _ = _MappingsFn.apply(x.contiguous(), phi, bias, alpha, iters)
        return pre, post, res
    return mappings_reference(x, phi, bias, alpha, iters)


def amax_gain(h_res: torch.Tensor):
    """(largest absolute row sum, largest absolute column sum) of the mixing matrices: 1.0 for doubly stochastic ones;
    a drift away from it is the stability signal the reference monitors."""
    if h_res.is_cuda:
        from ..ops import functional as ops
        if ops.native_enabled(h_res):
            from ..ops import native as nat
            g = nat.mhc_amax_gain(h_res.contiguous().float())
            return g[0], g[1]
    a = h_res.abs()
    return a.sum(-1).max(), a.sum(-2).max()


class MhcDynamicLayer(nn.Module):
    """Per-token mappings. ``phi`` starts at zero and the biases at (pre: uniform read, post: gain 1, res: near identity),
    so a fresh layer behaves like a plain residual connection on the mean stream."""

    def __init__(self, n_streams: int, hidden: int, sinkhorn_iters: int = 20):
        super().__init__()
        n = n_streams
        self.n, self.hidden, self.iters = n, hidden, sinkhorn_iters
        self.phi = nn.Parameter(torch.zeros(n * hidden, n * n + 2 * n))
        b = torch.zeros(n * n + 2 * n)
        b[:n] = -torch.log(torch.tensor(float(n - 1))) if n > 1 else 0.0      # sigmoid = 1 / n
        b[2 * n:] = (torch.eye(n) * 4.0).reshape(-1)
        self.bias = nn.Parameter(b)
        self.alpha = nn.Parameter(torch.full((3,), 0.01))

    def forward(self, xs: torch.Tensor, fn) -> torch.Tensor:
        pre, post, res = compute_mappings(xs, self.phi, self.bias, self.alpha, self.iters)
        h_out = fn(apply_pre(xs, pre))
        return apply_post_res(xs, h_out, res, post)
