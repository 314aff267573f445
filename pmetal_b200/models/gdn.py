"""Gated delta-net linear attention (Qwen3-Next / Qwen3.5 hybrid layers): recurrent step and chunk-parallel form.

State per head S [d_k, d_v]; per token with decay g_t in (0, 1], write strength beta_t:
    S <- g_t * S;   S <- S + k_t^T (beta_t (v_t - k_t S));   y_t = q_t S
(crates/pmetal-bridge/cpp/bridge_native.cpp:6-139 — gdn_metal_step / gdn_metal_state_update,
crates/pmetal-mlx/src/kernels/gated_delta.rs — chunked WY form + recurrent step). ``gdn_recurrent`` is the token-by-token
definition (decode and the oracle); ``gdn_chunked`` processes chunks of C tokens with matrix products: inside a chunk the
delta-rule corrections form a unit lower-triangular system that is solved once, the inter-chunk state is carried exactly."""
from __future__ import annotations

import torch


def gdn_step(S: torch.Tensor, q, k, v, g, beta):
    """One token. S [H, dk, dv]; q, k [H, dk]; v [H, dv]; g, beta [H]. Returns (y [H, dv], S')."""
    S = S * g[:, None, None]
    pred = torch.einsum("hk,hkv->hv", k, S)
    S = S + torch.einsum("hk,hv->hkv", k, beta[:, None] * (v - pred))
    return torch.einsum("hk,hkv->hv", q, S), S


def gdn_recurrent(q, k, v, g, beta, S0=None):
    """q, k [T, H, dk]; v [T, H, dv]; g, beta [T, H]. Returns (y [T, H, dv], S_T)."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, dk, dv, dtype=torch.float32, device=q.device) if S0 is None else S0.float().clone()
    ys = []
    for t in range(T):
        y, S = gdn_step(S, q[t].float(), k[t].float(), v[t].float(), g[t].float(), beta[t].float())
        ys.append(y)
    return torch.stack(ys), S


def gdn_chunked(q, k, v, g, beta, S0=None, chunk: int = 64):
    """Chunk-parallel evaluation, numerically equal to ``gdn_recurrent`` (fp32)."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, dk, dv, dtype=torch.float32, device=q.device) if S0 is None else S0.float().clone()
    out = torch.empty(T, H, dv, dtype=torch.float32, device=q.device)
    for a in range(0, T, chunk):
        b = min(T, a + chunk)
        C = b - a
        qc, kc, vc = (x[a:b].float().transpose(0, 1) for x in (q, k, v))          # [H, C, d]
        gc, bc = g[a:b].float().t(), beta[a:b].float().t()                          # [H, C]
        logg = torch.log(gc.clamp(min=1e-30))
        cum = torch.cumsum(logg, -1)                                                # log prod_{s<=t} g_s
        # decay from token s (exclusive) to token t (inclusive): exp(cum_t - cum_s) for s <= t
        # [H, C(t), C(s)]; entries above the diagonal are never used and would overflow for strong decay, so they are
        # forced to exp(-inf) = 0 before the exponential
        causal = torch.ones(C, C, device=q.device, dtype=torch.bool).tril(0)
        dec = torch.exp((cum[:, :, None] - cum[:, None, :]).masked_fill(~causal, float("-inf")))
        tri = torch.ones(C, C, device=q.device).tril(-1)
        # u_t = beta_t (v_t - k_t S_{t-1} g-decayed), with S_{t-1} = dec * S_in + sum_{s<t} dec(t-1.. ) k_s^T u_s
        # k_t (state before write t, after decay t) = exp(cum_t) k_t S_in + sum_{s<t} exp(cum_t - cum_s) (k_t . k_s) u_s
        kk = torch.einsum("htd,hsd->hts", kc, kc) * dec * tri                       # strictly lower
        A = torch.eye(C, device=q.device)[None] + bc[:, :, None] * kk               # (I + diag(beta) L) u = rhs
        rhs = bc[:, :, None] * (vc - torch.exp(cum)[:, :, None] * torch.einsum("htk,hkv->htv", kc, S))
        u = torch.linalg.solve_triangular(A, rhs, upper=False)                      # [H, C, dv]
        qk = torch.einsum("htd,hsd->hts", qc, kc) * dec * torch.ones(C, C, device=q.device).tril(0)
        y = torch.exp(cum)[:, :, None] * torch.einsum("htk,hkv->htv", qc, S) + torch.einsum("hts,hsv->htv", qk, u)
        out[a:b] = y.transpose(0, 1)
        tail = torch.exp(cum[:, -1:] - cum)                                         # decay from s to the chunk end
        S = torch.exp(cum[:, -1])[:, None, None] * S + torch.einsum("hsk,hsv->hkv", kc * tail[:, :, None], u)
    return out, S
