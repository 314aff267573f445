"""Context parallelism: causal ring attention over sequence chunks.

Rank r holds tokens [r*T, (r+1)*T) of one long sequence (``split_sequence``). Attention of the local queries over the
whole prefix is the online-softmax merge of ``world`` partial attentions, one per key/value chunk:
the local chunk with a causal mask, every earlier chunk without a mask, later chunks skipped. That fixes the two
defects of the reference's implementation — no causal mask across blocks and PassQ merging outputs of different
queries (crates/pmetal-distributed/src/context_parallel/ring_attention.rs:32-227, sequence_split.rs:28-95).

Two transports:
* ``ring_attention_fused`` — K/V chunks live in symmetric memory and the attention kernel's TMA loads read the remote
  chunk in place over NVLink (no staging copy, no separate send/recv): transfer overlaps the MMAs tile by tile. Every
  rank signals with a collective barrier before and after so chunks are complete and stay alive while peers read them.
* ``ring_attention_p2p`` — the reference's PassKV ring over NCCL send/recv, double-buffered; on CPU/gloo it runs the
  same schedule with PyTorch attention and is what the multi-process CPU tests exercise."""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def split_sequence(x: torch.Tensor, rank: int, world: int, dim: int = 0) -> torch.Tensor:
    """Contiguous chunk of ``x`` along ``dim`` (length must divide evenly)."""
    n = x.shape[dim]
    if n % world:
        raise ValueError(f"sequence length {n} is not divisible by {world}")
    return x.narrow(dim, rank * (n // world), n // world)


def gather_sequence(x: torch.Tensor, group=None, dim: int = 0) -> torch.Tensor:
    world = dist.get_world_size(group)
    parts = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=dim)


def merge_partials(outs: List[torch.Tensor], lses: List[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """outs [T, hq, d], lses [hq, T] (natural log; -inf for empty). Returns the merged (out fp32, lse)."""
    lse = torch.stack(lses)                                   # [n, hq, T]
    m = lse.max(0).values
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w = torch.exp(lse - m_safe)                               # [n, hq, T]
    tot = w.sum(0)
    out = sum(o.float() * (wi / tot.clamp(min=1e-30)).transpose(0, 1)[..., None] for o, wi in zip(outs, w))
    return out, m_safe + torch.log(tot.clamp(min=1e-30))


def _block_attention(q, k, v, scale: float, causal: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """One (query chunk, key chunk) partial. CUDA: the tcgen05 kernel; otherwise PyTorch."""
    from ..ops import functional as ops
    T, hq, d = q.shape
    Tk, hkv = k.shape[0], k.shape[1]
    if ops.use_native(q) and d == 128:
        from ..ops import native
        ss = torch.zeros(T, dtype=torch.int32, device=q.device)
        return native.attn_fwd_rect(q.contiguous(), k, v, ss, scale, 0 if causal else Tk)
    rep = hq // hkv
    kk = k.float().repeat_interleave(rep, 1).permute(1, 0, 2)
    vv = v.float().repeat_interleave(rep, 1).permute(1, 0, 2)
    s = torch.einsum("thd,hsd->hts", q.float(), kk) * scale
    if causal:
        s = s.masked_fill(torch.ones(T, Tk, dtype=torch.bool, device=q.device).triu(1), float("-inf"))
    lse = torch.logsumexp(s, -1)
    out = torch.einsum("hts,hsd->thd", torch.softmax(s, -1), vv)
    return out.to(q.dtype), lse


def ring_attention_p2p(q, k, v, scale: Optional[float] = None, group=None):
    """PassKV ring over send/recv. q [T, hq, d], k/v [T, hkv, d] local chunks. Returns (out [T, hq, d], lse [hq, T])."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    outs, lses = [], []
    cur_k, cur_v = k.contiguous(), v.contiguous()
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    for s in range(world):
        src = (rank - s) % world
        reqs = []
        if s + 1 < world:                      # start moving the next block while this one is computed
            nk, nv = torch.empty_like(cur_k), torch.empty_like(cur_v)
            ops_ = [dist.P2POp(dist.isend, cur_k, nxt, group), dist.P2POp(dist.isend, cur_v, nxt, group),
                    dist.P2POp(dist.irecv, nk, prv, group), dist.P2POp(dist.irecv, nv, prv, group)]
            reqs = dist.batch_isend_irecv(ops_)
        if src <= rank:                        # chunks after ours are entirely in the future
            o, l = _block_attention(q, cur_k, cur_v, scale, causal=(src == rank))
            outs.append(o)
            lses.append(l)
        for r in reqs:
            r.wait()
        if s + 1 < world:
            cur_k, cur_v = nk, nv
    out, lse = merge_partials(outs, lses)
    return out.to(q.dtype), lse


class FusedRingAttention:
    """K/V chunks in symmetric memory; remote chunks are read in place by the attention kernel."""

    def __init__(self, tokens_per_rank: int, hkv: int, d: int = 128, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.shape = (tokens_per_rank, hkv, d)
        n = tokens_per_rank * hkv * d
        self.kbuf = symm_mem.empty(n, dtype=torch.bfloat16, device=dev)
        self.vbuf = symm_mem.empty(n, dtype=torch.bfloat16, device=dev)
        g = group if group is not None else dist.group.WORLD
        self.hk = symm_mem.rendezvous(self.kbuf, g)
        self.hv = symm_mem.rendezvous(self.vbuf, g)

    def _peer(self, handle, r: int) -> torch.Tensor:
        return handle.get_buffer(r, self.shape, torch.bfloat16)

    @torch.no_grad()
    def forward(self, q, k, v, scale: Optional[float] = None):
        scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
        self.kbuf.view(self.shape).copy_(k)
        self.vbuf.view(self.shape).copy_(v)
        self.hk.barrier()                        # every rank's chunk is in place
        outs, lses = [], []
        for s in range(self.rank + 1):           # own chunk first (no NVLink traffic), then walk back in time
            src = self.rank - s
            kk = self._peer(self.hk, src)
            vv = self._peer(self.hv, src)
            o, l = _block_attention(q, kk, vv, scale, causal=(src == self.rank))
            outs.append(o)
            lses.append(l)
        out, lse = merge_partials(outs, lses)
        torch.cuda.current_stream().synchronize()
        self.hk.barrier()                        # nobody overwrites a chunk that a peer is still reading
        return out.to(q.dtype), lse


# ------------------------------------------------------------------------------------------- training: zig-zag + backward
def zigzag_chunks(rank: int, world: int) -> Tuple[int, int]:
    """The two chunk indices (of 2 * world equal chunks) that ``rank`` holds: one from the front of the sequence and its
    mirror image from the back, so that every rank does the same amount of causal work (the plain contiguous split gives
    rank r only r + 1 of ``world`` key blocks)."""
    return rank, 2 * world - 1 - rank


def zigzag_split(x: torch.Tensor, rank: int, world: int, dim: int = 0) -> torch.Tensor:
    n = x.shape[dim]
    if n % (2 * world):
        raise ValueError(f"sequence length {n} is not divisible by {2 * world}")
    c = n // (2 * world)
    a, b = zigzag_chunks(rank, world)
    return torch.cat([x.narrow(dim, a * c, c), x.narrow(dim, b * c, c)], dim=dim)


def zigzag_gather(x: torch.Tensor, group=None, dim: int = 0) -> torch.Tensor:
    """Inverse of ``zigzag_split`` over the group: the full sequence in its natural order, on every rank."""
    world = dist.get_world_size(group)
    parts = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(parts, x.contiguous(), group=group)
    c = x.shape[dim] // 2
    chunks = [None] * (2 * world)
    for r, p in enumerate(parts):
        a, b = zigzag_chunks(r, world)
        chunks[a], chunks[b] = p.narrow(dim, 0, c), p.narrow(dim, c, c)
    return torch.cat(chunks, dim=dim)


def _pair_backward_native(do, q, o, lse, k, v, scale: float, causal: bool):
    """Gradients of one (query chunk, key chunk) pair from the saved *global* log-sum-exp: with it every pair's share of
    the softmax is exact, so the pairs are additive. The diagonal pair is the square causal kernel as is. An earlier
    (fully visible) key chunk is run through the same kernel as the front half of a virtual sequence of twice the length:
    keys [K ; 0], values [V ; 0], queries [0 ; Q] with zero output gradient in the front half. Zero keys contribute nothing
    to dQ, zero output gradients nothing to dK / dV, and the back-half keys' own gradients are dropped."""
    from ..ops import native
    T, hq, d = q.shape
    hkv = k.shape[1]
    if causal:
        ss = torch.zeros(T, dtype=torch.int32, device=q.device)
        return native.attn_bwd(do, q, k, v, o, lse, ss, scale)
    z = lambda t: torch.zeros_like(t)      # noqa: E731
    q2, do2, o2 = torch.cat([z(q), q]), torch.cat([z(do), do]), torch.cat([z(o), o])
    k2, v2 = torch.cat([k, z(k)]), torch.cat([v, z(v)])
    lse2 = torch.cat([torch.zeros_like(lse), lse], dim=1).contiguous()
    ss = torch.zeros(2 * T, dtype=torch.int32, device=q.device)
    dq2, dk2, dv2 = native.attn_bwd(do2, q2, k2, v2, o2, lse2, ss, scale)
    return dq2[T:], dk2[:T], dv2[:T]


class _ZigzagAttentionFn(torch.autograd.Function):
    """Causal attention over a sequence that is split zig-zag over the group. Keys and values are gathered once into
    local memory (one all-gather each; every rank needs nearly all of them: its back chunk looks at everything before
    it), every (local query chunk, visible key chunk) pair runs on the attention kernels, partial outputs are merged by
    their log-sum-exp; the backward pass forms dQ locally and sends the key / value gradients home with one
    reduce-scatter each."""

    @staticmethod
    def forward(ctx, q, k, v, scale, group):
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        c = q.shape[0] // 2
        kf, vf = zigzag_gather(k, group), zigzag_gather(v, group)        # natural order, [2 W c, hkv, d]
        outs, lses = [], []
        for half, ci in enumerate(zigzag_chunks(rank, world)):
            qc = q[half * c:(half + 1) * c].contiguous()
            po, pl = [], []
            for cj in range(ci + 1):
                o_, l_ = _block_attention(qc, kf[cj * c:(cj + 1) * c], vf[cj * c:(cj + 1) * c], scale, causal=(cj == ci))
                po.append(o_)
                pl.append(l_)
            o_, l_ = merge_partials(po, pl)
            outs.append(o_.to(q.dtype))
            lses.append(l_)
        out = torch.cat(outs)
        lse = torch.cat(lses, dim=1).contiguous()
        ctx.save_for_backward(q, kf, vf, out, lse)
        ctx.cfg = (scale, group, rank, world, c)
        return out

    @staticmethod
    def backward(ctx, do):
        q, kf, vf, out, lse = ctx.saved_tensors
        scale, group, rank, world, c = ctx.cfg
        from ..ops import functional as ops
        native_ok = ops.use_native(q) and q.shape[-1] == 128
        do = do.contiguous()
        dq = torch.zeros_like(q, dtype=torch.float32)
        dkf = torch.zeros_like(kf, dtype=torch.float32)
        dvf = torch.zeros_like(vf, dtype=torch.float32)
        for half, ci in enumerate(zigzag_chunks(rank, world)):
            sl = slice(half * c, (half + 1) * c)
            qc, oc, doc, lc = q[sl].contiguous(), out[sl].contiguous(), do[sl].contiguous(), lse[:, sl].contiguous()
            for cj in range(ci + 1):
                ks = slice(cj * c, (cj + 1) * c)
                kc, vc = kf[ks].contiguous(), vf[ks].contiguous()
                if native_ok:
                    g_q, g_k, g_v = _pair_backward_native(doc, qc, oc, lc, kc, vc, scale, cj == ci)
                else:
                    g_q, g_k, g_v = _pair_backward_reference(doc, qc, oc, lc, kc, vc, scale, cj == ci)
                dq[sl] += g_q.float()
                dkf[ks] += g_k.float()
                dvf[ks] += g_v.float()
        # gradients of the gathered keys / values go back to their owners: sum over ranks, keep the own two chunks
        dist.all_reduce(dkf, group=group)
        dist.all_reduce(dvf, group=group)
        dk = zigzag_split(dkf, rank, world).to(q.dtype)
        dv = zigzag_split(dvf, rank, world).to(q.dtype)
        return dq.to(q.dtype), dk, dv, None, None


def _pair_backward_reference(do, q, o, lse, k, v, scale: float, causal: bool):
    """The same pair gradients in PyTorch (fp32): P = exp(S - lse), dS = P (dP - delta)."""
    T, hq, d = q.shape
    Tk, hkv = k.shape[0], k.shape[1]
    rep = hq // hkv
    qf, kf_, vf_ = q.float(), k.float().repeat_interleave(rep, 1), v.float().repeat_interleave(rep, 1)
    s = torch.einsum("thd,shd->hts", qf, kf_) * scale
    if causal:
        s = s.masked_fill(torch.ones(T, Tk, dtype=torch.bool, device=q.device).triu(1), float("-inf"))
    p = torch.exp(s - lse[:, :, None])
    dof = do.float()
    dv_r = torch.einsum("hts,thd->shd", p, dof)
    dp = torch.einsum("thd,shd->hts", dof, vf_)
    delta = (dof * o.float()).sum(-1).transpose(0, 1)                    # [hq, T]
    ds = p * (dp - delta[:, :, None]) * scale
    dq = torch.einsum("hts,shd->thd", ds, kf_)
    dk_r = torch.einsum("hts,thd->shd", ds, qf)
    dk = dk_r.reshape(Tk, hkv, rep, d).sum(2)
    dv = dv_r.reshape(Tk, hkv, rep, d).sum(2)
    return dq, dk, dv


def zigzag_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None, group=None):
    """Differentiable causal attention for context-parallel training. q [2c, hq, d], k / v [2c, hkv, d]: this rank's
    zig-zag share (``zigzag_split``) of one long sequence. Returns the attention output for the local queries."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    return _ZigzagAttentionFn.apply(q, k, v, scale, group)
