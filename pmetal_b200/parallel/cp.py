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
