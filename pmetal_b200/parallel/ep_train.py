"""Expert parallelism for training: every rank keeps a contiguous slice of each layer's experts, tokens travel to the
rank that owns their expert and come back, and autograd follows them both ways.

Forward of one mixture-of-experts layer on rank r with local tokens x [T, H] and routing (weights w, expert ids idx):
the T * k assignments are ordered by destination rank and exchanged with one all-to-all (rows) plus one for the local
expert ids; the owner runs its experts on what it received (``ops.moe_experts`` with one expert per row: grouped tcgen05
GEMMs with their input- and weight-gradient kernels on a GPU, a per-expert loop elsewhere); a second all-to-all returns
the rows, which are weighted and summed into the tokens. The backward of an all-to-all is the opposite all-to-all, so
expert weights receive the gradient of every token routed to them, from all ranks, and need no further reduction across
the expert-parallel group; router and non-expert parameters are replicated and are averaged like any data-parallel
parameter. The fused dispatch / combine engine of ``parallel/ep.py`` stays the inference path.
Reference: crates/pmetal-distributed/src/expert_parallel/dispatch.rs:66-214 (dispatch / combine), used for training
through the MLX autograd there."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from .ep import expert_range


class _AllToAllRows(torch.autograd.Function):
    """Rows of ``x`` split as ``send`` go out, rows split as ``recv`` come in; backward swaps the two lists."""

    @staticmethod
    def forward(ctx, x, send: List[int], recv: List[int], group):
        ctx.send, ctx.recv, ctx.group = send, recv, group
        out = x.new_empty((sum(recv),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), recv, send, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        back = g.new_empty((sum(ctx.send),) + tuple(g.shape[1:]))
        dist.all_to_all_single(back, g.contiguous(), ctx.send, ctx.recv, group=ctx.group)
        return back, None, None, None


def exchange_counts(send: torch.Tensor, group) -> List[int]:
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv.tolist()


def ep_moe_train_forward(block, x: torch.Tensor, w: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """Differentiable expert-parallel forward of a ``SparseMoeBlock`` prepared by :func:`shard_experts_for_training`."""
    from ..ops import functional as ops
    group = block.ep_group
    world = dist.get_world_size(group)
    T, k = idx.shape
    E = block.cfg.num_experts
    bounds = torch.tensor([expert_range(E, r, world)[0] for r in range(world)] + [E], device=idx.device)
    flat = idx.reshape(-1)
    dest = torch.bucketize(flat, bounds[1:], right=True)                 # owner rank of every assignment
    order = torch.argsort(dest, stable=True)
    send = torch.bincount(dest, minlength=world)
    send_l = send.tolist()
    recv_l = exchange_counts(send, group)
    tok = torch.div(order, k, rounding_mode="floor")
    rows = _AllToAllRows.apply(x[tok], send_l, recv_l, group)
    local_ids = (flat[order] - bounds[dest[order]]).to(torch.int64)      # expert index inside the owner's slice
    got_ids = local_ids.new_empty(sum(recv_l))
    dist.all_to_all_single(got_ids, local_ids.contiguous(), recv_l, send_l, group=group)
    ones = rows.new_ones(rows.shape[0], 1)
    ys = ops.moe_experts(rows, ones, got_ids[:, None], block.gate_up, block.down) if rows.shape[0] else rows
    back = _AllToAllRows.apply(ys, recv_l, send_l, group)
    back = back * w.reshape(-1)[order].to(back.dtype)[:, None]
    return torch.zeros_like(x).index_add(0, tok, back)


@torch.no_grad()
def shard_experts_for_training(model, group=None) -> int:
    """Cut the expert stacks of every mixture-of-experts layer to this rank's slice (parameters shrink in place) and mark
    the layers for :func:`ep_moe_train_forward`. Returns the number of layers changed."""
    from ..models.moe import SparseMoeBlock
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    n = 0
    for m in model.modules():
        if isinstance(m, SparseMoeBlock):
            a, b = expert_range(m.cfg.num_experts, rank, world)
            for name in ("gate_up", "down"):
                p = getattr(m, name)
                setattr(m, name, torch.nn.Parameter(p.data[a:b].clone(), requires_grad=p.requires_grad))
            m.local_experts = (a, b)
            m.ep_group = group if group is not None else (dist.group.WORLD if world > 1 else None)
            m.ep_train = world > 1
            n += 1
    return n


def expert_parameters(model) -> List[torch.nn.Parameter]:
    """Parameters that are sharded over the expert-parallel group (no gradient averaging across it)."""
    from ..models.moe import SparseMoeBlock
    out: List[torch.nn.Parameter] = []
    for m in model.modules():
        if isinstance(m, SparseMoeBlock) and getattr(m, "ep_train", False):
            out += [m.gate_up, m.down]
    return out


@torch.no_grad()
def average_replicated_gradients(model, group=None) -> None:
    """Mean over the group of the gradients of everything that is replicated (attention, norms, routers, embeddings);
    the expert slices already hold complete gradients, which are divided by the group size to match the mean loss."""
    world = dist.get_world_size(group)
    skip = {id(p) for p in expert_parameters(model)}
    for p in model.parameters():
        if p.grad is None:
            continue
        if id(p) in skip:
            p.grad.div_(world)
        else:
            dist.all_reduce(p.grad, group=group)
            p.grad.div_(world)
