"""Expert parallelism: placement helpers, capacity policy, and the fused dispatch/GEMM/combine engine.

``FusedExpertMoE`` runs a mixture-of-experts feed-forward with the kernels of csrc/moe_quant.cu (routing, sort,
gather, weighted combine) and csrc/moe_gemm.cu (grouped tcgen05 GEMMs whose loads pull token rows from the source
rank and whose epilogue pushes results back to it). With one rank it is the local grouped GEMM path.

Library pieces mirror the reference: ``expert_range`` / ``ExpertPlacement`` (crates/pmetal-distributed/src/
expert_parallel/placement.rs, expert_shard.rs:54-110), capacity factor with drop / redistribute and the Switch
auxiliary loss (capacity.rs:20-190), and the dispatcher semantics of dispatch.rs:66-214 (replicated routing, tokens sent
to the rank that owns the expert, results returned and combined with the routing weights)."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


# ------------------------------------------------------------------------------------------- placement / capacity
def expert_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous [start, end) of experts owned by ``rank``; the remainder goes to the first ranks."""
    base, rem = divmod(total, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


@dataclass
class ExpertPlacement:
    ranges: List[Tuple[int, int]]

    @classmethod
    def uniform(cls, total: int, world: int) -> "ExpertPlacement":
        return cls([expert_range(total, r, world) for r in range(world)])

    @classmethod
    def weighted(cls, total: int, capacities: Sequence[float]) -> "ExpertPlacement":
        """Experts proportional to each rank's capacity (memory); every rank gets at least one."""
        world = len(capacities)
        tot = float(sum(capacities))
        raw = [max(1, int(total * c / tot)) for c in capacities]
        while sum(raw) > total:
            raw[raw.index(max(raw))] -= 1
        i = 0
        while sum(raw) < total:
            raw[i % world] += 1
            i += 1
        out, s = [], 0
        for n in raw:
            out.append((s, s + n))
            s += n
        return cls(out)

    def owner(self, expert: int) -> int:
        for r, (a, b) in enumerate(self.ranges):
            if a <= expert < b:
                return r
        raise IndexError(expert)


def expert_capacity(tokens: int, num_experts: int, top_k: int, capacity_factor: float = 1.25) -> int:
    return max(1, int(capacity_factor * tokens * top_k / num_experts + 0.999999))


def apply_capacity(idx: torch.Tensor, w: torch.Tensor, num_experts: int, capacity: int, redistribute: bool = False):
    """Tokens beyond an expert's capacity (in token order) are dropped (weight 0) or, with ``redistribute``, have the
    remaining weights of the token renormalised. Returns (weights, dropped mask [T, k])."""
    T, k = idx.shape
    flat = idx.reshape(-1)
    onehot = torch.nn.functional.one_hot(flat, num_experts)
    pos = (onehot.cumsum(0) * onehot).sum(-1) - 1              # arrival order within the expert
    dropped = (pos >= capacity).reshape(T, k)
    w2 = torch.where(dropped, torch.zeros_like(w), w)
    if redistribute:
        w2 = w2 / w2.sum(-1, keepdim=True).clamp(min=1e-8) * w.sum(-1, keepdim=True)
    return w2, dropped


def switch_aux_loss(router_probs: torch.Tensor, idx: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Load-balancing loss  E * sum_e f_e * P_e  (fraction of assignments to e times mean router probability of e)."""
    f = torch.bincount(idx.reshape(-1), minlength=num_experts).float() / idx.numel()
    return num_experts * (f * router_probs.float().mean(0)).sum()


# ------------------------------------------------------------------------------------------- fused engine
def interleave_gate_up(gate_up: torch.Tensor) -> torch.Tensor:
    """[E, 2I, H] with gate rows then up rows  ->  per expert, blocks of 128 gate rows followed by their 128 up rows."""
    E, two_i, H = gate_up.shape
    I = two_i // 2
    assert I % 128 == 0, "expert intermediate size must be a multiple of 128"
    g = gate_up[:, :I].reshape(E, I // 128, 128, H)
    u = gate_up[:, I:].reshape(E, I // 128, 128, H)
    return torch.stack([g, u], dim=2).reshape(E, two_i, H).contiguous()


class FusedExpertMoE:
    """Holds one MoE layer's local expert weights and the exchange buffers for up to ``max_tokens`` local tokens."""

    def __init__(self, gate_up_local: torch.Tensor, down_local: torch.Tensor, num_experts: int, top_k: int,
                 max_tokens: int, group=None, norm_topk_prob: bool = True, timeout_s: float = 10.0):
        self.group = group
        self.distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.rank = dist.get_rank(group) if self.distributed else 0
        self.world = dist.get_world_size(group) if self.distributed else 1
        self.E, self.k, self.renorm, self.timeout_s = num_experts, top_k, norm_topk_prob, timeout_s
        self.e_loc = gate_up_local.shape[0]
        assert self.e_loc * self.world == num_experts
        self.I, self.H = down_local.shape[2], down_local.shape[1]
        dev = gate_up_local.device
        self.w1 = interleave_gate_up(gate_up_local.to(torch.bfloat16)).reshape(self.e_loc * 2 * self.I, self.H)
        self.w2 = down_local.to(torch.bfloat16).contiguous().reshape(self.e_loc * self.H, self.I)
        self.max_rows = max_tokens * top_k
        # worst case every peer routes everything here; an expert's rows from all sources share 128-row tiles
        self.max_tiles = self.world * self.max_rows // 128 + self.e_loc + 1
        self.max_runs = self.max_tiles + self.world * self.e_loc
        self._keep = []
        self.sorted_x, self._x_ptrs = self._buf(self.max_rows * self.H, torch.bfloat16)
        self.z, self._z_ptrs = self._buf(self.max_rows * self.H, torch.bfloat16)
        self.offsets, self._off_ptrs = self._buf(num_experts + 1, torch.int32)
        self.pad, self._pad_ptrs = self._buf(32, torch.int32)
        self.pad.zero_()
        self.offsets.zero_()
        self.h = torch.empty(self.max_tiles * 128, self.I, dtype=torch.bfloat16, device=dev)
        arr = ctypes.c_ulonglong * self.world
        self._h_ptrs = arr(*([self.h.data_ptr()] * self.world))
        self.xin = torch.empty(self.max_tiles * 128, self.H, dtype=torch.bfloat16, device=dev)     # staged-in token rows
        self.tile_ready = torch.zeros(self.max_tiles, dtype=torch.int32, device=dev)
        self.tiles = torch.zeros(self.max_tiles * 8, dtype=torch.int32, device=dev)
        self.runs = torch.zeros(self.max_runs * 4, dtype=torch.int32, device=dev)
        self.counts = torch.zeros(2, dtype=torch.int32, device=dev)
        if self.distributed:
            torch.cuda.synchronize()
            dist.barrier(group)

    def _buf(self, numel: int, dtype):
        arr = ctypes.c_ulonglong * self.world
        dev = torch.device("cuda", torch.cuda.current_device())
        if not self.distributed:
            t = torch.empty(numel, dtype=dtype, device=dev)
            return t, arr(t.data_ptr())
        import torch.distributed._symmetric_memory as symm_mem
        t = symm_mem.empty(numel, dtype=dtype, device=dev)
        h = symm_mem.rendezvous(t, self.group if self.group is not None else dist.group.WORLD)
        self._keep.append(h)
        return t, arr(*[int(p) for p in h.buffer_ptrs])

    @torch.no_grad()
    def forward(self, x: torch.Tensor, router_logits: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [T, H] bf16 local tokens, router_logits [T, E]. Returns [T, H] bf16 (+ residual when given)."""
        from ..ops import native
        T = x.shape[0]
        n = T * self.k
        assert n <= self.max_rows and x.dtype == torch.bfloat16
        lib = native.lib()
        r = native.moe_route(router_logits, self.k, self.renorm, offsets_out=self.offsets)
        sx = self.sorted_x[: n * self.H].view(n, self.H)
        native._chk(lib.pm_moe_gather(native._p(x.contiguous()), native._p(r["perm"]), ctypes.c_int(self.k), native._p(sx),
                                      ctypes.c_longlong(n), ctypes.c_int(self.H), native._stream()), "pm_moe_gather")
        st = native.status_word()
        lib.pm_ep_prepare.restype = ctypes.c_int
        lib.pm_moe_gemm.restype = ctypes.c_int
        native._chk(lib.pm_ep_prepare(self._off_ptrs, self._pad_ptrs, ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                      ctypes.c_int(self.e_loc), native._p(self.tiles), native._p(self.runs),
                                      ctypes.c_int(self.max_tiles), ctypes.c_int(self.max_runs), native._p(self.counts),
                                      ctypes.c_double(self.timeout_s), native._p(st), native._stream()), "pm_ep_prepare")
        native._chk(lib.pm_moe_gemm(native._p(self.xin), ctypes.c_int(self.max_tiles * 128), ctypes.c_int(self.H),
                                    native._p(self.w1), ctypes.c_int(self.H), ctypes.c_int(self.e_loc), self._h_ptrs,
                                    ctypes.c_int(self.I), native._p(self.tiles), native._p(self.runs),
                                    native._p(self.counts), ctypes.c_int(self.max_tiles), ctypes.c_int(2 * self.I),
                                    ctypes.c_int(self.H), ctypes.c_int(1), ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                    ctypes.c_int(0), self._pad_ptrs, self._x_ptrs, native._p(self.tile_ready),
                                    ctypes.c_double(self.timeout_s), native._p(st), native._stream()), "pm_moe_gemm")
        native._chk(lib.pm_moe_gemm(native._p(self.h), ctypes.c_int(self.max_tiles * 128), ctypes.c_int(self.I),
                                    native._p(self.w2), ctypes.c_int(self.I), ctypes.c_int(self.e_loc), self._z_ptrs,
                                    ctypes.c_int(self.H), native._p(self.tiles), native._p(self.runs),
                                    native._p(self.counts), ctypes.c_int(self.max_tiles), ctypes.c_int(self.H),
                                    ctypes.c_int(self.I), ctypes.c_int(0), ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                    ctypes.c_int(1), self._pad_ptrs, None, None, ctypes.c_double(self.timeout_s),
                                    native._p(st), native._stream()), "pm_moe_gemm")
        zz = self.z[: n * self.H].view(n, self.H)
        res = residual.contiguous() if residual is not None and residual.dtype == torch.bfloat16 else None
        y = native.moe_combine(zz, r["inv"], r["topk_w"], self.k, res)
        return y if res is not None or residual is None else y + residual


def shard_experts(block, group=None, max_tokens: int = 16384) -> FusedExpertMoE:
    """Attach a fused engine holding this rank's slice of ``block``'s experts (a ``SparseMoeBlock``)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    a, b = expert_range(block.cfg.num_experts, rank, world)
    eng = FusedExpertMoE(block.gate_up.data[a:b], block.down.data[a:b], block.cfg.num_experts,
                         block.cfg.num_experts_per_tok, max_tokens, group, block.cfg.norm_topk_prob)
    block.ep_engine = eng
    block.ep_group = group if world > 1 else None
    block.local_experts = (a, b)
    return eng


def ep_moe_forward(block, x: torch.Tensor, w: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """Expert-parallel forward for a block prepared by ``shard_experts``. The fused engine redoes the routing on the
    device from the router logits, so ``w`` / ``idx`` are only used by the library-collective baseline below."""
    eng = getattr(block, "ep_engine", None)
    if eng is not None and x.is_cuda and not torch.is_grad_enabled():
        logits = torch.nn.functional.linear(x, block.router)
        return eng.forward(x.to(torch.bfloat16), logits).to(x.dtype)
    return ep_moe_forward_nccl(block, x, w, idx)


def ep_moe_forward_nccl(block, x: torch.Tensor, w: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """Baseline with library collectives: all-gather tokens and assignments, run the local experts on everything
    routed to them, reduce-scatter the weighted results."""
    group = block.ep_group
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    a, b = block.local_experts
    T, H = x.shape
    xs = torch.empty(world * T, H, dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(xs, x.contiguous(), group=group)
    ws = torch.empty(world * T, w.shape[1], dtype=w.dtype, device=x.device)
    dist.all_gather_into_tensor(ws, w.contiguous(), group=group)
    ids = torch.empty(world * T, idx.shape[1], dtype=idx.dtype, device=x.device)
    dist.all_gather_into_tensor(ids, idx.contiguous(), group=group)
    out = torch.zeros(world * T, H, dtype=torch.float32, device=x.device)
    I = block.cfg.moe_intermediate_size
    for e in range(a, b):
        tok, slot = (ids == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        hgu = torch.nn.functional.linear(xs[tok], block.gate_up[e])
        hh = torch.nn.functional.silu(hgu[:, :I]) * hgu[:, I:]
        y = torch.nn.functional.linear(hh, block.down[e]).float() * ws[tok, slot].float()[:, None]
        out.index_add_(0, tok, y)
    mine = torch.empty(T, H, dtype=torch.float32, device=x.device)
    dist.reduce_scatter_tensor(mine, out, group=group)
    return mine.to(x.dtype)
