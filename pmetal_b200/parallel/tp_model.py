"""Tensor-parallel attention plus expert-parallel mixture-of-experts for serving one model on several GPUs.

``shard_for_serving(model, group)`` rewrites a ``DecoderLM`` in place so that every rank keeps

* the query heads ``[r * hq / W, (r + 1) * hq / W)`` of every attention layer together with the key/value heads they
  read (a slice of the kv heads when there are at least ``W`` of them, otherwise the one kv head the rank's query heads
  share: fewer kv heads than ranks means replication, as in the reference's plan,
  crates/pmetal-distributed/src/tensor_parallel/plan.rs:50-140), the matching columns of ``o_proj``
  (crates/pmetal-distributed/src/tensor_parallel/sharded_linear.rs:41-106: column-parallel q/k/v, row-parallel o), and a
  paged KV cache for its own kv heads only;
* the experts ``[r * E / W, (r + 1) * E / W)`` of every mixture-of-experts layer; dense feed-forward layers are split by
  intermediate channel (column-parallel gate/up, row-parallel down).

Activations are replicated: every rank runs every token through its slice, and the two partial results of a layer (the
attention output projection and the feed-forward) are summed across ranks. For the expert layers this is expert
parallelism without a dispatch step: a token already is where its experts are, so the exchange is one sum of
``[tokens, hidden]`` instead of two all-to-alls, which is the cheaper form for the few hundred tokens of a decode or
verification step (the all-to-all engine of ``parallel/ep.py`` remains the choice for sequence-sharded prefill).
The sum runs in ``AllReduce``: NCCL by default, or a one-kernel exchange over symmetric memory for small messages
(``PeerAllReduce``: every rank writes its partial into every peer's slot and sums the slots it received).

Expert routing, the padded expert-sorted layout, the grouped tcgen05 GEMMs and the weighted combine are the kernels of
``csrc/moe_quant.cu`` / ``csrc/grouped_gemm.cu``; on CPU (tests over gloo) the same arithmetic runs in PyTorch.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F


# ------------------------------------------------------------------------------------------- collectives
class AllReduce:
    """Sum of a replicated-shape tensor over the group (in place)."""

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(x, group=self.group)
        return x


class PeerAllReduce(AllReduce):
    """All-reduce of small bf16 messages in one kernel over symmetric memory (csrc/tp_fused.cu: ``peer_allreduce``):
    every rank stores its vector into slot ``rank`` of every peer's buffer, raises a flag there, waits (bounded) for the
    flags of all peers in its own buffer and sums the ``world`` slots. Two buffers alternate so that a rank that is one
    call ahead never overwrites a slot a slower peer is still reading. Larger messages fall back to NCCL."""

    def __init__(self, group=None, max_elems: int = 1 << 20, timeout_s: float = 10.0):
        super().__init__(group)
        self.rank = dist.get_rank(group)
        self.max_elems, self.timeout_s = max_elems, timeout_s
        import torch.distributed._symmetric_memory as symm_mem
        dev = torch.device("cuda", torch.cuda.current_device())
        g = group if group is not None else dist.group.WORLD
        self.buf = symm_mem.empty(2 * self.world * max_elems, dtype=torch.bfloat16, device=dev)
        hb = symm_mem.rendezvous(self.buf, g)
        self.pad = symm_mem.empty(64, dtype=torch.int32, device=dev)
        self.pad.zero_()
        hp = symm_mem.rendezvous(self.pad, g)
        arr = ctypes.c_ulonglong * self.world
        self._bufs = arr(*[int(p) for p in hb.buffer_ptrs])
        self._pads = arr(*[int(p) for p in hp.buffer_ptrs])
        self._keep = (hb, hp)
        self.calls = 0
        torch.cuda.synchronize()
        dist.barrier(group)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        n = x.numel()
        if self.world == 1:
            return x
        if x.dtype != torch.bfloat16 or n > self.max_elems or n % 8 or not x.is_contiguous():
            dist.all_reduce(x, group=self.group)
            return x
        from ..ops import native
        lib = native.lib()
        lib.pm_peer_allreduce.restype = ctypes.c_int
        self.calls += 1
        rc = lib.pm_peer_allreduce(native._p(x), ctypes.c_longlong(n), self._bufs, self._pads,
                                   ctypes.c_longlong(self.max_elems), ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                   ctypes.c_double(self.timeout_s), native._p(native.status_word()), native._stream())
        native._chk(rc, "pm_peer_allreduce")
        return x


# ------------------------------------------------------------------------------------------- head / expert ranges
def head_shard(hq: int, hkv: int, rank: int, world: int) -> Tuple[int, int, int, int]:
    """(first query head, query heads, first kv head, kv heads) of ``rank``. Query heads are split evenly; kv heads
    are split when there are enough of them and otherwise the single head that the rank's query heads read is kept."""
    if hq % world:
        raise ValueError(f"{hq} query heads do not divide over {world} ranks")
    q_loc = hq // world
    q0 = rank * q_loc
    rep = hq // hkv
    if hkv % world == 0:
        kv_loc = hkv // world
        return q0, q_loc, rank * kv_loc, kv_loc
    if q_loc > rep or rep % q_loc:
        raise ValueError(f"{hkv} kv heads cannot be replicated cleanly over {world} ranks ({hq} query heads)")
    return q0, q_loc, q0 // rep, 1


def _slice_rows(w: torch.Tensor, pieces) -> torch.Tensor:
    return torch.cat([w[a:b] for a, b in pieces], 0).contiguous()


@torch.no_grad()
def shard_for_serving(model, group=None, reduce: Optional[AllReduce] = None, rank: Optional[int] = None,
                      world: Optional[int] = None) -> AllReduce:
    """Cut ``model`` (a frozen ``DecoderLM`` without adapters) down to this rank's slice; see the module docstring.
    Returns the all-reduce object the layers use. ``rank`` / ``world`` override the process group's (cutting a slice
    offline, or timing one rank's share of the work on a single device with a ``reduce`` that does nothing)."""
    from ..models.decoder import MLP, FusedLinear
    if world is None:
        world = dist.get_world_size(group) if dist.is_initialized() else 1
    if rank is None:
        rank = dist.get_rank(group) if dist.is_initialized() else 0
    reduce = reduce or AllReduce(group)
    cfg = model.cfg
    hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    q0, q_loc, kv0, kv_loc = head_shard(hq, hkv, rank, world)
    for layer in model.layers:
        at = layer.self_attn
        qkv, o = at.qkv_proj, at.o_proj
        if qkv.lora_a is not None or o.lora_a is not None or getattr(qkv, "qweight", None) is not None:
            raise ValueError("tensor-parallel serving expects merged bf16 weights (fuse adapters first)")
        rows = [(q0 * d, (q0 + q_loc) * d), (hq * d + kv0 * d, hq * d + (kv0 + kv_loc) * d),
                ((hq + hkv) * d + kv0 * d, (hq + hkv) * d + (kv0 + kv_loc) * d)]
        nq = FusedLinear(qkv.in_features, qkv.seg_names, (q_loc * d, kv_loc * d, kv_loc * d), qkv.bias is not None,
                         qkv.weight.dtype, qkv.weight.device)
        nq.weight.data = _slice_rows(qkv.weight.data, rows)
        if qkv.bias is not None:
            nq.bias.data = _slice_rows(qkv.bias.data, rows)
        no = FusedLinear(q_loc * d, o.seg_names, o.seg_sizes, False, o.weight.dtype, o.weight.device)
        no.weight.data = o.weight.data[:, q0 * d:(q0 + q_loc) * d].contiguous()
        for m in (nq, no):
            m.weight.requires_grad_(False)
        at.qkv_proj, at.o_proj = nq, no
        at.hq_local, at.hkv_local, at.tp_reduce = q_loc, kv_loc, reduce
        mlp = layer.mlp
        if isinstance(mlp, MLP):
            I = mlp.down_proj.in_features
            if I % world:
                raise ValueError(f"intermediate size {I} does not divide over {world} ranks")
            il = I // world
            gu, dn = mlp.gate_up_proj, mlp.down_proj
            ng = FusedLinear(gu.in_features, gu.seg_names, (il, il), False, gu.weight.dtype, gu.weight.device)
            ng.weight.data = _slice_rows(gu.weight.data, [(rank * il, (rank + 1) * il), (I + rank * il, I + (rank + 1) * il)])
            nd = FusedLinear(il, dn.seg_names, dn.seg_sizes, False, dn.weight.dtype, dn.weight.device)
            nd.weight.data = dn.weight.data[:, rank * il:(rank + 1) * il].contiguous()
            for m in (ng, nd):
                m.weight.requires_grad_(False)
            mlp.gate_up_proj, mlp.down_proj = ng, nd
            mlp.tp_reduce = reduce
        else:
            E = cfg.num_experts
            if E % world:
                raise ValueError(f"{E} experts do not divide over {world} ranks")
            e_loc = E // world
            mlp.gate_up = torch.nn.Parameter(mlp.gate_up.data[rank * e_loc:(rank + 1) * e_loc].contiguous(), requires_grad=False)
            mlp.down = torch.nn.Parameter(mlp.down.data[rank * e_loc:(rank + 1) * e_loc].contiguous(), requires_grad=False)
            mlp.local_experts = (rank * e_loc, (rank + 1) * e_loc)
            mlp.tp_reduce = reduce
            mlp.ep_rank = rank
    model.kv_heads_local = kv_loc
    model.tp_world, model.tp_rank = world, rank
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    return reduce


# ------------------------------------------------------------------------------------------- local experts
class _Scratch:
    """Per-layer-shape buffers of the local-expert path, reused across steps (and CUDA-graph replays)."""

    def __init__(self):
        self.by_key = {}

    def get(self, T: int, k: int, e_loc: int, H: int, I: int, dev) -> dict:
        key = (T, k, e_loc, H, I, str(dev))
        b = self.by_key.get(key)
        if b is None:
            n = T * k
            cap = -(-(n + e_loc * 127) // 128) * 128
            i32 = lambda *s: torch.empty(*s, dtype=torch.int32, device=dev)      # noqa: E731
            b = self.by_key[key] = dict(cap=cap, idx=i32(T, k), w=torch.empty(T, k, dtype=torch.float32, device=dev),
                                        off=i32(e_loc + 1), dest=i32(n), src=i32(cap),
                                        xs=torch.empty(cap, H, dtype=torch.bfloat16, device=dev))
        return b


_SCRATCH = _Scratch()
SKINNY_MAX_TOKENS = int(__import__("os").environ.get("PMETAL_MOE_SKINNY_TOKENS", "128"))


def moe_local_forward(block, x: torch.Tensor, residual: Optional[torch.Tensor]) -> torch.Tensor:
    """Feed-forward of a mixture-of-experts block whose experts are split over ranks, for replicated tokens ``x``
    [T, H]: route over all experts, apply this rank's experts to the assignments that fall on them, sum the partial
    outputs over ranks, add the residual."""
    cfg = block.cfg
    e0, e1 = block.local_experts
    k = cfg.num_experts_per_tok
    T, H = x.shape
    from ..ops import functional as ops
    logits = F.linear(x, block.router)
    if ops.use_native(x) and H % 8 == 0:
        from ..ops import native as nat
        I = block.down.shape[2]
        lib = nat.lib()
        for fn in ("pm_moe_route_local", "pm_moe_gather_padded", "pm_moe_combine_local"):
            getattr(lib, fn).restype = ctypes.c_int
        lg = logits.contiguous()
        is_f32 = int(lg.dtype == torch.float32)
        if not is_f32 and lg.dtype != torch.bfloat16:
            lg, is_f32 = lg.float(), 1
        ci = ctypes.c_int
        y = torch.empty_like(x)
        # the residual joins the sum exactly once: on the rank that owns the first experts
        res = residual if (residual is not None and block.ep_rank == 0) else None
        step = max(4096 // k, 1)            # the one-CTA routing kernel handles 4096 assignments per call
        for t0 in range(0, T, step):
            n = min(step, T - t0)
            b = _SCRATCH.get(n, k, e1 - e0, H, I, x.device)
            xs_in, lg_in = x[t0:t0 + n], lg[t0:t0 + n]
            # a decode or verification step gives an expert at most n rows (one per token): the swapped-operand
            # kernels stream the weights once, need no slab padding and fuse SwiGLU; larger batches use 128-row tiles
            few = n <= SKINNY_MAX_TOKENS
            nat._chk(lib.pm_moe_route_local(nat._p(lg_in), ci(is_f32), ci(n), ci(cfg.num_experts), ci(k),
                                            ci(int(cfg.norm_topk_prob)), ci(e0), ci(e1 - e0), ci(1 if few else 128),
                                            nat._p(b["idx"]), nat._p(b["w"]), nat._p(b["off"]), nat._p(b["dest"]),
                                            nat._p(b["src"]), nat._stream()), "pm_moe_route_local")
            nat._chk(lib.pm_moe_gather_padded(nat._p(xs_in), nat._p(b["src"]), nat._p(b["off"][e1 - e0:]), ci(k),
                                              nat._p(b["xs"]), ci(b["cap"]), ci(H), nat._stream()), "pm_moe_gather_padded")
            if few:
                act = nat.grouped_gemm_skinny(b["xs"], block.gate_up, b["off"], swiglu=True, max_rows_per_expert=n)
                z = nat.grouped_gemm_skinny(act, block.down, b["off"], max_rows_per_expert=n)
            else:
                gu = nat.grouped_gemm(0, b["xs"], block.gate_up, b["off"], 2 * I, H)
                act = nat.swiglu_fwd(gu)
                z = nat.grouped_gemm(0, act, block.down, b["off"], H, I)
            nat._chk(lib.pm_moe_combine_local(nat._p(z), nat._p(b["dest"]), nat._p(b["w"]), ci(k),
                                              nat._p(res[t0:t0 + n] if res is not None else None), nat._p(y[t0:t0 + n]),
                                              ctypes.c_longlong(n), ci(H), nat._stream()), "pm_moe_combine_local")
        return block.tp_reduce(y)
    from ..models.moe import route_topk
    w, idx = route_topk(logits, k, cfg.norm_topk_prob)
    y = torch.zeros_like(x, dtype=torch.float32)
    for e in range(e0, e1):
        hit = (idx == e)
        rows = hit.any(-1).nonzero().flatten()
        if rows.numel() == 0:
            continue
        xe = x[rows]
        g = F.linear(xe, block.gate_up[e - e0])
        half = g.shape[-1] // 2
        oe = F.linear(F.silu(g[:, :half]) * g[:, half:], block.down[e - e0])
        y[rows] += (w[rows] * hit[rows]).sum(-1, keepdim=True).float() * oe.float()
    if residual is not None and block.ep_rank == 0:
        y += residual.float()
    return block.tp_reduce(y).to(x.dtype)
