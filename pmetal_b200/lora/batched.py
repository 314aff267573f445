"""Several LoRA adapters in one batch: every row of the input picks its adapter by index (S-LoRA style serving of many
fine-tunes over one base model; cf. the reference's ``BatchedLora`` / ``BatchedLoraAdapters``,
crates/pmetal-metal/src/kernels/batched_lora.rs:290-330).

    y[t] = x[t] W^T + scale[id(t)] * (x[t] A_id(t)^T) B_id(t)^T          id(t) = -1: base model only

The base product is one dense GEMM for the whole batch. The low-rank part is two *grouped* GEMMs over the rows sorted by
adapter, i.e. the expert kernels with "adapter" in the place of "expert": the swapped-operand kernel for the handful of
rows of a decode step, the 128-row-tile kernel for prefill (csrc/grouped_gemm.cu). For a fused projection (q|k|v, gate|up)
the factors are stored as ``A`` [n_seg r, K] stacked over the segments and ``B`` [N, n_seg r] block-diagonal, so the whole
group is still two products. On CPU the same arithmetic runs as a loop over the adapters that occur in the batch."""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

NO_ADAPTER = -1


class BatchedLoraAdapters:
    """Factor storage for up to ``max_adapters`` adapters of one (possibly fused) projection."""

    def __init__(self, max_adapters: int, in_features: int, seg_sizes: Sequence[int], rank: int, dtype=torch.bfloat16,
                 device=None):
        self.n, self.k, self.r = max_adapters, in_features, rank
        self.seg_sizes = tuple(int(s) for s in seg_sizes)
        self.out = sum(self.seg_sizes)
        self.rt = len(self.seg_sizes) * rank                     # stacked rank of the fused projection
        # slot n is the all-zero adapter that rows with NO_ADAPTER are sent to
        self.a = torch.zeros(max_adapters + 1, self.rt, in_features, dtype=dtype, device=device)
        self.b = torch.zeros(max_adapters + 1, self.out, self.rt, dtype=dtype, device=device)
        self.scale = torch.zeros(max_adapters + 1, dtype=torch.float32, device=device)
        self.loaded = [False] * max_adapters

    @torch.no_grad()
    def load_adapter(self, idx: int, a: torch.Tensor, b: torch.Tensor, scale: float) -> None:
        """``a`` [n_seg r, K] stacked over segments, ``b`` [N, r] (row block of each segment), as ``FusedLinear`` keeps them."""
        if not 0 <= idx < self.n:
            raise IndexError(f"adapter slot {idx} outside 0..{self.n - 1}")
        if tuple(a.shape) != (self.rt, self.k) or tuple(b.shape) != (self.out, self.r):
            raise ValueError(f"adapter factors {tuple(a.shape)} / {tuple(b.shape)} do not match "
                             f"{(self.rt, self.k)} / {(self.out, self.r)}")
        self.a[idx].copy_(a)
        self.b[idx].zero_()
        o = 0
        for s, sz in enumerate(self.seg_sizes):
            self.b[idx, o:o + sz, s * self.r:(s + 1) * self.r].copy_(b[o:o + sz])
            o += sz
        self.scale[idx] = float(scale)
        self.loaded[idx] = True

    def unload_adapter(self, idx: int) -> None:
        self.a[idx].zero_()
        self.b[idx].zero_()
        self.scale[idx] = 0.0
        self.loaded[idx] = False


def _sorted_layout(ids: torch.Tensor, n_slots: int):
    """Rows grouped by adapter: (order [T] so that x[order] is sorted, off int32 [n_slots + 1]). Device-side only."""
    order = torch.argsort(ids, stable=True)
    counts = torch.bincount(ids, minlength=n_slots)
    off = torch.zeros(n_slots + 1, dtype=torch.int32, device=ids.device)
    off[1:] = torch.cumsum(counts, 0).to(torch.int32)
    return order, off


def batched_lora_delta(x: torch.Tensor, ids: torch.Tensor, store: BatchedLoraAdapters) -> torch.Tensor:
    """scale[id] * (x A_id^T) B_id^T for every row; ``ids`` int64 [T] with NO_ADAPTER for rows that use the base model."""
    T = x.shape[0]
    slot = torch.where(ids < 0, torch.full_like(ids, store.n), ids)
    from ..ops import functional as ops
    if ops.use_native(x) and store.k % 8 == 0 and store.rt % 8 == 0 and store.out % 8 == 0:
        from ..ops import native as nat
        order, off = _sorted_layout(slot, store.n + 1)
        xs = x.index_select(0, order).contiguous()
        if T <= 128:                   # a decode or verification step: few rows per adapter, unpadded slabs
            t = nat.grouped_gemm_skinny(xs, store.a, off, max_rows_per_expert=T)
            d = nat.grouped_gemm_skinny(t, store.b, off, max_rows_per_expert=T)
        else:                          # prefill: 128-row tiles in the padded layout
            dest, poff, cap = ops.padded_expert_layout(slot.reshape(-1, 1), store.n + 1)
            xp = torch.zeros(cap, store.k, dtype=x.dtype, device=x.device).index_copy_(0, dest, x)
            t = nat.grouped_gemm(0, xp, store.a, poff, store.rt, store.k)
            d = nat.grouped_gemm(0, t, store.b, poff, store.out, store.rt)
            return d.index_select(0, dest) * store.scale[slot].to(d.dtype)[:, None]
        out = torch.empty_like(d)
        out.index_copy_(0, order, d * store.scale[slot.index_select(0, order)].to(d.dtype)[:, None])
        return out
    out = torch.zeros(T, store.out, dtype=x.dtype, device=x.device)
    for i in torch.unique(slot).tolist():
        if i == store.n:
            continue
        rows = (slot == i).nonzero().flatten()
        t = F.linear(x[rows], store.a[i].to(x.dtype))
        out[rows] = (F.linear(t, store.b[i].to(x.dtype)) * store.scale[i].to(x.dtype)).to(x.dtype)
    return out


def batched_lora_linear(x: torch.Tensor, weight: torch.Tensor, store: BatchedLoraAdapters, ids: torch.Tensor,
                        residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Base projection for the whole batch plus each row's own adapter."""
    from ..ops import functional as ops
    if ops.use_native(x) and weight.dtype == torch.bfloat16:
        from ..ops import native as nat
        y = nat.gemm(x, weight, residual=residual)
    else:
        y = F.linear(x, weight.to(x.dtype))
        if residual is not None:
            y = y + residual
    return y + batched_lora_delta(x, ids, store)


# ------------------------------------------------------------------------------------------- whole models
class AdapterSet:
    """Named adapters attached to every fused projection of a ``DecoderLM``; ``set_rows`` says which adapter each row of
    the next forward uses. Adapters are read from directories written by ``lora.adapter.save_adapter``."""

    def __init__(self, model, max_adapters: int, rank: int):
        self.model, self.max_adapters, self.rank = model, max_adapters, rank
        self.names: List[Optional[str]] = [None] * max_adapters
        p = model.embed_tokens
        for _, _, fl in model.fused_linears():
            fl.batched = BatchedLoraAdapters(max_adapters, fl.in_features, fl.seg_sizes, rank, p.dtype if p.is_cuda
                                             else torch.float32, p.device)
        model.adapter_rows = None

    def index(self, name: Optional[str]) -> int:
        if name is None or name == "":
            return NO_ADAPTER
        if name not in self.names:
            raise KeyError(f"unknown adapter {name!r}; loaded: {[n for n in self.names if n]}")
        return self.names.index(name)

    @torch.no_grad()
    def load(self, name: str, adapter_dir: str, slot: Optional[int] = None) -> int:
        """Load ``lora_weights.safetensors`` + ``adapter_config.json`` from ``adapter_dir`` into a free slot."""
        from ..utils import safetensors_io as st
        if slot is None:
            slot = self.names.index(name) if name in self.names else self.names.index(None)
        with open(os.path.join(adapter_dir, "adapter_config.json"), "r", encoding="utf-8") as fh:
            cfg = json.load(fh)
        r = int(cfg.get("r", cfg.get("rank", self.rank)))
        if r != self.rank:
            raise ValueError(f"adapter rank {r} differs from the set's rank {self.rank}")
        alpha = float(cfg.get("lora_alpha", cfg.get("alpha", r)))
        scale = alpha / (r ** 0.5 if cfg.get("use_rslora") else r)
        sd = st.load_file(os.path.join(adapter_dir, "lora_weights.safetensors"))
        self.load_state(name, sd, scale, slot)
        return slot

    @torch.no_grad()
    def load_state(self, name: str, sd: Dict[str, torch.Tensor], scale: float, slot: int) -> None:
        """``sd`` in the adapter file's key layout: ``layers.{i}.{block}.{proj}.lora_a`` [r, K] / ``.lora_b`` [N, r]."""
        for i, block, fl in self.model.fused_linears():
            st_ = fl.batched
            a = torch.zeros(st_.rt, st_.k)
            b = torch.zeros(st_.out, st_.r)
            o = 0
            for s, (seg, sz) in enumerate(zip(fl.seg_names, fl.seg_sizes)):
                ka, kb = f"layers.{i}.{block}.{seg}.lora_a", f"layers.{i}.{block}.{seg}.lora_b"
                if ka in sd and sd[ka].shape[0] == st_.r:
                    a[s * st_.r:(s + 1) * st_.r] = sd[ka].float()
                    b[o:o + sz] = sd[kb].float()
                o += sz
            st_.load_adapter(slot, a.to(st_.a.device), b.to(st_.b.device), scale)
        self.names[slot] = name

    def unload(self, name: str) -> None:
        slot = self.names.index(name)
        for _, _, fl in self.model.fused_linears():
            fl.batched.unload_adapter(slot)
        self.names[slot] = None

    def set_rows(self, ids) -> None:
        """Adapter index of every row of the next forward (int64 tensor or list; NO_ADAPTER = base model); None turns
        the adapters off."""
        rows = None
        if ids is not None:
            rows = torch.as_tensor(ids, dtype=torch.int64, device=self.model.embed_tokens.device)
        self.model.adapter_rows = rows
        for _, _, fl in self.model.fused_linears():
            fl.adapter_rows = rows
