"""Mixture-of-experts inference with the routed experts kept on disk (``--experts-dir``).

``pack-experts`` writes one ``layer_NN.bin`` per MoE layer (expert ``E`` at byte ``E * expert_size``; gate, up and down
as affine 4- or 2-bit groups with bf16 scales and biases) and a ``layout.json``. This module is the reader side:

* ``PackedExpertStore``  positional reads (``os.preadv``) of whole expert records on a persistent thread pool, into
  pinned host buffers when a GPU is present; a bounded host LRU of raw records doubles as the landing zone of the
  prefetcher; counters for reads, bytes, seconds and prefetch hits / misses.
* ``LayerExperts``       the device side of one layer: a fixed pool of ``slots`` dequantised experts
  (``gate_up`` [S, 2I, H], ``down`` [S, H, I]) with least-recently-used replacement. A forward maps the routed expert
  ids to slot ids, so the grouped expert GEMMs run on the pool as they would on the full stack, without a copy.
* ``enable_expert_offloading``  drops the stacked expert parameters of every ``SparseMoeBlock`` and attaches the above;
  while a layer computes, the next MoE layer's router is applied to this layer's input to predict its experts, and
  their records are read in the background.

With 180 GB of HBM per GPU and expert parallelism this is for models that exceed one node's memory, or for keeping most
of a GPU free; the file format is the reference's, so packed directories are interchangeable.
Reference: crates/pmetal-models/src/expert_io.rs (pread pool, file manager), expert_layout.rs (record layout),
expert_prefetch.rs (next-layer prediction, hit-rate), expert_dequant.rs (bytes to typed weights)."""
from __future__ import annotations

import json
import os
import threading
import time
from collections import OrderedDict
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

FIELDS = (("weight", torch.int32), ("scales", torch.bfloat16), ("biases", torch.bfloat16))


class PackedExpertStore:
    def __init__(self, pack_dir: str, threads: int = 8, host_cache_bytes: int = 8 << 30):
        with open(os.path.join(pack_dir, "layout.json"), "r", encoding="utf-8") as fh:
            self.layout = json.load(fh)
        lay = self.layout
        self.bits = {"Four": 4, "Two": 2}.get(lay["bits"], lay["bits"])
        self.group_size, self.expert_size = int(lay["group_size"]), int(lay["expert_size"])
        self.hidden, self.inter, self.num_experts = int(lay["hidden_dim"]), int(lay["intermediate_dim"]), int(lay["num_experts"])
        self.record = lay.get("record") or _default_record(self.hidden, self.inter, self.group_size, self.bits)
        self.layers: List[int] = list(lay["moe_layer_indices"])
        self.fds: Dict[int, int] = {}
        for layer in self.layers:
            path = os.path.join(pack_dir, f"layer_{layer:02d}.bin")
            want = self.num_experts * self.expert_size
            if os.path.getsize(path) < want:
                raise ValueError(f"{path}: {os.path.getsize(path)} bytes, {want} expected")
            self.fds[layer] = os.open(path, os.O_RDONLY)
        self.pool = ThreadPoolExecutor(max_workers=max(1, threads), thread_name_prefix="pmetal-expert-io")
        self.pin = torch.cuda.is_available()
        self.host_cache_bytes = host_cache_bytes
        self._host: "OrderedDict[Tuple[int, int], torch.Tensor]" = OrderedDict()
        self._pending: Dict[Tuple[int, int], Future] = {}
        self._prefetched: set = set()
        self._lock = threading.Lock()
        self.stats = {"reads": 0, "bytes": 0, "read_seconds": 0.0, "prefetch_hits": 0, "prefetch_misses": 0,
                      "prefetch_issued": 0}

    # ------------------------------------------------------------------ reads
    def _read_one(self, layer: int, expert: int) -> torch.Tensor:
        if not 0 <= expert < self.num_experts:
            raise IndexError(f"expert {expert} out of range (0..{self.num_experts - 1})")
        t0 = time.perf_counter()
        buf = torch.empty(self.expert_size, dtype=torch.uint8, pin_memory=self.pin)
        view = memoryview(buf.numpy())
        got, base = 0, expert * self.expert_size
        while got < self.expert_size:                       # a positional read may return short
            n = os.preadv(self.fds[layer], [view[got:]], base + got)
            if n <= 0:
                raise IOError(f"short read of expert {expert} in layer {layer}")
            got += n
        with self._lock:
            self.stats["reads"] += 1
            self.stats["bytes"] += self.expert_size
            self.stats["read_seconds"] += time.perf_counter() - t0
        return buf

    def _remember(self, key: Tuple[int, int], buf: torch.Tensor) -> None:
        self._host[key] = buf
        self._host.move_to_end(key)
        while len(self._host) * self.expert_size > self.host_cache_bytes and len(self._host) > 1:
            old, _ = self._host.popitem(last=False)
            self._prefetched.discard(old)

    def prefetch(self, layer: int, experts: Iterable[int]) -> int:
        """Start background reads of records that are neither cached nor on their way; returns how many were started."""
        n = 0
        with self._lock:
            for e in experts:
                key = (layer, int(e))
                if key in self._host or key in self._pending:
                    continue
                self._pending[key] = self.pool.submit(self._read_one, layer, int(e))
                self._prefetched.add(key)
                n += 1
            self.stats["prefetch_issued"] += n
        return n

    def raw(self, layer: int, experts: Sequence[int]) -> List[torch.Tensor]:
        """The records of ``experts`` as uint8 host tensors. Records the prefetcher brought (or is bringing) count as
        hits, the others are read now, in parallel."""
        keys = [(layer, int(e)) for e in experts]
        futs: Dict[Tuple[int, int], Future] = {}
        got: Dict[Tuple[int, int], torch.Tensor] = {}           # held here: the host LRU may evict during this call
        with self._lock:
            for key in keys:
                if key in got or key in futs:
                    continue
                if key in self._host:
                    got[key] = self._host[key]
                    self._host.move_to_end(key)
                    if key in self._prefetched:
                        self.stats["prefetch_hits"] += 1
                        self._prefetched.discard(key)
                elif key in self._pending:
                    futs[key] = self._pending[key]
                    self.stats["prefetch_hits"] += 1
                    self._prefetched.discard(key)
                else:
                    futs[key] = self._pending[key] = self.pool.submit(self._read_one, *key)
                    self.stats["prefetch_misses"] += 1
        for key, f in futs.items():
            got[key] = f.result()
            with self._lock:
                self._pending.pop(key, None)
                self._remember(key, got[key])
        with self._lock:
            self._collect_finished()
        return [got[k] for k in keys]

    def _collect_finished(self) -> None:
        for key in [k for k, f in self._pending.items() if f.done()]:
            f = self._pending.pop(key)
            if f.exception() is None:
                self._remember(key, f.result())

    # ------------------------------------------------------------------ bytes to weights
    def dequantize(self, raw: torch.Tensor, dtype=torch.bfloat16) -> Tuple[torch.Tensor, torch.Tensor]:
        """``raw`` [U, expert_size] uint8 (any device) -> ``gate_up`` [U, 2I, H] and ``down`` [U, H, I]."""
        from ..quant.mlx_affine import dequantize_affine
        mats = {}
        for name in ("gate", "up", "down"):
            parts = {}
            for field, dt in FIELDS:
                c = self.record[f"{name}_{field}"]
                cols = raw[:, c["offset"]:c["offset"] + c["size"]].contiguous()
                parts[field] = cols.view(dt).reshape(raw.shape[0], *c["shape"])
            mats[name] = dequantize_affine(parts["weight"], parts["scales"], parts["biases"], self.bits, self.group_size, dtype)
        return torch.cat([mats["gate"], mats["up"]], 1), mats["down"]

    def fetch(self, layer: int, experts: Sequence[int], device, dtype=torch.bfloat16) -> Tuple[torch.Tensor, torch.Tensor]:
        bufs = self.raw(layer, experts)
        dev = torch.device(device)
        if dev.type == "cuda":
            raw = torch.empty(len(bufs), self.expert_size, dtype=torch.uint8, device=dev)
            for i, b in enumerate(bufs):
                raw[i].copy_(b, non_blocking=True)
        else:
            raw = torch.stack(bufs)
        return self.dequantize(raw, dtype)

    def hit_rate(self) -> float:
        n = self.stats["prefetch_hits"] + self.stats["prefetch_misses"]
        return self.stats["prefetch_hits"] / n if n else 0.0

    def close(self) -> None:
        self.pool.shutdown(wait=True)
        for fd in self.fds.values():
            os.close(fd)
        self.fds.clear()
        self._host.clear()
        self._pending.clear()


def _default_record(hidden: int, inter: int, group: int, bits: int) -> dict:
    """Field table of a layout file that carries none (directories written by the reference's packer)."""
    pf = 32 // bits
    comps, off = {}, 0
    for name, rows, cols in (("gate", inter, hidden), ("up", inter, hidden), ("down", hidden, inter)):
        for field, size, shape in ((f"{name}_weight", rows * (cols // pf) * 4, [rows, cols // pf]),
                                   (f"{name}_scales", rows * (cols // group) * 2, [rows, cols // group]),
                                   (f"{name}_biases", rows * (cols // group) * 2, [rows, cols // group])):
            comps[field] = {"offset": off, "size": size, "shape": shape}
            off += size
    return comps


class LayerExperts:
    """Device pool of one layer: ``slots`` dequantised experts with least-recently-used replacement."""

    def __init__(self, store: PackedExpertStore, layer: int, slots: int):
        self.store, self.layer = store, layer
        self.slots = max(1, min(slots, store.num_experts))
        self.slot_of: "OrderedDict[int, int]" = OrderedDict()      # expert -> slot, oldest first
        self.free: List[int] = []
        self.gate_up: Optional[torch.Tensor] = None
        self.down: Optional[torch.Tensor] = None
        self.loads = 0
        self.reuses = 0

    def _ensure(self, device, dtype, need: int) -> None:
        s = self.store
        if self.gate_up is not None and self.gate_up.device == device and self.gate_up.dtype == dtype and need <= self.slots:
            return
        self.slots = max(self.slots, need)                  # one call may route to more experts than the pool held
        self.gate_up = torch.empty(self.slots, 2 * s.inter, s.hidden, dtype=dtype, device=device)
        self.down = torch.empty(self.slots, s.hidden, s.inter, dtype=dtype, device=device)
        self.slot_of.clear()
        self.free = list(range(self.slots - 1, -1, -1))

    def slots_for(self, experts: Sequence[int], device, dtype) -> Dict[int, int]:
        """Make ``experts`` resident; returns expert -> slot. Experts of this call are never evicted by it."""
        experts = [int(e) for e in experts]
        self._ensure(torch.device(device), dtype, len(experts))
        missing = [e for e in experts if e not in self.slot_of]
        for e in experts:
            if e in self.slot_of:
                self.slot_of.move_to_end(e)
                self.reuses += 1
        if missing:
            keep = set(experts)
            targets = []
            for e in missing:
                if self.free:
                    slot = self.free.pop()
                else:
                    victim = next(v for v in self.slot_of if v not in keep)
                    slot = self.slot_of.pop(victim)
                targets.append(slot)
            gu, dn = self.store.fetch(self.layer, missing, device, dtype)
            idx = torch.tensor(targets, device=device, dtype=torch.int64)
            self.gate_up.index_copy_(0, idx, gu)
            self.down.index_copy_(0, idx, dn)
            for e, slot in zip(missing, targets):
                self.slot_of[e] = slot
            self.loads += len(missing)
        return {e: self.slot_of[e] for e in experts}


@torch.no_grad()
def offloaded_experts_forward(block, x: torch.Tensor, w: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """The expert part of a ``SparseMoeBlock`` whose experts live in a ``LayerExperts`` pool. ``w`` / ``idx`` [T, k] are
    the routing weights and expert ids."""
    from ..ops import functional as ops
    from .moe import route_topk
    pool: LayerExperts = block.offload
    uniq = torch.unique(idx)
    nxt = getattr(block, "next_moe", None)
    guess = None
    if nxt is not None and pool.store is nxt.offload.store:
        # the next MoE layer's router on this layer's input predicts its experts; the reads run while this layer computes
        _, g = route_topk(torch.nn.functional.linear(x, nxt.router), nxt.cfg.num_experts_per_tok, nxt.cfg.norm_topk_prob)
        guess = torch.unique(g)
        both = torch.cat([uniq, guess]).tolist()               # one synchronisation for both lists
        mine, ahead = both[:uniq.numel()], both[uniq.numel():]
        pool.store.prefetch(nxt.offload.layer, ahead)
    else:
        mine = uniq.tolist()
    slot = pool.slots_for(mine, x.device, x.dtype)
    remap = torch.zeros(pool.store.num_experts, dtype=torch.int64, device=x.device)
    remap[uniq] = torch.tensor([slot[e] for e in mine], dtype=torch.int64, device=x.device)
    return ops.moe_experts(x, w, remap[idx], pool.gate_up, pool.down)


def enable_expert_offloading(model, experts_dir: str, slots: Optional[int] = None, threads: int = 8,
                             prefetch: bool = True) -> PackedExpertStore:
    """Serve the routed experts of ``model`` from a packed directory. ``slots`` experts per layer stay dequantised on the
    device (default: four times the experts per token, at least 8)."""
    from .moe import SparseMoeBlock
    store = PackedExpertStore(experts_dir, threads)
    blocks = [(i, layer.mlp) for i, layer in enumerate(model.layers) if isinstance(getattr(layer, "mlp", None), SparseMoeBlock)]
    if not blocks:
        store.close()
        raise ValueError("the model has no mixture-of-experts layers")
    cfg = model.cfg
    if (store.hidden, store.inter, store.num_experts) != (cfg.hidden_size, cfg.moe_intermediate_size, cfg.num_experts):
        store.close()
        raise ValueError(f"packed experts are {store.num_experts} x [{store.inter}, {store.hidden}], the model wants "
                         f"{cfg.num_experts} x [{cfg.moe_intermediate_size}, {cfg.hidden_size}]")
    absent = [i for i, _ in blocks if i not in store.fds]
    if absent:
        store.close()
        raise ValueError(f"no packed file for layers {absent}")
    n = slots or max(8, 4 * cfg.num_experts_per_tok)
    prev = None
    for i, blk in blocks:
        if blk.ep_group is not None or getattr(blk, "ep_engine", None) is not None:
            raise ValueError("expert offloading and expert parallelism exclude each other")
        dev, dt = blk.router.device, blk.router.dtype
        blk.gate_up = nn.Parameter(torch.empty(0, dtype=dt, device=dev), requires_grad=False)
        blk.down = nn.Parameter(torch.empty(0, dtype=dt, device=dev), requires_grad=False)
        blk.offload = LayerExperts(store, i, n)
        # plain attributes: the next block must not become a sub-module of this one
        object.__setattr__(blk, "next_moe", None)
        if prev is not None and prefetch:
            object.__setattr__(prev, "next_moe", blk)
        prev = blk
    model.expert_store = store
    return store
