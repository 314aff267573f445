"""Moving tensors out of device memory while they are not needed: activations saved for the backward pass, embedding
tables, frozen parameters; and the per-layer decision between keeping, recomputing and offloading activations
(crates/pmetal-mlx/src/offloading.rs: ``OffloadConfig`` / ``ActivationOffloader`` / ``OffloadedEmbedding`` /
``FrozenParameterManager``; crates/pmetal-mlx/src/smart_checkpoint.rs: ``CheckpointPolicy`` / ``LayerType`` /
``SmartCheckpointConfig``).

On a B200 the host side is pinned memory reached over PCIe / NVLink-C2C rather than the other half of a unified memory, so
the offloader is built around asynchronous copies: tensors that autograd saves inside an ``ActivationOffloader`` context
leave on a side stream into pinned buffers (recycled from step to step) and come back when the backward pass asks for
them; the compute stream only waits for the copy of the tensor it needs. Disk offload writes the same bytes to files."""
from __future__ import annotations

import os
import uuid
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

GPU, CPU, DISK = "gpu", "cpu", "disk"


@dataclass
class OffloadConfig:
    embedding_target: str = CPU
    activation_target: str = CPU
    offload_dir: Optional[str] = None
    size_threshold: int = 1 << 20            # tensors below this many bytes stay where they are
    async_offload: bool = True
    prefetch_embeddings: bool = True
    memory_threshold: float = 0.85           # offload only while more than this fraction of device memory is in use

    @classmethod
    def aggressive(cls) -> "OffloadConfig":
        return cls(DISK, DISK, "_pmetal_offload", 512 << 10, True, True, 0.70)

    @classmethod
    def moderate(cls) -> "OffloadConfig":
        return cls(CPU, GPU, None, 2 << 20, True, False, 0.90)

    def with_offload_dir(self, d: str) -> "OffloadConfig":
        self.offload_dir = d
        return self

    def with_memory_threshold(self, t: float) -> "OffloadConfig":
        self.memory_threshold = min(max(float(t), 0.0), 1.0)
        return self


@dataclass
class OffloadStats:
    bytes_to_cpu: int = 0
    bytes_to_disk: int = 0
    loads: int = 0
    saves: int = 0
    skipped: int = 0

    @property
    def device_bytes_saved(self) -> int:
        return self.bytes_to_cpu + self.bytes_to_disk


class _Handle:
    __slots__ = ("kind", "host", "event", "path", "shape", "dtype", "device", "strides")


class ActivationOffloader:
    """Context manager: tensors that autograd saves for backward inside it are moved to pinned host memory (or disk) and
    brought back on demand. Parameters and tensors under the size threshold are left alone. With ``memory_threshold`` the
    offload only happens while the device is fuller than that fraction (always, for tensors that are not on a GPU)."""

    def __init__(self, config: Optional[OffloadConfig] = None, always: bool = False):
        self.cfg = config or OffloadConfig()
        self.always = always
        self.stats = OffloadStats()
        self._pool: Dict[tuple, List[torch.Tensor]] = {}
        self._stream: Optional[torch.cuda.Stream] = None
        self._hooks = None
        if self.cfg.activation_target == DISK:
            self.dir = os.path.join(self.cfg.offload_dir or "_pmetal_offload", uuid.uuid4().hex[:8])
            os.makedirs(self.dir, exist_ok=True)

    # ------------------------------------------------------------------ policy
    def _wanted(self, t: torch.Tensor) -> bool:
        if self.cfg.activation_target == GPU or not t.is_floating_point():
            return False
        base = t._base if t._base is not None else t
        if isinstance(base, torch.nn.Parameter) or (base.is_leaf and base.requires_grad):      # weights (and views of
            return False                                                                        # them) stay put
        if t.numel() * t.element_size() < self.cfg.size_threshold:
            return False
        if getattr(t, "_pmetal_keep", False):
            return False
        if t.is_cuda and not self.always:
            free, total = torch.cuda.mem_get_info(t.device)
            return (total - free) / total >= self.cfg.memory_threshold
        return True

    def _host_buffer(self, t: torch.Tensor) -> torch.Tensor:
        key = (tuple(t.shape), t.dtype)
        bucket = self._pool.get(key)
        if bucket:
            return bucket.pop()
        return torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=t.is_cuda)

    # ------------------------------------------------------------------ hooks
    def _pack(self, t: torch.Tensor):
        if not self._wanted(t):
            self.stats.skipped += 1
            return t
        h = _Handle()
        h.shape, h.dtype, h.device, h.strides = t.shape, t.dtype, t.device, None
        nbytes = t.numel() * t.element_size()
        self.stats.saves += 1
        if self.cfg.activation_target == DISK:
            h.kind, h.path = DISK, os.path.join(self.dir, f"{self.stats.saves}.bin")
            t.detach().contiguous().cpu().view(torch.uint8).numpy().tofile(h.path)
            self.stats.bytes_to_disk += nbytes
            return h
        h.kind = CPU
        h.host = self._host_buffer(t)
        h.event = None
        if t.is_cuda and self.cfg.async_offload:
            if self._stream is None:
                self._stream = torch.cuda.Stream(t.device)
            self._stream.wait_stream(torch.cuda.current_stream(t.device))
            with torch.cuda.stream(self._stream):
                h.host.copy_(t.detach(), non_blocking=True)
                h.event = torch.cuda.Event()
                h.event.record(self._stream)
            t.record_stream(self._stream)          # the device block is not reused before the copy has read it
        else:
            h.host.copy_(t.detach())
        self.stats.bytes_to_cpu += nbytes
        return h

    def _unpack(self, obj):
        if not isinstance(obj, _Handle):
            return obj
        self.stats.loads += 1
        if obj.kind == DISK:
            import numpy as np
            raw = torch.from_numpy(np.fromfile(obj.path, dtype=np.uint8))
            out = raw.view(obj.dtype).reshape(obj.shape).to(obj.device)
            try:
                os.remove(obj.path)
            except OSError:
                pass
            return out
        if obj.event is not None:
            torch.cuda.current_stream(obj.device).wait_event(obj.event)
        out = obj.host.to(obj.device, non_blocking=True)
        # the pinned buffer can go back to the pool: the next copy into it is queued on the side stream, which first
        # waits for the compute stream, where this copy back has just been queued
        self._pool.setdefault((tuple(obj.shape), obj.dtype), []).append(obj.host)
        return out

    def __enter__(self):
        self._hooks = torch.autograd.graph.saved_tensors_hooks(self._pack, self._unpack)
        self._hooks.__enter__()
        return self

    def __exit__(self, *exc):
        self._hooks.__exit__(*exc)
        self._hooks = None
        return False

    def clear(self) -> None:
        self._pool.clear()
        d = getattr(self, "dir", None)
        if d and os.path.isdir(d):
            for f in os.listdir(d):
                try:
                    os.remove(os.path.join(d, f))
                except OSError:
                    pass

    def reset_stats(self) -> None:
        self.stats = OffloadStats()


class OffloadedEmbedding:
    """An embedding table kept on the host (pinned) or on disk (memory-mapped); a lookup gathers the requested rows
    there and ships only those to the device. ``get_weights`` materialises (and caches) the whole table on the device."""

    def __init__(self, weight: torch.Tensor, target: str = CPU, device=None, offload_dir: Optional[str] = None):
        self.num, self.dim, self.dtype = weight.shape[0], weight.shape[1], weight.dtype
        self.device = torch.device(device) if device is not None else weight.device
        self.target = target
        self._gpu: Optional[torch.Tensor] = None
        self._cpu: Optional[torch.Tensor] = None
        self._path: Optional[str] = None
        if target == GPU:
            self._gpu = weight.detach().to(self.device)
        elif target == CPU:
            self._cpu = weight.detach().to("cpu").contiguous()
            if self.device.type == "cuda":
                self._cpu = self._cpu.pin_memory()
        else:
            d = offload_dir or "_pmetal_offload"
            os.makedirs(d, exist_ok=True)
            self._path = os.path.join(d, f"embedding_{uuid.uuid4().hex[:8]}.bin")
            weight.detach().to("cpu").contiguous().view(torch.uint8).numpy().tofile(self._path)

    def _host_table(self) -> torch.Tensor:
        if self._cpu is not None:
            return self._cpu
        import numpy as np
        mm = np.memmap(self._path, dtype=np.uint8, mode="c")        # copy-on-write: readable as a tensor, file untouched
        return torch.from_numpy(mm).view(self.dtype).reshape(self.num, self.dim)

    def get_weights(self) -> torch.Tensor:
        if self._gpu is None:
            self._gpu = self._host_table().to(self.device)
        return self._gpu

    def lookup(self, indices: torch.Tensor) -> torch.Tensor:
        if self._gpu is not None:
            return self._gpu[indices.to(self._gpu.device)]
        idx = indices.reshape(-1).to("cpu")
        uniq, inv = torch.unique(idx, return_inverse=True)
        rows = self._host_table()[uniq].to(self.device, non_blocking=True)
        return rows[inv.to(self.device)].reshape(*indices.shape, self.dim)

    def evict_gpu_cache(self) -> None:
        if self.target != GPU:
            self._gpu = None

    def memory_usage(self) -> Dict[str, int]:
        nbytes = self.num * self.dim * torch.empty((), dtype=self.dtype).element_size()
        return {"gpu": nbytes if self._gpu is not None else 0, "cpu": nbytes if self._cpu is not None else 0,
                "disk": nbytes if self._path is not None else 0}


class FrozenParameterManager:
    """Frozen weights live on the host; ``get`` brings one to the device and keeps the most recently used ones there up
    to ``gpu_budget_bytes`` (least recently used are dropped first)."""

    def __init__(self, device, gpu_budget_bytes: int):
        self.device = torch.device(device)
        self.budget = int(gpu_budget_bytes)
        self.host: Dict[str, torch.Tensor] = {}
        self.resident: "OrderedDict[str, torch.Tensor]" = OrderedDict()
        self.hits = self.misses = self.evictions = 0

    def register_frozen_params(self, named) -> int:
        n = 0
        for name, p in named:
            if getattr(p, "requires_grad", False):
                continue
            h = p.detach().to("cpu").contiguous()
            self.host[name] = h.pin_memory() if self.device.type == "cuda" else h
            n += 1
        return n

    def gpu_memory_usage(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.resident.values())

    def get(self, name: str) -> torch.Tensor:
        t = self.resident.get(name)
        if t is not None:
            self.resident.move_to_end(name)
            self.hits += 1
            return t
        self.misses += 1
        h = self.host[name]
        need = h.numel() * h.element_size()
        while self.resident and self.gpu_memory_usage() + need > self.budget:
            self.resident.popitem(last=False)
            self.evictions += 1
        t = h.to(self.device, non_blocking=True)
        self.resident[name] = t
        return t

    def evict(self, name: str) -> None:
        if self.resident.pop(name, None) is not None:
            self.evictions += 1

    def evict_all(self) -> None:
        self.evictions += len(self.resident)
        self.resident.clear()

    def memory_savings_percent(self) -> float:
        total = sum(t.numel() * t.element_size() for t in self.host.values())
        return 100.0 * (1.0 - self.gpu_memory_usage() / total) if total else 0.0


# ------------------------------------------------------------------------------------------- smart checkpointing
ALWAYS_SAVE, ALWAYS_RECOMPUTE, SMART, OFFLOAD_CPU, OFFLOAD_DISK = "save", "recompute", "smart", "offload_cpu", "offload_disk"

# (recompute cost relative to a standard layer, memory factor in units of hidden^2) per layer type
LAYER_COSTS = {"attention": (3.0, 4.0), "moe_expert": (2.5, 2.0), "mlp": (1.5, 2.0), "moe_router": (0.5, 0.1),
               "norm": (0.2, 0.1), "embedding": (0.1, 1.0), "output": (0.1, 1.0), "unknown": (1.0, 1.0)}


@dataclass
class SmartCheckpointConfig:
    enabled: bool = True
    target_memory_fraction: float = 0.8
    layer_policies: Dict[str, str] = field(default_factory=lambda: {
        "attention": SMART, "mlp": ALWAYS_RECOMPUTE, "norm": ALWAYS_RECOMPUTE, "embedding": ALWAYS_SAVE,
        "output": ALWAYS_SAVE, "moe_router": ALWAYS_RECOMPUTE, "moe_expert": SMART})
    min_layers_per_block: int = 1
    max_layers_per_block: int = 4
    allow_cpu_offload: bool = False
    allow_disk_offload: bool = False
    offload_path: Optional[str] = None
    recompute_cost_threshold: float = 2.0

    @classmethod
    def aggressive(cls) -> "SmartCheckpointConfig":
        return cls(target_memory_fraction=0.5, recompute_cost_threshold=5.0)

    @classmethod
    def balanced(cls) -> "SmartCheckpointConfig":
        return cls()

    @classmethod
    def minimal(cls) -> "SmartCheckpointConfig":
        return cls(target_memory_fraction=0.95, recompute_cost_threshold=1.0)

    def with_layer_policy(self, layer_type: str, policy: str) -> "SmartCheckpointConfig":
        self.layer_policies[layer_type] = policy
        return self

    def with_cpu_offload(self) -> "SmartCheckpointConfig":
        self.allow_cpu_offload = True
        return self

    def with_disk_offload(self, path: str) -> "SmartCheckpointConfig":
        self.allow_disk_offload, self.offload_path = True, path
        return self

    def get_policy(self, layer_type: str) -> str:
        return self.layer_policies.get(layer_type, SMART)

    def resolve(self, layer_type: str, memory_pressure: float) -> str:
        """What to do with the activations of a layer of this type when ``memory_pressure`` (fraction of device memory
        in use) is known: a SMART layer is saved while there is room; under pressure it is recomputed when that is
        cheap enough, else offloaded where offloading is allowed, else recomputed."""
        pol = self.get_policy(layer_type)
        if not self.enabled:
            return ALWAYS_SAVE
        if pol != SMART:
            return pol
        if memory_pressure < self.target_memory_fraction:
            return ALWAYS_SAVE
        cost = LAYER_COSTS.get(layer_type, LAYER_COSTS["unknown"])[0]
        if cost <= self.recompute_cost_threshold:
            return ALWAYS_RECOMPUTE
        if self.allow_cpu_offload:
            return OFFLOAD_CPU
        if self.allow_disk_offload:
            return OFFLOAD_DISK
        return ALWAYS_RECOMPUTE


def transformer_layer_types(num_layers: int, has_moe: bool) -> List[str]:
    """Sequence of layer types of a decoder: embedding, per block (norm, attention, norm, mlp or router + experts),
    final norm, output."""
    out = ["embedding"]
    for _ in range(num_layers):
        out += ["norm", "attention", "norm"] + (["moe_router", "moe_expert"] if has_moe else ["mlp"])
    return out + ["norm", "output"]


def plan_decoder_layers(cfg: SmartCheckpointConfig, num_layers: int, has_moe: bool, memory_pressure: float) -> List[str]:
    """One decision per decoder block ("save", "recompute", "offload_cpu", "offload_disk"): a block is as expensive to
    recompute as its attention half, so the attention policy decides; blocks are grouped so that at most
    ``max_layers_per_block`` consecutive blocks are recomputed from one saved input."""
    att = cfg.resolve("attention", memory_pressure)
    mlp = cfg.resolve("moe_expert" if has_moe else "mlp", memory_pressure)
    if att == ALWAYS_SAVE and memory_pressure < cfg.target_memory_fraction:
        return [ALWAYS_SAVE] * num_layers
    block = att if att != ALWAYS_SAVE else mlp
    return [block] * num_layers


def apply_to_model(model, plan: List[str], offload_cfg: Optional[OffloadConfig] = None) -> Optional[ActivationOffloader]:
    """Install a per-block plan on a ``DecoderLM``: ``model.layer_policies`` is read by ``forward_hidden`` (recompute
    through activation checkpointing, offload through the returned offloader)."""
    off = None
    if any(p in (OFFLOAD_CPU, OFFLOAD_DISK) for p in plan):
        oc = offload_cfg or OffloadConfig()
        oc.activation_target = DISK if OFFLOAD_DISK in plan else CPU
        off = ActivationOffloader(oc, always=True)
    model.layer_policies = list(plan)
    model.activation_offloader = off
    return off
