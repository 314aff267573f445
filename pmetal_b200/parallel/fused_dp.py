"""Data-parallel step as one kernel per rank over NVLink peer memory.

``FusedDataParallel`` re-homes the optimizer's flat gradient, fp32 parameter and bf16
shadow buffers into symmetric memory (``torch.distributed._symmetric_memory``: one
allocation per rank, peer-mapped into every rank of the node). ``reduce_and_step``
then launches ``dp_reduce_adamw_kernel`` (csrc/dp_fused.cu), which reduce-scatters
the gradients with P2P loads, applies each rank's clip/accumulation/mean coefficient,
runs AdamW on the owned shard and all-gathers updated parameters with P2P stores.
NCCL is only used for bootstrap and scalar bookkeeping. The kernel is captured in
the training step's CUDA graph like any other launch.

Ordering follows the reference: each rank clips its own gradient *before* the mean
(crates/pmetal-trainer/src/training_loop/mod.rs:820-833,1004-1009). The
clip-after-reduce variant needs the norm of the averaged gradient and runs on the
NCCL baseline path.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from .dp import DistContext


def shard_range(total: int, rank: int, world: int, chunk: int = 1024) -> tuple:
    """[lo, hi) of the flat buffer that ``rank`` owns in the fused step: whole 1024-element chunks, split evenly with
    the remainder on the last ranks' side left empty (the same arithmetic as ``pm_dp_reduce_adamw``)."""
    chunks = total // chunk
    per = -(-chunks // world)
    return min(per * rank, chunks) * chunk, min(per * (rank + 1), chunks) * chunk


@torch.no_grad()
def gather_sharded_(t: torch.Tensor, lo: int, hi: int, group=None) -> torch.Tensor:
    """In place: every rank contributes ``t[lo:hi]`` (its own shard, disjoint across ranks) and ends up with the whole
    vector. Entries outside a rank's shard are ignored, whatever they hold."""
    full = torch.zeros_like(t)
    full[lo:hi] = t[lo:hi]
    dist.all_reduce(full, group=group)
    t.copy_(full)
    return t


class FusedDataParallel(DistContext):
    fused = True

    def __init__(self, group=None, timeout_s: float = 30.0, ctas: int = 64):
        super().__init__(group)
        self.timeout_s, self.ctas = timeout_s, ctas
        self._bound = None

    # ------------------------------------------------------------------ setup
    def _symm(self, numel: int, dtype) -> tuple:
        import torch.distributed._symmetric_memory as symm_mem
        t = symm_mem.empty(numel, dtype=dtype, device=torch.device("cuda", torch.cuda.current_device()))
        h = symm_mem.rendezvous(t, self.group if self.group is not None else dist.group.WORLD)
        return t, h

    def bind_optimizer(self, opt) -> None:
        """Move the optimizer's flat buffers into symmetric memory and exchange peer addresses."""
        if self.world_size == 1:
            return
        g, hg = self._symm(opt.total, torch.float32)
        p, hp = self._symm(opt.total, torch.float32)
        g.zero_()
        p.copy_(opt.flat_p)
        sh = hs = None
        if opt.flat_shadow is not None:
            sh, hs = self._symm(opt.total, opt.flat_shadow.dtype)
            sh.copy_(opt.flat_shadow)
        pad, hpad = self._symm(32, torch.int32)
        pad.zero_()
        opt.rehome(p, g, sh)
        arr = ctypes.c_ulonglong * self.world_size
        self._ptrs = {
            "g": arr(*[int(x) for x in hg.buffer_ptrs]), "p": arr(*[int(x) for x in hp.buffer_ptrs]),
            "s": arr(*[int(x) for x in hs.buffer_ptrs]) if hs is not None else None,
            "pad": arr(*[int(x) for x in hpad.buffer_ptrs]),
        }
        self._keep = (g, p, sh, pad, hg, hp, hs, hpad)
        self._pad = pad
        self._bound = opt
        torch.cuda.synchronize()
        dist.barrier(self.group)

    def gather_optimizer_state(self, opt) -> None:
        """Collective. The fused step updates the Adam moments of the owned shard only, so ``flat_m`` / ``flat_v`` of a
        rank are current on [lo, hi) and stale elsewhere; before a checkpoint every rank collects the other shards, so
        that the file rank 0 writes holds the moments of every parameter and any rank can resume from it."""
        if self.world_size == 1 or self._bound is not opt:
            return
        lo, hi = shard_range(opt.total, self.rank, self.world_size)
        gather_sharded_(opt.flat_m, lo, hi, self.group)
        gather_sharded_(opt.flat_v, lo, hi, self.group)

    def reset_flags(self) -> None:
        """Collective: clear the signal pads after a timed-out step."""
        torch.cuda.synchronize()
        dist.barrier(self.group)
        self._pad.zero_()
        torch.cuda.synchronize()
        dist.barrier(self.group)

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def reduce_and_step(self, opt, grad_scale: float, clip_after_reduce: bool = False) -> torch.Tensor:
        if clip_after_reduce or self._bound is not opt:
            return super().reduce_and_step(opt, grad_scale, clip_after_reduce)
        from ..ops import native
        opt.step_count += 1
        b1, b2 = opt.betas
        native.sumsq(opt.flat_g, opt.grad_norm)
        lib = native.lib()
        lib.pm_dp_reduce_adamw.restype = ctypes.c_int
        P = self._ptrs
        rc = lib.pm_dp_reduce_adamw(P["g"], P["p"], P["s"], P["pad"], native._p(opt.flat_m), native._p(opt.flat_v),
                                    native._p(opt.lr_mult), native._p(opt.wd_tab), native._p(opt.grad_norm),
                                    native._p(opt._hp if opt.device_hparams else None),
                                    ctypes.c_longlong(opt.total), ctypes.c_int(self.rank),
                                    ctypes.c_int(self.world_size), ctypes.c_float(opt.lr), ctypes.c_float(b1),
                                    ctypes.c_float(b2), ctypes.c_float(opt.eps), ctypes.c_int(opt.step_count),
                                    ctypes.c_float(grad_scale), ctypes.c_float(opt.max_grad_norm or 0.0),
                                    ctypes.c_double(self.timeout_s), ctypes.c_int(self.ctas),
                                    native._p(native.status_word()), native._stream())
        native._chk(rc, "pm_dp_reduce_adamw")
        return opt.grad_norm.sqrt() * grad_scale
