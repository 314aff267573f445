"""Data-parallel gradient synchronisation.

The reference syncs once per optimizer step: clip locally, flatten every gradient
(sorted by name) into one f32 buffer, all-reduce with Mean over its TCP ring, scatter
back, then run the optimizer (crates/pmetal-trainer/src/distributed_bridge.rs:164-221).
Here gradients already live in one flat buffer, so the baseline is a single NCCL
all-reduce of that buffer; ``parallel.fused_dp`` replaces reduce + scale + clip +
AdamW + parameter all-gather with one kernel over NVLink peer memory.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist


def shutdown_process_group(timeout_s: float = 30.0) -> None:
    """Orderly end of a multi-rank job: barrier, drain the device, drop unreachable objects (captured CUDA graphs keep
    the streams, and on the NCCL path the communicator's work, they were recorded on; symmetric-memory handles keep
    peer mappings), then destroy the process group. The caller should already have released its graphs and models.
    A watchdog thread ends the process if the communicator has not shut down after ``timeout_s`` seconds, so that a
    stuck teardown cannot hold the node's GPUs."""
    import gc
    import threading
    if not dist.is_initialized():
        return
    try:
        dist.barrier()
    except Exception:
        pass
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    watchdog = threading.Timer(timeout_s, lambda: os._exit(0))
    watchdog.daemon = True
    watchdog.start()
    try:
        dist.destroy_process_group()
    finally:
        watchdog.cancel()


@torch.no_grad()
def step_on_summed_gradient(opt, grad_scale: float, world: int, group=None) -> torch.Tensor:
    """Optimiser step on a gradient buffer that holds the sum over ``world`` ranks, clipping by the norm of the mean.

    Every rank holds the same numbers, but the norm is a parallel sum whose order (and last bit) can differ from rank to
    rank; replicas that clip with their own value drift apart by an ulp per step. The largest norm is agreed on first,
    so that all ranks scale by the same coefficient."""
    if not opt.max_grad_norm:
        return opt.step(grad_scale / world)
    norm = opt.compute_grad_norm().reshape(1) * (grad_scale / world)
    if world > 1:
        dist.all_reduce(norm, op=dist.ReduceOp.MAX, group=group)
    coef = torch.clamp(opt.max_grad_norm / (norm + 1e-6), max=1.0) * (grad_scale / world)
    opt.flat_g.mul_(coef)
    saved, opt.max_grad_norm = opt.max_grad_norm, 0.0
    try:
        opt.step(1.0)
    finally:
        opt.max_grad_norm = saved
    return norm


class DistContext:
    """Rank bookkeeping + the collectives the training loop needs."""

    fused = False

    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world_size = dist.get_world_size(group) if dist.is_initialized() else 1

    @classmethod
    def from_env(cls, backend: Optional[str] = None) -> "DistContext":
        """torchrun-style environment (RANK/WORLD_SIZE/LOCAL_RANK/MASTER_*); PMETAL_RANK is accepted as an
        alias of RANK as in the reference (distributed_bridge.rs:304-307)."""
        if "RANK" not in os.environ and "PMETAL_RANK" in os.environ:
            os.environ["RANK"] = os.environ["PMETAL_RANK"]
        if int(os.environ.get("WORLD_SIZE", "1")) > 1 and not dist.is_initialized():
            use_cuda = torch.cuda.is_available()
            if use_cuda:
                torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
            dist.init_process_group(backend or ("nccl" if use_cuda else "gloo"))
        return cls()

    def barrier(self) -> None:
        if self.world_size > 1:
            dist.barrier(self.group)

    def mean_scalar(self, x: float) -> float:
        if self.world_size == 1:
            return x
        dev = "cuda" if dist.get_backend(self.group) == "nccl" else "cpu"
        t = torch.tensor([x], dtype=torch.float64 if dev == "cpu" else torch.float32, device=dev)
        dist.all_reduce(t, group=self.group)
        return float(t.item()) / self.world_size

    def max_scalar(self, x: float) -> float:
        if self.world_size == 1:
            return x
        dev = "cuda" if dist.get_backend(self.group) == "nccl" else "cpu"
        t = torch.tensor([x], dtype=torch.float32, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return float(t.item())

    def broadcast_object(self, obj, src: int = 0):
        """``obj`` of rank ``src`` on every rank (a small picklable value: a path, a step number)."""
        if self.world_size == 1:
            return obj
        box = [obj if self.rank == src else None]
        dist.broadcast_object_list(box, src=src, group=self.group)
        return box[0]

    def bind_optimizer(self, opt) -> None:
        pass

    def gather_optimizer_state(self, opt) -> None:
        """Collective hook called by every rank before rank 0 writes ``optimizer.pt``. The all-reduce path keeps
        identical full moments on every rank, so there is nothing to collect."""
        return None

    @torch.no_grad()
    def reduce_and_step(self, opt, grad_scale: float, clip_after_reduce: bool = False) -> torch.Tensor:
        """Baseline path: local clip (reference order) → all-reduce mean → AdamW."""
        n = self.world_size
        if clip_after_reduce or not opt.max_grad_norm:
            dist.all_reduce(opt.flat_g, group=self.group)
            return step_on_summed_gradient(opt, grad_scale, n, self.group)
        # clip-before-reduce: scale the local gradient by its own clip coefficient, then average
        norm = opt.compute_grad_norm() * grad_scale
        coef = torch.clamp(opt.max_grad_norm / (norm + 1e-6), max=1.0) * grad_scale / n
        opt.flat_g.mul_(coef)
        dist.all_reduce(opt.flat_g, group=self.group)
        saved, opt.max_grad_norm = opt.max_grad_norm, 0.0
        try:
            opt.step(1.0)
        finally:
            opt.max_grad_norm = saved
        return norm.reshape(1)
