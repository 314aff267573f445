"""Gradient all-reduce overlapped with backward for full-parameter data parallelism.

The flat fp32 gradient buffer of ``FlatAdamW`` is laid out in parameter order (embedding, layer 0 .. L-1, final norm,
head) while backward finishes the layers in the opposite order. The decoder calls ``grad_ready_hook(i)`` when the
gradient with respect to the input of layer ``i`` exists, i.e. when every parameter of layers >= i (and of the norm and
the head) has its final gradient. Layers are grouped into buckets of at least ``bucket_mb``; a bucket's slice of the
flat buffer is all-reduced on a side stream the moment its lowest layer reports, optionally as bf16 (half the bytes
over NVLink, converted on the way in and out), while the tensor cores keep working on the layers below. ``finish``
reduces what is left (the embedding), waits for everything and returns. Clipping then uses the norm of the averaged
gradient (the overlapped order cannot clip each rank's gradient before it is summed).

Role in the reference: crates/pmetal-trainer/src/distributed_bridge.rs:36-323 (gradient synchronisation) with the
bucketing of crates/pmetal-distributed/src/gradient_buckets.rs.
"""
from __future__ import annotations

import re
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

_LAYER = re.compile(r"(?:^|\.)layers\.(\d+)\.")


class OverlappedGradReducer:
    def __init__(self, opt, model, group=None, bucket_mb: float = 32.0, reduce_dtype: Optional[torch.dtype] = None):
        self.opt, self.group, self.reduce_dtype = opt, group, reduce_dtype
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        n_layers = len(model.layers)
        lo = [None] * n_layers
        hi = [None] * n_layers
        for (name, p), o in zip(opt.named, opt.offsets):
            m = _LAYER.search(name)
            if m:
                i = int(m.group(1))
                lo[i] = o if lo[i] is None else min(lo[i], o)
                hi[i] = max(hi[i] or 0, o + p.numel())
        trained = [i for i in range(n_layers) if lo[i] is not None]
        # buckets from the top of the network down; the first one also takes everything stored after the last layer
        self.buckets: List[Tuple[int, int, int]] = []           # (lowest layer, start, end) in flat elements
        end = opt.total
        min_elems = int(bucket_mb * (1 << 20) / 4)
        start_layer = None
        for i in reversed(trained):
            start_layer = i
            if end - lo[i] >= min_elems:
                self.buckets.append((i, lo[i], end))
                end = lo[i]
                start_layer = None
        if start_layer is not None:
            self.buckets.append((start_layer, lo[start_layer], end))
            end = lo[start_layer]
        self.rest = (0, end)                                    # embedding and whatever precedes layer 0
        self.cuda = opt.flat_g.is_cuda
        self.stream = torch.cuda.Stream(device=opt.flat_g.device) if self.cuda else None
        self.armed = False
        self._next = 0
        self._pending: list = []
        self.launched_early = 0                                 # buckets sent before backward ended (for tests / logs)
        model.grad_ready_hook = self._on_ready

    # ------------------------------------------------------------------ protocol of one optimiser step
    def arm(self) -> None:
        """Call before the backward pass whose gradients are final (the last micro-batch of an accumulation)."""
        self.armed, self._next, self._pending, self.launched_early = True, 0, [], 0

    def _on_ready(self, layer: int) -> None:
        if not self.armed or self.world == 1:
            return
        while self._next < len(self.buckets) and self.buckets[self._next][0] >= layer:
            _, a, b = self.buckets[self._next]
            self._launch(a, b)
            self._next += 1
            self.launched_early += 1

    def _launch(self, a: int, b: int) -> None:
        if b <= a:
            return
        view = self.opt.flat_g[a:b]
        if self.cuda:
            self.stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.stream):
                buf = view.to(self.reduce_dtype) if self.reduce_dtype is not None else view
                work = dist.all_reduce(buf, group=self.group, async_op=True)
        else:
            buf = view.to(self.reduce_dtype) if self.reduce_dtype is not None else view
            work = dist.all_reduce(buf, group=self.group, async_op=True)
        self._pending.append((work, buf, view))

    @torch.no_grad()
    def finish(self) -> None:
        """Send the remaining slices, wait for all of them; ``flat_g`` then holds the sum over ranks."""
        if self.world == 1:
            self.armed = False
            return
        while self._next < len(self.buckets):                   # hooks that never fired (e.g. frozen lower layers)
            _, a, b = self.buckets[self._next]
            self._launch(a, b)
            self._next += 1
        self._launch(*self.rest)
        for work, buf, view in self._pending:
            if self.cuda:
                with torch.cuda.stream(self.stream):
                    work.wait()
                    if buf is not view:
                        view.copy_(buf)
            else:
                work.wait()
                if buf is not view:
                    view.copy_(buf)
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.stream)
        self._pending = []
        self.armed = False

    @torch.no_grad()
    def finish_and_step(self, grad_scale: float = 1.0) -> torch.Tensor:
        from .dp import step_on_summed_gradient
        self.finish()
        return step_on_summed_gradient(self.opt, grad_scale, self.world, self.group)
