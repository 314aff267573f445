"""Measured GPU-to-GPU copy bandwidth, the denominator of every "fraction of the link" figure.

Every rank copies ``mb`` MiB from its own GPU into a buffer on its right neighbour's GPU (a plain peer copy over
NVLink, the same path the fused kernels' loads and stores take) while its left neighbour does the same to it, so the
number is bytes per second per direction per GPU with all links busy. It is timed on the device with CUDA events and
the slowest rank counts. Where the neighbour's GPU is not visible to this process (several nodes, restricted device
lists) the exchange goes through NCCL point-to-point instead, which reaches less than the link gives. With one rank (or
without CUDA) there is nothing to measure and the figure this class of machine gave before is returned, marked as such."""
from __future__ import annotations

from typing import Tuple

FALLBACK_GBS = 770.0          # earlier measurement of a peer copy on an NVLink 5 / NVSwitch node


def measure_link_gbs(dist, dev, mb: int = 256, iters: int = 5) -> Tuple[float, str]:
    """(GB/s per direction per GPU, "peer copy" | "nccl p2p" | "fallback")."""
    import torch
    world = dist.get_world_size() if dist.is_initialized() else 1
    if world < 2 or dev.type != "cuda":
        return FALLBACK_GBS, "fallback"
    rank = dist.get_rank()
    n = mb * (1 << 20)
    src = torch.empty(n, dtype=torch.uint8, device=dev)
    ndev = torch.cuda.device_count()
    peer = (dev.index + 1) % ndev if ndev >= world else -1
    direct = torch.tensor([int(peer >= 0 and peer != dev.index and torch.cuda.can_device_access_peer(dev.index, peer))],
                          device=dev)
    dist.all_reduce(direct, op=dist.ReduceOp.MIN)              # all ranks take the same route
    if int(direct.item()):
        dst = torch.empty(n, dtype=torch.uint8, device=torch.device("cuda", peer))
        how = "peer copy"

        def once():
            dst.copy_(src, non_blocking=True)
    else:
        dst = torch.empty_like(src)
        right, left = (rank + 1) % world, (rank - 1) % world
        how = "nccl p2p"

        def once():
            ops = [dist.P2POp(dist.isend, src, right), dist.P2POp(dist.irecv, dst, left)]
            for w in dist.batch_isend_irecv(ops):
                w.wait()

    for _ in range(2):
        once()
    torch.cuda.synchronize(dev)
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        once()
    e1.record()
    torch.cuda.synchronize(dev)
    t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    del dst
    if ms <= 0:
        return FALLBACK_GBS, "fallback"
    return n / (ms * 1e-3) / 1e9, how
