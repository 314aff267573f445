"""``pmetal cluster`` runtime for one NVSwitch node (crates/pmetal-distributed/src/cluster_runtime.rs:20-280,
crates/pmetal/src/commands/cluster.rs:24-390).

* ``status``          device / P2P / NVLink table (replaces peer discovery: the node's GPUs are the cluster).
* ``bench``           all-reduce of ``--mb`` MiB for ``--iters`` iterations on N GPUs: NCCL vs the fused peer-memory
                      reduce kernel, reporting algorithm and bus bandwidth (bus = 2 (N-1)/N x algorithm, the reference's
                      per-link normalisation) and the fraction of the measured NVLink copy bandwidth.
* ``pipeline-bench``  activation send/recv ring over NCCL p2p with the pipeline wire message sizes.
* ``train`` / ``serve``  launch the corresponding command under ``torch.distributed.run`` on N GPUs.
Workers are spawned as one process per GPU with 127.0.0.1 rendezvous."""
from __future__ import annotations

import json
import os
import subprocess
import sys



def _torchrun(n: int, module_args, port: int = 29611) -> int:
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(port)] + module_args
    try:
        return subprocess.call(cmd)
    except KeyboardInterrupt:                  # the interrupt reached the workers as well; they wind down by themselves
        return 130


def _snapshot(a, n: int) -> dict:
    """The status document: devices, ring order, link classes and the ports in use."""
    import torch

    from ..utils.sysinfo import system_info
    from . import discovery
    info = system_info()
    probe = torch.cuda.is_available() and not getattr(a, "no_discovery", False)
    fabric = discovery.probe_fabric(n) if probe else []
    peers = discovery.discover_local(num_devices=n)
    info["cluster"] = {"world_size": n, "topology": "nvswitch-all-to-all" if n > 1 else "single",
                       "ring_order": [p.device for p in discovery.ring_order(peers)],
                       "links": [[link.name for link in row] for row in fabric],
                       "ring_bandwidth_gbs": discovery.ring_bandwidth(fabric, list(range(n))) if fabric else 0.0,
                       "ports": {"gradients": getattr(a, "gradient_port", 0) or discovery.GRADIENT_PORT,
                                 "discovery": getattr(a, "discovery_port", 0) or discovery.DISCOVERY_PORT,
                                 "activations": getattr(a, "activation_port", 0) or discovery.GRADIENT_PORT + 1,
                                 "results": getattr(a, "result_port", 0) or discovery.GRADIENT_PORT + 2}}
    return info


def run(a) -> int:
    import torch
    n = a.gpus or (torch.cuda.device_count() if torch.cuda.is_available() else 0)
    need = int(getattr(a, "min_peers", 0) or 0) + 1
    if getattr(a, "min_peers", 0) and n < need:
        print(f"error: {need} GPUs wanted (--min-peers {need - 1}), {n} present", file=sys.stderr)
        return 1
    if a.action in ("status", "up"):
        import time
        deadline = time.monotonic() + (float(getattr(a, "wait", 0) or 0) if a.action == "up" else 0.0)
        while True:
            print(json.dumps(_snapshot(a, n), indent=None if getattr(a, "json", False) else 2), flush=True)
            left = deadline - time.monotonic()
            if left <= 0:
                return 0
            time.sleep(min(max(float(getattr(a, "status_interval", 10) or 10), 0.05), left))
    if n < 1:
        print("error: no CUDA devices", file=sys.stderr)
        return 1
    here = os.path.abspath(__file__)
    if a.action == "bench":
        return _torchrun(n, [here, "bench", str(a.mb), str(a.iters)], getattr(a, "gradient_port", 0) or 29611)
    if a.action == "pipeline-bench":
        return _torchrun(n, [here, "pipeline", str(a.mb), str(a.iters), str(getattr(a, "hidden_dim", 0) or 0),
                             str(getattr(a, "tokens", 0) or 0), str(getattr(a, "timeout", 0) or 0)],
                        getattr(a, "activation_port", 0) or 29611)
    if a.action in ("train", "serve"):
        rest = [x for x in a.rest if x != "--"]
        return _torchrun(n, ["-m", "pmetal_b200.cli.main", a.action] + rest)
    return 2


# ------------------------------------------------------------------------------------------- workers
def _worker_setup(timeout_s: float = 0.0):
    import datetime

    import torch
    import torch.distributed as dist
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    kw = {"timeout": datetime.timedelta(seconds=timeout_s)} if timeout_s > 0 else {}
    dist.init_process_group("nccl", device_id=dev, **kw)
    return dist, dev, dist.get_rank(), dist.get_world_size()


def _time_max(dist, dev, fn, iters: int) -> float:
    """Median device time of ``fn`` in ms, maximum over ranks."""
    import statistics

    import torch
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    t = torch.tensor([statistics.median(ts)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _bench_worker(mb: int, iters: int) -> None:
    import torch
    dist, dev, rank, world = _worker_setup()
    n = mb * 1024 * 1024 // 4
    n -= n % (1024 * world)
    x = torch.randn(n, device=dev)
    out = {"world_size": world, "mb": mb, "iters": iters}
    ms = _time_max(dist, dev, lambda: dist.all_reduce(x), iters)
    alg = n * 4 / (ms * 1e-3) / 1e9
    out["nccl"] = {"ms": round(ms, 4), "algbw_gbs": round(alg, 1), "busbw_gbs": round(alg * 2 * (world - 1) / world, 1)}
    try:
        from ..ops import native
        from .fused_dp import FusedDataParallel
        from ..trainer.optimizer import FlatAdamW
        p = torch.nn.Parameter(torch.zeros(n, device=dev))
        opt = FlatAdamW([("bench.weight", p)], lr=1e-4, weight_decay=0.0, max_grad_norm=1.0)
        ctx = FusedDataParallel(timeout_s=10.0)
        ctx.bind_optimizer(opt)
        opt.flat_g.normal_()
        ms2 = _time_max(dist, dev, lambda: ctx.reduce_and_step(opt, 1.0), iters)
        native.check_status()
        alg2 = n * 4 / (ms2 * 1e-3) / 1e9
        out["fused_reduce_adamw"] = {"ms": round(ms2, 4), "algbw_gbs": round(alg2, 1),
                                     "busbw_gbs": round(alg2 * 2 * (world - 1) / world, 1),
                                     "note": "reduce-scatter + clip + AdamW + all-gather in one kernel"}
    except Exception as e:          # the collective bench must still report the library number
        out["fused_reduce_adamw"] = {"error": f"{type(e).__name__}: {e}"}
    from .linkbw import measure_link_gbs
    link, src = measure_link_gbs(dist, dev)
    out["link_gbs_per_direction"] = {"value": round(link, 1), "source": src}
    for k in ("nccl", "fused_reduce_adamw"):
        if "busbw_gbs" in out[k]:
            out[k]["frac_of_nvlink_copy"] = round(out[k]["busbw_gbs"] / link, 3)
    if rank == 0:
        print(json.dumps(out), flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    from pmetal_b200.parallel.dp import shutdown_process_group
    shutdown_process_group()


def _pipeline_worker(mb: int, iters: int, hidden: int = 0, tokens: int = 0, timeout_s: float = 0.0) -> None:
    """Activation message [1, tokens, hidden] bf16 around the stage ring; ``tokens`` defaults to what ``mb`` MiB hold."""
    import torch
    dist, dev, rank, world = _worker_setup(timeout_s)
    from .pipeline import ActivationMessage, pipeline_ring_step
    hidden = hidden or 4096
    tokens = tokens or max(mb * 1024 * 1024 // (hidden * 2), 1)
    x = torch.randn(1, tokens, hidden, device=dev).bfloat16()
    msg = ActivationMessage(nonce=1, layer_id=rank, tensor=x)
    ms = _time_max(dist, dev, lambda: pipeline_ring_step(msg, rank, world), iters) if world > 1 else 0.0
    from .linkbw import measure_link_gbs
    link, src = measure_link_gbs(dist, dev)
    if rank == 0:
        gbs = x.numel() * 2 / (ms * 1e-3) / 1e9 if ms > 0 else 0.0
        print(json.dumps({"world_size": world, "message_mb": round(x.numel() * 2 / 2 ** 20, 2), "ms": round(ms, 4),
                          "gbs_per_hop": round(gbs, 1), "link_gbs_per_direction": round(link, 1), "link_source": src,
                          "frac_of_nvlink_copy": round(gbs / link, 3)}), flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    from pmetal_b200.parallel.dp import shutdown_process_group
    shutdown_process_group()


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    __package__ = "pmetal_b200.parallel"
    kind, mb, iters = sys.argv[1], int(sys.argv[2]), int(sys.argv[3])
    if kind == "bench":
        _bench_worker(mb, iters)
    else:
        extra = [float(x) for x in sys.argv[4:7]] + [0.0] * 3
        _pipeline_worker(mb, iters, int(extra[0]), int(extra[1]), extra[2])
