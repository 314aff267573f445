"""Fused compute+collective kernels against their library-collective baselines (run under torch.distributed.run):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29650 \
        -m pmetal_b200.bench.comm [--tokens 8192] [--iters 20]

For each case it reports the device time (CUDA events, median, maximum over ranks) of the fused kernel and of the
NCCL + matmul baseline, and the fused kernel's fraction of its roofline: the slower of FLOPs at the measured GEMM peak and
the bytes that must cross NVLink at the measured per-direction copy bandwidth.
Cases: TP all-gather->GEMM (column-parallel), TP GEMM->reduce-scatter (row-parallel), EP dispatch + grouped expert GEMMs +
combine (Qwen3-30B-A3B layer shapes: hidden 2048, 128 experts, top-8, expert width 768), DP reduce+AdamW."""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

from ..parallel.linkbw import FALLBACK_GBS, measure_link_gbs

NVLINK_GBS = FALLBACK_GBS     # replaced by the ring-exchange measurement of this run in main()


def _peak_tflops() -> float:
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as fh:
            return float(json.load(fh)["bf16_tflops"])
    return 1590.0


def time_max(fn, iters: int, dev) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ts = []
    for _ in range(iters):
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    t = torch.tensor([statistics.median(ts)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def roofline_ms(flops: float, nvlink_bytes: float, peak_tflops: float) -> float:
    return max(flops / (peak_tflops * 1e12), nvlink_bytes / (NVLINK_GBS * 1e9)) * 1e3


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192, help="tokens per rank")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--hidden", type=int, default=2048)
    a = ap.parse_args(argv)
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    from ..ops import native
    from ..parallel.ep import FusedExpertMoE, expert_range
    from ..parallel.tp import ColumnParallelLinear, RowParallelLinear
    peak = _peak_tflops()
    global NVLINK_GBS
    NVLINK_GBS, link_src = measure_link_gbs(dist, dev)
    H, T = a.hidden, a.tokens
    rows = T - T % 128
    out = {"world_size": world, "tokens_per_rank": rows, "hidden": H, "peak_tflops": peak,
           "nvlink_gbs": round(NVLINK_GBS, 1), "nvlink_gbs_source": link_src}
    g = torch.Generator(device=dev).manual_seed(1 + rank)

    # ---- TP column-parallel: qkv-like projection, N_loc = 3H / world ... use 4H / world
    n_loc = max(256, (4 * H // world) // 256 * 256)
    w = (torch.randn(n_loc, H, device=dev, generator=g) * 0.02).bfloat16()
    col = ColumnParallelLinear(w, rows)
    x = torch.randn(rows, H, device=dev, generator=g).bfloat16()
    col.input_buffer.copy_(x)
    fused = time_max(lambda: col.forward(None), a.iters, dev)
    base = time_max(lambda: col.forward_nccl(x), a.iters, dev)
    flops = 2.0 * rows * world * n_loc * H
    remote = (world - 1) * rows * H * 2.0
    rf = roofline_ms(flops, remote, peak)
    out["tp_allgather_gemm"] = {"fused_ms": round(fused, 4), "nccl_ms": round(base, 4), "speedup": round(base / fused, 3),
                                "roofline_ms": round(rf, 4), "frac_of_roofline": round(rf / fused, 3)}

    # ---- TP row-parallel: o/down-like projection, K_loc = 4H / world
    k_loc = max(64, (4 * H // world) // 64 * 64)
    w2 = (torch.randn(H, k_loc, device=dev, generator=g) * 0.02).bfloat16()
    row = RowParallelLinear(w2, rows)
    x2 = torch.randn(rows * world, k_loc, device=dev, generator=g).bfloat16()
    fused = time_max(lambda: row.forward(x2), a.iters, dev)
    base = time_max(lambda: row.forward_nccl(x2), a.iters, dev)
    flops = 2.0 * rows * world * H * k_loc
    remote = (world - 1) * rows * H * 2.0
    rf = roofline_ms(flops, remote, peak)
    out["tp_gemm_reduce_scatter"] = {"fused_ms": round(fused, 4), "nccl_ms": round(base, 4), "speedup": round(base / fused, 3),
                                     "roofline_ms": round(rf, 4), "frac_of_roofline": round(rf / fused, 3)}

    # ---- EP MoE layer
    E, k, I = 128, 8, 768
    e0, e1 = expert_range(E, rank, world)
    gw = torch.Generator(device=dev).manual_seed(7)
    gate_up = (torch.randn(e1 - e0, 2 * I, H, device=dev, generator=gw) * 0.02).bfloat16()
    down = (torch.randn(e1 - e0, H, I, device=dev, generator=gw) * 0.02).bfloat16()
    te = min(rows, 4096)
    eng = FusedExpertMoE(gate_up, down, E, k, max_tokens=te, timeout_s=10.0)
    xe = torch.randn(te, H, device=dev, generator=g).bfloat16()
    logits = torch.randn(te, E, device=dev, generator=g)
    fused = time_max(lambda: eng.forward(xe, logits), a.iters, dev)
    flops = 2.0 * te * k * (3 * I * H)                    # per rank on average (uniform routing)
    remote = 2.0 * te * k * H * 2.0 * (world - 1) / world    # dispatch + combine rows that live on other ranks
    rf = roofline_ms(flops, remote, peak)
    out["ep_moe_layer"] = {"fused_ms": round(fused, 4), "roofline_ms": round(rf, 4), "frac_of_roofline": round(rf / fused, 3),
                           "tokens": te, "experts": E, "top_k": k}
    native.check_status()
    if rank == 0:
        print(json.dumps(out), flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    from pmetal_b200.parallel.dp import shutdown_process_group
    shutdown_process_group()


if __name__ == "__main__":
    raise SystemExit(main())
