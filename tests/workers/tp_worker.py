"""Worker for the multi-GPU tensor-parallel test: fused all-gather->GEMM and GEMM->reduce-scatter kernels against an
fp32 reference built from NCCL-gathered operands. Several calls in a row exercise the epoch flags and the
double-buffered staging."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from pmetal_b200.ops import native
    from pmetal_b200.parallel.tp import ColumnParallelLinear, RowParallelLinear
    rows, K, n_loc = 256, 520, 392          # K and N are deliberately not tile multiples
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    w_col = (torch.randn(n_loc, K, device=dev, generator=g) * 0.05).bfloat16()
    col = ColumnParallelLinear(w_col, rows, timeout_s=5.0)
    N, k_loc = 648, 264
    w_row = (torch.randn(N, k_loc, device=dev, generator=g) * 0.05).bfloat16()
    row = RowParallelLinear(w_row, rows, timeout_s=5.0)
    for it in range(4):
        x_loc = torch.randn(rows, K, device=dev, generator=g).bfloat16()
        y = col.forward(x_loc)
        full = torch.empty(rows * world, K, dtype=torch.bfloat16, device=dev)
        dist.all_gather_into_tensor(full, x_loc)
        ref = full.float() @ w_col.float().t()
        err = (y.float() - ref).abs().max().item()
        assert err < 0.02 * ref.abs().max().item() + 1e-3, f"column-parallel iter {it}: err {err}"
        yb = col.forward_nccl(x_loc)
        assert (yb.float() - ref).abs().max().item() < 0.02 * ref.abs().max().item() + 1e-3

        xr = torch.randn(rows * world, k_loc, device=dev, generator=g).bfloat16()
        out = row.forward(xr)
        part = xr.float() @ w_row.float().t()
        dist.all_reduce(part)
        ref2 = part[rank * rows:(rank + 1) * rows]
        err2 = (out.float() - ref2).abs().max().item()
        assert err2 < 0.03 * ref2.abs().max().item() + 1e-3, f"row-parallel iter {it}: err {err2}"
        torch.cuda.synchronize()
        native.check_status()
    if rank == 0:
        print(f"tp fused ok: col err {err:.3e} row err {err2:.3e}", flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        print("TP_WORKER_OK", flush=True)
    sys.stdout.flush()
    from pmetal_b200.parallel.dp import shutdown_process_group
    shutdown_process_group()


if __name__ == "__main__":
    main()
