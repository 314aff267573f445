"""Worker for the expert-parallel test: fused dispatch/GEMM/combine engine against a dense fp32 MoE reference."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def dense_reference(x, logits, gate_up, down, k, renorm):
    p = torch.softmax(logits.float(), -1)
    w, idx = p.topk(k, -1)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    I = down.shape[2]
    out = torch.zeros(x.shape[0], down.shape[1], dtype=torch.float32, device=x.device)
    for e in range(gate_up.shape[0]):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel():
            h = x[tok].float() @ gate_up[e].float().t()
            h = (torch.nn.functional.silu(h[:, :I]) * h[:, I:]).bfloat16().float()
            out.index_add_(0, tok, (h @ down[e].float().t()).bfloat16().float() * w[tok, slot][:, None])
    return out


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from pmetal_b200.ops import native
    from pmetal_b200.parallel.ep import FusedExpertMoE, expert_range
    E, k, H, I, T = 16, 4, 512, 256, 700
    g = torch.Generator(device=dev).manual_seed(7)            # same weights on every rank
    gate_up = (torch.randn(E, 2 * I, H, device=dev, generator=g) * 0.05).bfloat16()
    down = (torch.randn(E, H, I, device=dev, generator=g) * 0.05).bfloat16()
    a, b = expert_range(E, rank, world)
    eng = FusedExpertMoE(gate_up[a:b], down[a:b], E, k, max_tokens=1024, timeout_s=5.0)
    g2 = torch.Generator(device=dev).manual_seed(100 + rank)   # different tokens per rank
    for it in range(3):
        x = torch.randn(T, H, device=dev, generator=g2).bfloat16()
        logits = torch.randn(T, E, device=dev, generator=g2)
        y = eng.forward(x, logits)
        torch.cuda.synchronize()
        native.check_status()
        ref = dense_reference(x, logits, gate_up, down, k, True)
        err = (y.float() - ref).abs().max().item()
        assert err < 0.03 * ref.abs().max().item() + 2e-3, f"iter {it}: err {err} vs max {ref.abs().max().item()}"
    if rank == 0:
        print(f"ep fused ok: err {err:.3e}", flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        print("EP_WORKER_OK", flush=True)
    sys.stdout.flush()
    from pmetal_b200.parallel.dp import shutdown_process_group
    shutdown_process_group()


if __name__ == "__main__":
    main()
