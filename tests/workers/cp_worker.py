"""Worker for the fused ring-attention test on GPUs: remote K/V chunks are read in place by the attention kernel."""
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
    from pmetal_b200.parallel import cp
    T, hq, hkv, d = 512, 4, 2, 128
    g = torch.Generator(device=dev).manual_seed(3)            # same full sequence on every rank
    q = torch.randn(T * world, hq, d, device=dev, generator=g).bfloat16()
    k = torch.randn(T * world, hkv, d, device=dev, generator=g).bfloat16()
    v = torch.randn(T * world, hkv, d, device=dev, generator=g).bfloat16()
    ss = torch.zeros(T * world, dtype=torch.int32, device=dev)
    full, full_lse = native.attn_fwd(q, k, v, ss, d ** -0.5)
    ring = cp.FusedRingAttention(T, hkv, d)
    ql, kl, vl = (cp.split_sequence(t, rank, world).contiguous() for t in (q, k, v))
    for it in range(2):
        out, lse = ring.forward(ql, kl, vl)
        want = cp.split_sequence(full, rank, world)
        err = (out.float() - want.float()).abs().max().item()
        assert err < 0.03, f"fused ring attention err {err}"
        out2, _ = cp.ring_attention_p2p(ql, kl, vl)
        assert (out2.float() - want.float()).abs().max().item() < 0.03
    torch.cuda.synchronize()
    native.check_status()
    dist.barrier()
    if rank == 0:
        print("CP_WORKER_OK", flush=True)
    sys.stdout.flush()
    from pmetal_b200.parallel.dp import shutdown_process_group
    shutdown_process_group()


if __name__ == "__main__":
    main()
