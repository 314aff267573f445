"""Worker (gloo on CPU, NCCL on GPUs): context-parallel causal attention with zig-zag sharding, forward and backward,
against the same attention computed on the whole sequence by one process."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    gpu = torch.cuda.is_available() and os.environ.get("PMETAL_TEST_CPU", "0") != "1"
    if gpu:
        local = int(os.environ["LOCAL_RANK"])
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    from pmetal_b200.parallel import cp
    assert [cp.zigzag_chunks(r, 4) for r in range(4)] == [(0, 7), (1, 6), (2, 5), (3, 4)]
    c, hq, hkv, d = (256, 4, 2, 128) if gpu else (6, 4, 2, 8)
    T = 2 * world * c
    dt = torch.bfloat16 if gpu else torch.float32
    g = torch.Generator().manual_seed(11)                 # the same full sequence on every rank
    q = (torch.randn(T, hq, d, generator=g) * 0.8).to(dt).to(dev)
    k = (torch.randn(T, hkv, d, generator=g) * 0.8).to(dt).to(dev)
    v = torch.randn(T, hkv, d, generator=g).to(dt).to(dev)
    do = torch.randn(T, hq, d, generator=g).to(dt).to(dev)
    # whole sequence, fp32 reference
    qf, kf, vf = (t.float().clone().requires_grad_(True) for t in (q, k, v))
    rep = hq // hkv
    s = torch.einsum("thd,shd->hts", qf, kf.repeat_interleave(rep, 1)) * d ** -0.5
    s = s.masked_fill(torch.ones(T, T, dtype=torch.bool, device=dev).triu(1), float("-inf"))
    ref = torch.einsum("hts,shd->thd", torch.softmax(s, -1), vf.repeat_interleave(rep, 1))
    ref.backward(do.float())
    # sharded
    ql, kl, vl = (cp.zigzag_split(t, rank, world).contiguous().requires_grad_(True) for t in (q, k, v))
    assert torch.equal(cp.zigzag_gather(ql.detach()), q)
    out = cp.zigzag_attention(ql, kl, vl)
    out.backward(cp.zigzag_split(do, rank, world).contiguous())
    tol = 4e-2 if gpu else 1e-4

    def close(a, b, what):
        err = (a.float() - b.float()).abs().max().item()
        assert err <= tol * max(1.0, b.float().abs().max().item()), f"{what}: err {err}"
    close(out, cp.zigzag_split(ref.detach(), rank, world), "output")
    close(ql.grad, cp.zigzag_split(qf.grad, rank, world), "dq")
    close(kl.grad, cp.zigzag_split(kf.grad, rank, world), "dk")
    close(vl.grad, cp.zigzag_split(vf.grad, rank, world), "dv")
    if gpu:
        from pmetal_b200.ops import native
        torch.cuda.synchronize()
        native.check_status()
    dist.barrier()
    print("CP_TRAIN_WORKER_OK", flush=True)
    if gpu:
        from pmetal_b200.parallel.dp import shutdown_process_group
        shutdown_process_group()
    else:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
