"""Worker (gloo on CPU, NCCL on GPUs): a mixture-of-experts decoder whose experts are sharded over the ranks gives, for
every rank's own tokens, the outputs and gradients of the unsharded model, and the expert slices receive the gradient
contributions of all ranks' tokens."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    gpu = torch.cuda.is_available() and os.environ.get("PMETAL_TEST_CPU", "0") != "1"
    from pmetal_b200.models.config import preset
    from pmetal_b200.models.decoder import DecoderLM
    from pmetal_b200.models.moe import SparseMoeBlock
    from pmetal_b200.parallel.dp import DistContext, shutdown_process_group
    from pmetal_b200.parallel.ep_train import average_replicated_gradients, expert_parameters, shard_experts_for_training
    DistContext.from_env("nccl" if gpu else "gloo")
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"])) if gpu else torch.device("cpu")
    dtype = torch.bfloat16 if gpu else torch.float32
    cfg = preset("tiny-qwen3-moe")
    if gpu:
        cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads = 128, 2, 1
    full = DecoderLM(cfg, dtype=dtype).init_weights(0.1, 0).to(dev)
    sharded = DecoderLM(cfg, dtype=dtype).init_weights(0.1, 0).to(dev)
    assert shard_experts_for_training(sharded) == cfg.num_hidden_layers
    blk = next(m for m in sharded.modules() if isinstance(m, SparseMoeBlock))
    a, b = blk.local_experts
    assert blk.gate_up.shape[0] == b - a == cfg.num_experts // world
    for m in (full, sharded):
        for p in m.parameters():
            p.requires_grad_(True)
    # every rank has its own tokens; the reference model sees all of them
    g = torch.Generator().manual_seed(7)
    all_ids = torch.randint(0, cfg.vocab_size, (world, 48), generator=g).to(dev)
    read = torch.randn(world, 48, cfg.hidden_size, generator=g).to(dev)

    def run(model, ids, r):
        T = ids.numel()
        pos = torch.arange(T, dtype=torch.int32, device=dev)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        h = model.forward_hidden(ids, pos, cu, torch.zeros(T, dtype=torch.int32, device=dev))
        return h, (h.float() * r.float()).sum() / world

    h_s, loss_s = run(sharded, all_ids[rank], read[rank])
    loss_s.backward()
    average_replicated_gradients(sharded)
    total = 0.0
    outs = []
    for r in range(world):
        h_f, loss_f = run(full, all_ids[r], read[r])
        loss_f.backward()
        outs.append(h_f.detach())
    tol = 3e-2 if gpu else 1e-5
    err = (h_s.detach().float() - outs[rank].float()).norm() / outs[rank].float().norm()
    assert float(err) < tol, f"rank {rank}: hidden states differ by {float(err)}"
    fb = next(m for m in full.modules() if isinstance(m, SparseMoeBlock))
    for name in ("gate_up", "down"):
        want = getattr(fb, name).grad[a:b].float() / world          # the mean over ranks of the summed loss
        got = getattr(blk, name).grad.float()
        e = (got - want).norm() / want.norm().clamp(min=1e-12)
        assert float(e) < (8e-2 if gpu else 1e-4), f"rank {rank}: expert gradient {name} differs by {float(e)}"
    for (n1, p1), (n2, p2) in zip(sharded.named_parameters(), full.named_parameters()):
        if p1.shape != p2.shape or p1.grad is None:
            continue
        want = p2.grad.float() / world
        e = (p1.grad.float() - want).norm() / want.norm().clamp(min=1e-12)
        assert float(e) < (8e-2 if gpu else 1e-4), f"rank {rank}: gradient of {n1} differs by {float(e)}"
    assert len(expert_parameters(sharded)) == 2 * cfg.num_hidden_layers
    dist.barrier()
    print("EP_TRAIN_WORKER_OK", flush=True)
    shutdown_process_group()


if __name__ == "__main__":
    main()
