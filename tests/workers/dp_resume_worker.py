"""CPU (gloo) worker: every rank of a data-parallel job resumes from the checkpoint that rank 0 wrote, and optimizer
moments that are sharded across ranks are collected before they are saved."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    out_dir = os.environ["PMETAL_TEST_DIR"]
    dist.init_process_group("gloo")
    from pmetal_b200.core.config import LoraConfig, TrainingConfig
    from pmetal_b200.lora import apply_lora
    from pmetal_b200.lora.adapter import lora_state_dict
    from pmetal_b200.models.config import ModelArgs
    from pmetal_b200.models.decoder import DecoderLM
    from pmetal_b200.parallel.dp import DistContext
    from pmetal_b200.parallel.fused_dp import gather_sharded_, shard_range
    from pmetal_b200.trainer.checkpoint import CheckpointManager
    from pmetal_b200.trainer.loop import TrainingLoop

    # ---- shard arithmetic and collection of sharded moments
    total = 5 * 1024
    los = [shard_range(total, r, world) for r in range(world)]
    assert los[0][0] == 0 and los[-1][1] == total and all(a[1] == b[0] for a, b in zip(los, los[1:]))
    full = torch.arange(total, dtype=torch.float32)
    lo, hi = los[rank]
    mine = torch.full((total,), -7.0)               # stale values outside the owned shard must not survive
    mine[lo:hi] = full[lo:hi]
    gather_sharded_(mine, lo, hi)
    assert torch.equal(mine, full)

    # ---- train a few steps on different data per rank, save on rank 0, resume on every rank
    def build(seed):
        cfg = ModelArgs(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2,
                        num_key_value_heads=1, head_dim=16)
        m = DecoderLM(cfg).init_weights(0.05, 0)
        apply_lora(m, LoraConfig(r=4, alpha=8), seed=seed)
        return m
    dctx = DistContext()
    tcfg = TrainingConfig(gradient_accumulation_steps=1, warmup_steps=0, learning_rate=1e-2, lr_scheduler="cosine",
                          save_steps=3)
    ck = CheckpointManager(os.path.join(out_dir, "checkpoints"), keep=2, async_write=False) if rank == 0 else None
    loop = TrainingLoop(build(1), tcfg, dist=dctx, checkpoint_manager=ck, total_steps=10)
    g = torch.Generator().manual_seed(100 + rank)
    for _ in range(3):
        ids = torch.randint(0, 128, (2, 16), generator=g)
        loop.train_step({"input_ids": ids, "labels": ids})
    loop.state.epoch = 1
    dctx.gather_optimizer_state(loop.opt)
    if rank == 0:
        loop.save_checkpoint()
        ck.wait()
    dctx.barrier()

    # a fresh job (different adapter seed): the path comes from rank 0, every rank loads it
    loop2 = TrainingLoop(build(2), tcfg, dist=dctx, total_steps=10)
    latest = ck.latest_path() if ck is not None else None
    latest = dctx.broadcast_object(latest, src=0)
    assert latest and latest.endswith("step_3")
    loop2.resume(latest)
    assert loop2.state.step == 3 and loop2.state.epoch == 1 and loop2.opt.step_count == 3
    flat = torch.cat([v.reshape(-1).float() for _, v in sorted(lora_state_dict(loop2.model).items())])
    mom = torch.cat([loop2.opt.flat_m, loop2.opt.flat_v])
    for t, ref in ((flat, torch.cat([v.reshape(-1).float() for _, v in sorted(lora_state_dict(loop.model).items())])),
                   (mom, torch.cat([loop.opt.flat_m, loop.opt.flat_v]))):
        got = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(got, t)
        assert all(torch.equal(got[0], x) for x in got), "ranks differ after resume"
        assert torch.equal(t, ref), "resumed state differs from the saved one"
    assert abs(loop2.current_lr() - loop.current_lr()) < 1e-12
    # one more step keeps the ranks identical (same lr, same bias correction, same moments)
    ids = torch.randint(0, 128, (2, 16), generator=g)
    loop2.train_step({"input_ids": ids, "labels": ids})
    flat = torch.cat([v.reshape(-1).float() for _, v in sorted(lora_state_dict(loop2.model).items())])
    got = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(got, flat)
    assert all(torch.equal(got[0], x) for x in got)
    dist.barrier()
    print("DP_RESUME_WORKER_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
