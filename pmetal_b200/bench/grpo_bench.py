"""GRPO step benchmark: generation phase and policy-update phase timed separately.

    python -m pmetal_b200.bench.grpo_bench [--prompts 8] [--group 8] [--new-tokens 1024] [--steps 2]
    (multi-GPU: under torch.distributed.run; prompts are per GPU, gradients go through the fused data-parallel step)

Workload per step and GPU: ``prompts`` prompts of 256 uniform-random tokens, ``group`` rollouts each, up to ``new-tokens``
sampled at temperature 1.0 / top-p 1.0 on the paged KV cache; reward = fraction of tokens congruent to 0 mod 7 plus
0.001 * length; group-normalised advantages, clip 0.2, KL beta 0.04 against the frozen base."""
from __future__ import annotations

import argparse
import json
import os

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--prompts", type=int, default=8)
    ap.add_argument("--group", type=int, default=8)
    ap.add_argument("--new-tokens", type=int, default=1024)
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--model", default="qwen3-0.6b")
    ap.add_argument("--no-merged-rollout", action="store_true",
                    help="generate through the adapter-aware decode path instead of folded bf16 weights")
    a = ap.parse_args(argv)
    import torch.distributed as dist

    from ..core.config import LoraConfig
    from ..lora import apply_lora
    from ..models.config import preset
    from ..models.decoder import DecoderLM
    from ..ops import native
    from ..trainer.grpo import GrpoConfig, GrpoTrainer, mod7_length_reward
    world, rank, local = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dctx = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        from ..parallel.fused_dp import FusedDataParallel
        dctx = FusedDataParallel()
    cfg = preset(a.model)

    def build(lora: bool):
        m = DecoderLM(cfg).init_weights(0.02, 0).to(dev)
        for p in m.parameters():
            p.data = p.data.to(torch.bfloat16)
            p.requires_grad_(False)
        if lora:
            apply_lora(m, LoraConfig(r=16, alpha=32.0, target_modules=["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj",
                                                                       "up_proj", "down_proj"]), seed=1)
            m = m.to(dev)
            m.prepare_for_training()
        return m
    policy, ref = build(True), build(False).eval()
    gc = GrpoConfig(num_generations=a.group, max_prompt_length=a.prompt_len, max_completion_length=a.new_tokens, beta=0.04,
                    temperature=1.0, top_p=1.0, top_k=0, epsilon_low=0.2, epsilon_high=0.2, learning_rate=1e-6,
                    rollout_merged=not a.no_merged_rollout)
    blocks = a.prompts * a.group * ((a.prompt_len + a.new_tokens) // 64 + 2) + 64
    tr = GrpoTrainer(policy, gc, mod7_length_reward, reference=ref, kv_blocks=blocks, dist=dctx)
    g = torch.Generator().manual_seed(100 + rank)
    gen_s, train_s, toks, rewards = [], [], [], []
    for step in range(a.steps + 1):
        prompts = [torch.randint(0, cfg.vocab_size, (a.prompt_len,), generator=g).tolist() for _ in range(a.prompts)]
        st = tr.step(prompts)
        if step > 0:                    # the first step pays for graph captures and lazy initialisation
            gen_s.append(st.generation_seconds)
            train_s.append(st.train_seconds)
            toks.append(st.completion_tokens)
            rewards.append(st.mean_reward)
    native.check_status()

    def agg(x, op):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=op)
        return float(t.item())
    gs = agg(sum(gen_s) / len(gen_s), dist.ReduceOp.MAX if world > 1 else None)
    ts = agg(sum(train_s) / len(train_s), dist.ReduceOp.MAX if world > 1 else None)
    tk = agg(float(sum(toks) / len(toks)), dist.ReduceOp.SUM if world > 1 else None)
    if rank == 0:
        print(json.dumps({"bench": "grpo_step", "model": a.model, "n_gpus": world, "prompts_per_gpu": a.prompts, "group": a.group,
                          "max_new_tokens": a.new_tokens, "generation_s": round(gs, 3), "policy_update_s": round(ts, 3),
                          "completion_tokens_per_step": int(tk), "generation_tok_s": round(tk / gs, 1),
                          "step_tok_s": round(tk / (gs + ts), 1), "mean_reward": round(sum(rewards) / len(rewards), 4)}), flush=True)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        from pmetal_b200.parallel.dp import shutdown_process_group
        shutdown_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
