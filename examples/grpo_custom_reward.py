"""GRPO with a reward written in Python: completions that contain more distinct tokens score higher.

    python examples/grpo_custom_reward.py --model random:tiny-qwen3 --steps 2 --device cpu

A reward function receives the prompts and the sampled completions as token lists (one entry per completion, grouped by
prompt) and returns one float per completion; use ``model.tokenizer.decode`` inside it to score text."""
import argparse
import json

import torch

from pmetal_b200.core.config import LoraConfig
from pmetal_b200.lora import apply_lora
from pmetal_b200.models.loader import load_pretrained
from pmetal_b200.trainer.grpo import GrpoConfig, GrpoTrainer


def distinct_token_reward(prompts, completions):
    return [len(set(c)) / max(len(c), 1) for c in completions]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="random:tiny-qwen3")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--device", default=None)
    a = ap.parse_args()
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    model, args, _ = load_pretrained(a.model, dtype=torch.bfloat16 if dev.startswith("cuda") else torch.float32, device=dev)
    apply_lora(model, LoraConfig(r=8, alpha=16.0))
    model.to(dev).train()
    cfg = GrpoConfig(num_generations=4, max_completion_length=16, beta=0.0, learning_rate=1e-4)
    trainer = GrpoTrainer(model, cfg, distinct_token_reward, kv_blocks=256)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, args.vocab_size, (12,), generator=g).tolist() for _ in range(4)]
    for step in range(a.steps):
        st = trainer.step(prompts[step % 2 * 2:step % 2 * 2 + 2])
        print(json.dumps({"step": step + 1, "mean_reward": round(st.mean_reward, 4), "loss": round(st.loss, 5),
                          "generated_tokens": st.completion_tokens}))


if __name__ == "__main__":
    main()
