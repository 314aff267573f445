"""Tiny decode run for launch-list profiling: one sequence, a few greedy tokens, no CUDA graphs.

    python -m pmetal_b200.bench.decode_trace [--tokens 6]
"""
import argparse
import os

os.environ.setdefault("PMETAL_DECODE_GRAPHS", "0")


def main() -> int:
    import torch

    from ..models.generation import Generator
    from ..models.loader import load_pretrained
    from ..models.sampling import SamplingParams
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=6)
    ap.add_argument("--model", default="random:qwen3-0.6b")
    a = ap.parse_args()
    m, _, _ = load_pretrained(a.model, dtype=torch.bfloat16, device="cuda")
    m.eval()
    for p in m.parameters():
        p.requires_grad_(False)
    g = Generator(m, num_blocks=256, cuda_graphs=False)
    r = g.generate([list(range(1, 65))], SamplingParams.greedy(a.tokens))
    torch.cuda.synchronize()
    print("generated", r.generated_tokens)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
