"""Tiny decode runs for profiling.

    python -m pmetal_b200.bench.decode_trace [--tokens 6]             one sequence, a few greedy tokens, no CUDA graphs
                                                                       (launch lists under a profiler)
    python -m pmetal_b200.bench.decode_trace --phases [--batch 1]     per-phase device timestamps of the whole-step
                                                                       decode kernel (csrc/decode_mega.cu): staging,
                                                                       mat-vec, attention and barrier time per layer
"""
import argparse
import json
import os

PHASES = ["P1 stage", "P1 qkv mat-vec", "P1 barrier", "P2 attention", "P2 barrier", "P3 stage", "P3 o-proj mat-vec",
          "P3 barrier", "P4 stage", "P4 gate/up mat-vec", "P4 barrier", "P5 stage", "P5 down mat-vec", "P5 barrier"]


def phase_trace(model, batch: int, prompt_len: int = 128) -> dict:
    """Median duration (us) of every phase over the layers of one decode step, read from the timestamps that CTA 0
    writes when the kernel is given a trace buffer."""
    import torch

    from ..models.generation import Generator
    from ..ops import native
    n_layers = len(model.layers)
    dev = model.embed_tokens.device
    gen = Generator(model, num_blocks=1024, cuda_graphs=False)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, model.cfg.vocab_size, (prompt_len,), generator=g).tolist() for _ in range(batch)]
    seqs = [gen.new_seq() for _ in prompts]
    ids = gen.prefill(seqs, prompts).argmax(-1)
    for _ in range(3):
        ids = gen.decode_step(seqs, ids).argmax(-1)
    trace = torch.zeros(n_layers * 16, dtype=torch.int64, device=dev)
    make = native.decode_scratch

    def with_trace(*a, **k):
        d = make(*a, **k)
        d["trace"] = trace
        return d
    native.decode_scratch = with_trace
    model._mega_scratch.clear()
    try:
        for _ in range(3):
            ids = gen.decode_step(seqs, ids).argmax(-1)
        torch.cuda.synchronize()
    finally:
        native.decode_scratch = make
        model._mega_scratch.clear()
    t = trace.view(n_layers, 16).cpu()
    d = (t[:, 1:15] - t[:, 0:14]).float()
    out = {name: round(d[2:, i].median().item() / 1e3, 2) for i, name in enumerate(PHASES)}
    out["layer_us"] = round(float((t[2:, 14] - t[2:, 0]).float().median()) / 1e3, 2)
    out["all_layers_ms"] = round(float(t[-1, 14] - t[0, 0]) / 1e6, 3)
    return out


def add_arguments(ap) -> None:
    ap.add_argument("--tokens", type=int, default=6)
    ap.add_argument("--model", default="random:qwen3-0.6b")
    ap.add_argument("--phases", action="store_true")
    ap.add_argument("--batch", type=int, default=1)


def main(argv=None, args=None) -> int:
    """Also reachable as ``pmetal bench-decode`` (which passes its parsed arguments as ``args``)."""
    os.environ.setdefault("PMETAL_DECODE_GRAPHS", "0")      # eager launches: one kernel per launch under a profiler
    import torch

    from ..models.generation import Generator
    from ..models.loader import load_pretrained
    from ..models.sampling import SamplingParams
    a = args
    if a is None:
        ap = argparse.ArgumentParser()
        add_arguments(ap)
        a = ap.parse_args(argv)
    m, _, _ = load_pretrained(a.model, dtype=torch.bfloat16, device="cuda")
    m.eval()
    for p in m.parameters():
        p.requires_grad_(False)
    if a.phases:
        print(json.dumps({"batch": a.batch, **phase_trace(m, a.batch)}))
        return 0
    g = Generator(m, num_blocks=256, cuda_graphs=False)
    r = g.generate([list(range(1, 65))], SamplingParams.greedy(a.tokens))
    torch.cuda.synchronize()
    print("generated", r.generated_tokens)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
