"""Workload benchmark (the analogue of ``pmetal bench-workload`` / ``bench-gen``,
crates/pmetal/src/commands/bench.rs:152-368,2549-2692): real prefill / decode sessions and a short LoRA training run on
one model, reporting prefill tok/s, decode tok/s, ms/token and training tok/s with step times."""
from __future__ import annotations

import json
import statistics
import time


def _sync():
    import torch
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def bench_generation(model, prompts, decode_steps: int = 16, sessions: int = 3) -> dict:
    from ..models.generation import Generator
    from ..models.sampling import SamplingParams
    gen = Generator(model, num_blocks=max(256, sum(len(p) for p in prompts) // 64 + 64))
    pre, dec = [], []
    for _ in range(sessions):
        r = gen.generate(prompts, SamplingParams.greedy(decode_steps))
        pre.append(r.prefill_tok_per_s)
        dec.append(r.decode_tok_per_s)
    return {"prefill_tok_s_median": round(statistics.median(pre), 1), "decode_tok_s_median": round(statistics.median(dec), 1),
            "ms_per_token": round(1000.0 * len(prompts) / max(statistics.median(dec), 1e-9), 3),
            "batch": len(prompts), "decode_steps": decode_steps}


def bench_training(model, vocab: int, samples: int = 4, steps: int = 2, seq_len: int = 2048) -> dict:
    import torch

    from ..core.config import LoraConfig, TrainingConfig
    from ..data.dataloader import synthetic_documents
    from ..data.packing import PackerConfig, SequencePacker, collate_packs
    from ..lora import apply_lora
    from ..trainer.loop import TrainingLoop
    dev = model.embed_tokens.device
    apply_lora(model, LoraConfig(r=16, alpha=32.0, target_modules=["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj",
                                                                  "up_proj", "down_proj"]))
    model.to(dev)
    model.prepare_for_training()
    loop = TrainingLoop(model, TrainingConfig(learning_rate=2e-4, gradient_accumulation_steps=1, warmup_steps=0))
    docs = synthetic_documents(samples * steps * 4 + 8, 64, seq_len, vocab, seed=3)
    packs = SequencePacker(PackerConfig(max_length=seq_len, max_seq_length=seq_len)).pack(docs)
    times, toks = [], []
    for s in range(steps + 1):
        b = collate_packs([packs[(s * samples + j) % len(packs)] for j in range(samples)], seq_len).to(dev)
        _sync()
        t0 = time.perf_counter()
        loop.train_step(b)
        _sync()
        if s > 0:                       # the first step initialises optimiser state
            times.append(time.perf_counter() - t0)
            toks.append(b.total_tokens)
    tps = [n / t for n, t in zip(toks, times)]
    return {"train_tok_s_median": round(statistics.median(tps), 1), "train_tok_s_mean": round(sum(tps) / len(tps), 1),
            "step_ms_median": round(1000 * statistics.median(times), 2), "steps": steps, "samples_per_step": samples}


def main(a) -> int:
    import torch

    from ..models.loader import load_pretrained
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    dtype = torch.bfloat16 if dev.startswith("cuda") else torch.float32
    experts_dir = getattr(a, "experts_dir", None)
    model, args, _ = load_pretrained(a.model, dtype=dtype, device=dev, experts_dir=experts_dir)
    model.eval()
    for p in model.parameters():
        p.requires_grad_(False)
    g = torch.Generator().manual_seed(0)
    bs, sl = getattr(a, "batch_size", None), getattr(a, "seq_len", None)
    lens = [sl or 512] * bs if bs else ((sl,) * 4 if sl else (128, 256, 512, 1024))
    prompts = [torch.randint(0, args.vocab_size, (n,), generator=g).tolist() for n in lens]
    out = {"model": a.model, "device": dev, "generation": bench_generation(model, prompts)}
    store = getattr(model, "expert_store", None)
    if store is not None:                      # experts streamed from a packed directory: what the reads cost
        st = store.stats
        out["expert_io"] = {"reads": st["reads"], "gib": round(st["bytes"] / 2 ** 30, 3),
                            "read_seconds": round(st["read_seconds"], 3), "prefetch_hit_rate": round(store.hit_rate(), 3)}
    if a.what == "workload" and store is None:
        out["training"] = bench_training(model, args.vocab_size, samples=bs or 4,
                                         seq_len=sl or (2048 if dev.startswith("cuda") else 256))
    print(json.dumps(out))
    if a.json:
        with open(a.json, "w", encoding="utf-8") as fh:
            json.dump(out, fh, indent=2)
    return 0
