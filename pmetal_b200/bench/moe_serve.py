"""Mixture-of-experts serving benchmark: concurrent requests on a Qwen3-30B-A3B-shaped model with expert parallelism.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29660 \
        -m pmetal_b200.bench.moe_serve [--requests 64] [--prompt-len 512] [--new-tokens 256] [--model qwen3-30b-a3b]

Parallelism: every rank holds the attention weights and serves ``requests / N`` of the requests (data-parallel attention
with its own paged KV cache); the experts are split across ranks and every MoE layer runs the fused
routing + dispatch + grouped-GEMM + combine kernels over NVLink peer memory (parallel/ep.py). All ranks step in
lock-step (same number of requests, prompt lengths and greedy decode steps), which the device-side flags require.
Reported: prefill tokens/s, decode tokens/s and requests/s for the whole job, device-timed, maximum over ranks.

``--tp`` selects the other layout: tensor-parallel attention (every rank keeps ``heads / N`` query heads and the kv heads
they read) with the experts split over the ranks, all requests replicated on every rank and the two partial results
of a layer summed across ranks (``parallel/tp_model.py``; ``--reduce peer`` uses the one-kernel exchange over
symmetric memory instead of NCCL). ``--draft qwen3-0.6b --spec-k 4`` adds a replicated draft model that proposes
``k`` tokens per round, verified by the target in one forward of ``k + 1`` tokens per request (greedy)."""
from __future__ import annotations

import argparse
import json
import os
import time

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--model", default="qwen3-30b-a3b")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (0 = the architecture's own)")
    ap.add_argument("--tp", action="store_true", help="tensor-parallel attention + experts split over ranks, replicated requests")
    ap.add_argument("--reduce", default="nccl", choices=["nccl", "peer"])
    ap.add_argument("--draft", default=None, help="draft architecture for speculative decoding (e.g. qwen3-0.6b)")
    ap.add_argument("--spec-k", type=int, default=4)
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--emulate-world", type=int, default=0,
                    help="with --tp on one GPU: run rank 0's slice of a W-rank layout without the cross-rank sums "
                         "(one rank's share of the work per step)")
    ap.add_argument("--profile", action="store_true", help="print per-kernel device times of a few decode steps")
    a = ap.parse_args(argv)
    if a.tp:
        return main_tp(a)
    import torch.distributed as dist

    from ..models.config import preset
    from ..models.decoder import DecoderLM
    from ..models.generation import Generator
    from ..ops import native
    from ..parallel.ep import shard_experts
    world, rank, local = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = preset(a.model)
    if a.layers:
        cfg.num_hidden_layers = a.layers
    t0 = time.time()
    model = DecoderLM(cfg, dtype=torch.bfloat16, device=dev).init_weights_on_device(0.02, 0).eval()
    for p in model.parameters():
        p.requires_grad_(False)
    per_rank = a.requests // world
    chunk = 2048
    for layer in model.layers:
        if hasattr(layer.mlp, "router"):
            shard_experts(layer.mlp, None if world == 1 else dist.group.WORLD, max_tokens=chunk)
            # the engine holds this rank's experts; the stacked originals are no longer needed
            layer.mlp.gate_up = torch.nn.Parameter(torch.empty(0, dtype=torch.bfloat16, device=dev), requires_grad=False)
            layer.mlp.down = torch.nn.Parameter(torch.empty(0, dtype=torch.bfloat16, device=dev), requires_grad=False)
    torch.cuda.empty_cache()
    build_s = time.time() - t0
    blocks = per_rank * ((a.prompt_len + a.new_tokens) // 64 + 2) + 64
    gen = Generator(model, num_blocks=blocks)
    g = torch.Generator().manual_seed(10 + rank)
    prompts = [torch.randint(0, cfg.vocab_size, (a.prompt_len,), generator=g).tolist() for _ in range(per_rank)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def run(new_tokens: int):
        seqs = [gen.new_seq() for _ in prompts]
        barrier()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        logits = gen.prefill(seqs, prompts, chunk)
        ids = logits.argmax(-1)
        e1.record()
        for _ in range(new_tokens - 1):
            logits = gen.decode_step(seqs, ids)
            ids = logits.argmax(-1)
            _ = ids.tolist()
        e2.record()
        barrier()
        for s in seqs:
            gen.cache.free_sequence(s)
        return e0.elapsed_time(e1), e1.elapsed_time(e2)
    run(8)                                    # warm-up: graph captures, lazy initialisation
    pre_ms, dec_ms = run(a.new_tokens)
    native.check_status()

    def mx(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    pre_ms, dec_ms = mx(pre_ms), mx(dec_ms)
    if rank == 0:
        total = per_rank * world
        print(json.dumps({"bench": "moe_serve", "model": a.model, "layers": cfg.num_hidden_layers, "n_gpus": world,
                          "requests": total, "prompt_len": a.prompt_len, "new_tokens": a.new_tokens,
                          "parallelism": f"dp-attention x ep{world}", "build_s": round(build_s, 1),
                          "prefill_tok_s": round(total * a.prompt_len / (pre_ms / 1e3), 1),
                          "decode_tok_s": round(total * (a.new_tokens - 1) / (dec_ms / 1e3), 1),
                          "decode_ms_per_step": round(dec_ms / (a.new_tokens - 1), 3),
                          "requests_per_s": round(total / ((pre_ms + dec_ms) / 1e3), 3)}), flush=True)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        from pmetal_b200.parallel.dp import shutdown_process_group
        shutdown_process_group()
    return 0


def main_tp(a) -> int:
    import torch.distributed as dist

    from ..models.config import preset
    from ..models.decoder import DecoderLM
    from ..models.generation import Generator
    from ..models.speculative import SpeculativeConfig, SpeculativeDecoder
    from ..ops import native
    from ..parallel.tp_model import AllReduce, PeerAllReduce, shard_for_serving
    world, rank, local = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = preset(a.model)
    if a.layers:
        cfg.num_hidden_layers = a.layers
    t0 = time.time()
    model = DecoderLM(cfg, dtype=torch.bfloat16, device=dev).init_weights_on_device(0.02, 0).eval()
    for p in model.parameters():
        p.requires_grad_(False)
    red = None
    if world > 1:
        red = PeerAllReduce(None, max_elems=1 << 20) if a.reduce == "peer" else AllReduce(None)
        shard_for_serving(model, None, red)
    elif a.emulate_world > 1:
        class _NoSum:
            world = a.emulate_world

            def __call__(self, x):
                return x
        shard_for_serving(model, None, _NoSum(), rank=0, world=a.emulate_world)
    build_s = time.time() - t0
    n_req = a.requests
    blocks = n_req * ((a.prompt_len + a.new_tokens + 8) // 64 + 2) + 64
    graphs = False if a.no_graphs else None
    g = torch.Generator().manual_seed(10)                # the same requests on every rank
    prompts = [torch.randint(0, cfg.vocab_size, (a.prompt_len,), generator=g).tolist() for _ in range(n_req)]
    draft = None
    if a.draft:
        dcfg = preset(a.draft)
        dcfg.vocab_size = cfg.vocab_size
        draft = DecoderLM(dcfg, dtype=torch.bfloat16, device=dev).init_weights_on_device(0.02, 1).eval()
        for p in draft.parameters():
            p.requires_grad_(False)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def mx(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    gen = Generator(model, num_blocks=blocks, cuda_graphs=graphs)

    def run(new_tokens: int):
        seqs = [gen.new_seq() for _ in prompts]
        barrier()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        logits = gen.prefill(seqs, prompts, 4096)
        ids = logits.argmax(-1)
        e1.record()
        for _ in range(new_tokens - 1):
            logits = gen.decode_step(seqs, ids)
            ids = logits.argmax(-1)
            _ = ids.tolist()
        e2.record()
        barrier()
        for s_ in seqs:
            gen.cache.free_sequence(s_)
        return e0.elapsed_time(e1), e1.elapsed_time(e2)
    run(8)
    pre_ms, dec_ms = run(a.new_tokens)
    native.check_status()
    if a.profile and rank == 0:
        from torch.profiler import ProfilerActivity, profile
        seqs = [gen.new_seq() for _ in prompts]
        ids = gen.prefill(seqs, prompts, 4096).argmax(-1)
        for _ in range(3):
            ids = gen.decode_step(seqs, ids).argmax(-1)
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(5):
                ids = gen.decode_step(seqs, ids).argmax(-1)
            torch.cuda.synchronize()
        print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=24, max_name_column_width=56), flush=True)
        for s_ in seqs:
            gen.cache.free_sequence(s_)
    pre_ms, dec_ms = mx(pre_ms), mx(dec_ms)
    out = {"bench": "moe_serve", "model": a.model, "layers": cfg.num_hidden_layers, "n_gpus": world, "requests": n_req,
           "prompt_len": a.prompt_len, "new_tokens": a.new_tokens,
           "parallelism": (f"tp{world} attention x ep{world} experts (replicated requests, {a.reduce} all-reduce)" if world > 1
                           else f"rank 0 of an emulated tp{a.emulate_world} x ep{a.emulate_world} layout, no cross-rank sums"
                           if a.emulate_world > 1 else "one GPU"),
           "build_s": round(build_s, 1), "prefill_tok_s": round(n_req * a.prompt_len / (pre_ms / 1e3), 1),
           "decode_tok_s": round(n_req * (a.new_tokens - 1) / (dec_ms / 1e3), 1),
           "decode_ms_per_step": round(dec_ms / (a.new_tokens - 1), 3),
           "requests_per_s": round(n_req / ((pre_ms + dec_ms) / 1e3), 3)}
    if draft is not None:
        del gen
        torch.cuda.empty_cache()
        sd = SpeculativeDecoder(model, draft, SpeculativeConfig(num_draft_tokens=a.spec_k, temperature=0.0, adaptive_k=False),
                                target_blocks=blocks, draft_blocks=blocks, cuda_graphs=graphs)
        sd.generate(prompts[:8], 8)                      # warm-up
        sd.stats.__init__()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        toks = sd.generate(prompts, a.new_tokens)
        e1.record()
        barrier()
        native.check_status()
        ms = mx(e0.elapsed_time(e1))
        n_out = sum(len(t) for t in toks)
        out["speculative"] = {"draft": a.draft, "k": a.spec_k, "acceptance_rate": round(sd.stats.acceptance_rate, 4),
                              "tokens_per_round": round(sd.stats.tokens_per_round, 3), "rounds": sd.stats.rounds,
                              "total_ms": round(ms, 1), "tok_s_incl_prefill": round(n_out / (ms / 1e3), 1),
                              "ms_per_round": round(ms / max(sd.stats.rounds, 1), 3)}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        del model, draft, red
        from pmetal_b200.parallel.dp import shutdown_process_group
        shutdown_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
