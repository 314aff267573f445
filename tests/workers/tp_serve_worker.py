"""CPU (gloo) worker: a model cut into tensor-parallel attention + expert-parallel (or channel-parallel) feed-forward
slices gives, on every rank, the logits of the whole model; greedy decoding and speculative decoding with a replicated
draft stay token-for-token identical to the single-process run."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def build(kind: str, hkv: int):
    from pmetal_b200.models.config import ModelArgs
    from pmetal_b200.models.decoder import DecoderLM
    kw = dict(model_type="qwen3_moe", num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32) if kind == "moe" else {}
    cfg = ModelArgs(vocab_size=97, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=hkv, head_dim=8, **kw)
    m = DecoderLM(cfg).init_weights(0.2, 0).eval()
    for p in m.parameters():
        p.requires_grad_(False)
    return m


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    from pmetal_b200.models.generation import Generator
    from pmetal_b200.models.sampling import SamplingParams
    from pmetal_b200.parallel.tp_model import head_shard, shard_for_serving
    assert head_shard(32, 4, 5, 8) == (20, 4, 2, 1) and head_shard(16, 8, 3, 4) == (12, 4, 6, 2)
    prompts = [[5, 9, 11, 3, 60, 61, 7], list(range(1, 40))]
    for kind, hkv in (("moe", 2), ("moe", 1), ("dense", 2)):
        whole = build(kind, hkv)
        ref_gen = Generator(whole, num_blocks=16)
        ref = ref_gen.generate(prompts, SamplingParams.greedy(10))
        s1, s2 = ref_gen.new_seq(), ref_gen.new_seq()
        ref_logits = ref_gen.prefill([s1, s2], prompts)
        cut = build(kind, hkv)
        shard_for_serving(cut)
        assert cut.kv_heads_local == max(hkv // world, 1)
        n_full = sum(p.numel() for p in whole.parameters())
        n_cut = sum(p.numel() for p in cut.parameters())
        assert n_cut < 0.8 * n_full
        gen = Generator(cut, num_blocks=16)
        assert gen.cache.hkv == cut.kv_heads_local
        a, b = gen.new_seq(), gen.new_seq()
        logits = gen.prefill([a, b], prompts)
        assert torch.allclose(logits, ref_logits, rtol=1e-4, atol=1e-4), (kind, hkv, (logits - ref_logits).abs().max())
        gen.cache.free_sequence(a); gen.cache.free_sequence(b)
        out = gen.generate(prompts, SamplingParams.greedy(10))
        assert out.tokens == ref.tokens, (kind, hkv, out.tokens, ref.tokens)
        got = [None] * world
        dist.all_gather_object(got, out.tokens)
        assert all(g == got[0] for g in got)
    dist.barrier()
    print("TP_SERVE_WORKER_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
