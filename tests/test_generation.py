import pytest
import torch

from pmetal_b200.models.config import preset
from pmetal_b200.models.decoder import DecoderLM
from pmetal_b200.models.generation import Generator
from pmetal_b200.models.kv_cache import BLOCK, PagedKVCache
from pmetal_b200.models.sampling import Sampler, SamplingParams, filtered_logprobs
from pmetal_b200.models.speculative import (LayerSplitDraft, SpeculativeConfig, SpeculativeDecoder, adjust_k,
                                            verify_greedy, verify_sampling)


def _model(seed=0, **kw):
    return DecoderLM(preset("tiny-qwen3", **kw)).init_weights(0.05, seed).eval()


def test_paged_decode_matches_full_forward():
    m = _model()
    g = Generator(m, num_blocks=64)
    prompt = torch.randint(0, 1024, (70,), generator=torch.Generator().manual_seed(0)).tolist()
    res = g.generate([prompt], SamplingParams.greedy(12))
    seq = list(prompt)
    for _ in range(12):
        nxt = int(m(torch.tensor(seq)[None])[0, -1].argmax())
        seq.append(nxt)
    assert res.tokens[0] == seq[len(prompt):]
    assert g.cache.num_free() == 64


def test_batched_generation_with_forks_and_chunked_prefill():
    m = _model(1)
    g = Generator(m, num_blocks=128)
    gen = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 1024, (n,), generator=gen).tolist() for n in (5, 130, 64)]
    single = [Generator(m, num_blocks=32).generate([p], SamplingParams.greedy(6)).tokens[0] for p in prompts]
    import pmetal_b200.models.generation as G
    old, G.PREFILL_CHUNK = G.PREFILL_CHUNK, 50
    try:
        res = g.generate(prompts, SamplingParams.greedy(6), num_return_sequences=2)
    finally:
        G.PREFILL_CHUNK = old
    assert res.tokens[0] == res.tokens[1] == single[0]
    assert res.tokens[2] == single[1] and res.tokens[4] == single[2]
    assert g.cache.num_free() == 128


def test_cache_fork_copy_on_write_and_truncate():
    c = PagedKVCache(1, 1, 8, 8, dtype=torch.float32, device="cpu")
    c.add_sequence(0)
    s0 = c.reserve(0, 70)
    c.k[0].view(-1, 1, 8)[torch.tensor(s0)] = torch.arange(70.0)[:, None, None].expand(70, 1, 8)
    c.fork(0, 1)
    assert c.seqs[1].blocks == c.seqs[0].blocks and c.num_free() == 6
    s1 = c.reserve(1, 1)                       # writes into the shared tail block -> copied first
    assert c.seqs[1].blocks[0] == c.seqs[0].blocks[0] and c.seqs[1].blocks[1] != c.seqs[0].blocks[1]
    k1, _ = c.gather(0, 1)
    assert torch.equal(k1[:70, 0, 0], torch.arange(70.0))
    c.truncate(1, 64)
    assert len(c.seqs[1].blocks) == 1
    c.free_sequence(0); c.free_sequence(1)
    assert c.num_free() == 8


def test_sampler_filters():
    logits = torch.log(torch.tensor([[0.5, 0.25, 0.15, 0.07, 0.03]]))
    lp = filtered_logprobs(logits, SamplingParams(top_k=3, top_p=1.0, min_p=0.0))
    assert torch.isinf(lp[0, 3:]).all() and not torch.isinf(lp[0, :3]).any()
    lp = filtered_logprobs(logits, SamplingParams(top_k=0, top_p=0.8, min_p=0.0))
    assert (~torch.isinf(lp[0])).tolist() == [True, True, True, False, False]
    lp = filtered_logprobs(logits, SamplingParams(top_k=0, top_p=1.0, min_p=0.2))
    assert (~torch.isinf(lp[0])).tolist() == [True, True, True, False, False]
    s = Sampler(SamplingParams.greedy())
    assert s.sample(logits).tolist() == [0]
    counts = torch.tensor([[3, 0, 0, 0, 0]])
    pen = Sampler(SamplingParams(do_sample=False, repetition_penalty=5.0, temperature=0.0))
    assert pen.sample(torch.tensor([[2.0, 1.0, 0.5, 0.1, 0.0]]), counts).tolist() == [1]
    draws = Sampler(SamplingParams(temperature=1.0, top_k=2, top_p=1.0, min_p=0.0, repetition_penalty=1.0, seed=0))
    ids = torch.stack([draws.sample(logits) for _ in range(200)])
    assert set(ids.flatten().tolist()) <= {0, 1}


def test_verify_rules():
    V = 6
    tl = torch.full((2, 4, V), -5.0)
    tgt = torch.tensor([[1, 2, 3, 4], [1, 5, 3, 4]])
    tl.scatter_(2, tgt[..., None], 5.0)
    draft = torch.tensor([[1, 2, 3], [1, 2, 3]])
    n, nxt = verify_greedy(tl, draft)
    assert n.tolist() == [3, 1] and nxt.tolist() == [4, 5]
    assert adjust_k(5, 5, 0.9) == 6 and adjust_k(10, 5, 0.95) == 10 and adjust_k(1, 5, 0.0) == 1
    # sampling verification reproduces the target distribution
    g = torch.Generator().manual_seed(0)
    pt = torch.tensor([0.6, 0.3, 0.1]); pd = torch.tensor([0.2, 0.2, 0.6])
    N = 20000
    d = torch.multinomial(pd, N, replacement=True, generator=g)[:, None]
    tl2 = torch.log(pt)[None, None, :].expand(N, 2, 3).contiguous()
    n_acc, new = verify_sampling(tl2, d, pd[None, None, :].expand(N, 1, 3).contiguous(), 1.0, g)
    first = torch.where(n_acc > 0, d[:, 0], new)
    freq = torch.bincount(first, minlength=3).float() / N
    assert torch.allclose(freq, pt, atol=0.02)


def test_two_model_speculative_equals_target_greedy():
    tgt = _model(0)
    draft = _model(5, num_hidden_layers=1)
    prompts = [torch.randint(0, 1024, (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (9, 33)]
    ref = Generator(tgt, num_blocks=32).generate(prompts, SamplingParams.greedy(20)).tokens
    sd = SpeculativeDecoder(tgt, draft, SpeculativeConfig(num_draft_tokens=4), 32, 32)
    out = sd.generate(prompts, 20)
    assert out == ref
    assert sd.stats.rounds > 0 and sd.t.cache.num_free() == 32 and sd.d.cache.num_free() == 32


def test_layer_split_self_speculation():
    tgt = _model(2, num_hidden_layers=3)
    draft = LayerSplitDraft(tgt)
    assert len(draft.layers) == 1
    prompts = [list(range(1, 12))]
    ref = Generator(tgt, num_blocks=16).generate(prompts, SamplingParams.greedy(10)).tokens
    out = SpeculativeDecoder(tgt, draft, SpeculativeConfig(num_draft_tokens=2), 16, 16).generate(prompts, 10)
    assert out == ref


def test_cache_mode_rule_and_paged_cache_variants_on_cpu():
    """The cache choice rule, and the int8 / rotating variants of the paged cache against the plain one (CPU path)."""
    import torch
    from pmetal_b200.models.config import ModelArgs
    from pmetal_b200.models.decoder import DecoderLM
    from pmetal_b200.models.generation import Generator
    from pmetal_b200.models.kv_cache import select_cache_mode
    from pmetal_b200.models.sampling import SamplingParams
    GB = 1 << 30
    assert select_cache_mode(10 * GB, 10 * GB, 180 * GB).source == "auto_fp16"
    m = select_cache_mode(100 * GB, 40 * GB, 180 * GB)
    assert (m.kind, m.bits, m.source) == ("quantized", 8, "auto_q8")
    assert select_cache_mode(100 * GB, 40 * GB, 180 * GB, no_kv_quant=True).source == "forced_fp16"
    assert select_cache_mode(100 * GB, 40 * GB, 180 * GB, kv_quant=0).kind == "standard"
    m = select_cache_mode(1, 1, 180 * GB, kv_quant=4)
    assert (m.kind, m.bits, m.source) == ("quantized", 4, "explicit")
    m = select_cache_mode(1, 1, 180 * GB, k_bits=8, v_bits=4)
    assert (m.kind, m.k_bits, m.v_bits) == ("asymmetric", 8, 4)
    m = select_cache_mode(1, 1, 180 * GB, k_bits=4)
    assert (m.kind, m.k_bits, m.v_bits) == ("asymmetric", 4, 8)
    assert select_cache_mode(1, 1, None, turboquant=True, kv_quant=3).kind == "turboquant"

    cfg = ModelArgs(vocab_size=300, hidden_size=128, intermediate_size=128, num_hidden_layers=2, num_attention_heads=2,
                    num_key_value_heads=1, head_dim=64)
    model = DecoderLM(cfg).init_weights(0.08, 0).eval()
    for p in model.parameters():
        p.requires_grad_(False)
    prompt = list(range(3, 150))
    plain = Generator(model, cache=model.new_cache(32)).generate([prompt], SamplingParams.greedy(20))
    q8 = Generator(model, cache=model.new_cache(32, quant="int8"))
    lg_a = Generator(model, cache=model.new_cache(32)).prefill([0], [prompt]) if False else None
    out8 = q8.generate([prompt], SamplingParams.greedy(20))
    same = sum(a == b for a, b in zip(plain.tokens[0], out8.tokens[0]))
    assert same >= 15, (plain.tokens[0], out8.tokens[0])          # int8 keys and values barely move the logits
    # logits with the int8 cache stay close to the 16-bit ones
    g1, g2 = Generator(model, cache=model.new_cache(32)), Generator(model, cache=model.new_cache(32, quant="int8"))
    s1, s2 = g1.new_seq(), g2.new_seq()
    l1, l2 = g1.prefill([s1], [prompt]), g2.prefill([s2], [prompt])
    assert (l1 - l2).abs().max() < 0.05 * l1.abs().max()
    # rotating cache: a window as long as the whole text changes nothing, and blocks behind the window are recycled
    win = Generator(model, cache=model.new_cache(32, window=4096, sink=4)).generate([prompt], SamplingParams.greedy(20))
    assert win.tokens[0] == plain.tokens[0]
    small = model.new_cache(32, window=64, sink=8)
    gs = Generator(model, cache=small)
    sid = gs.new_seq()
    gs.prefill([sid], [prompt])
    for _ in range(70):
        gs.decode_step([sid], torch.tensor([5]))
    assert small.length(sid) == len(prompt) + 70
    assert small.live_blocks(sid) <= 3 and small.seqs[sid].blocks[0] >= 0        # sink block + the window's blocks
    assert small.num_free() >= 32 - 3
    # the windowed result equals dense attention restricted to sink + window (the CPU path applies the same mask)
    small.free_sequence(sid)
    assert small.num_free() == 32


def test_rotated_4bit_cache_reference_path():
    """The rotated 4-bit code-book cache on the CPU path: written with the PyTorch quantiser, read back de-rotated; the
    logits stay close to the 16-bit cache and most greedy tokens agree."""
    from pmetal_b200.models.config import ModelArgs
    from pmetal_b200.models.decoder import DecoderLM
    from pmetal_b200.models.generation import Generator
    from pmetal_b200.models.sampling import SamplingParams
    cfg = ModelArgs(vocab_size=300, hidden_size=256, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                    num_key_value_heads=1, head_dim=128)
    model = DecoderLM(cfg).init_weights(0.05, 0).eval()
    for p in model.parameters():
        p.requires_grad_(False)
    prompt = list(range(3, 150))
    g1, g2 = Generator(model, cache=model.new_cache(32)), Generator(model, cache=model.new_cache(32, quant="tq4"))
    assert g2.cache.k[0].dtype == torch.uint8 and g2.cache.k[0].shape[-1] == 64
    s1, s2 = g1.new_seq(), g2.new_seq()
    l1, l2 = g1.prefill([s1], [prompt]), g2.prefill([s2], [prompt])
    assert (l1 - l2).norm() < 0.25 * l1.norm()           # a randomly initialised model amplifies the 10 % key error
    k16, _ = g1.cache.gather(0, s1)
    k4, _ = g2.cache.gather(0, s2)
    rel = (k16.float() - k4.float()).norm() / k16.float().norm()
    assert rel < 0.12, rel                          # 4-bit Lloyd-Max on unit-variance coordinates: about 10 % error
    with pytest.raises(ValueError):
        model.new_cache(8, quant="q2")
