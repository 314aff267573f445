"""Two-model speculative decoding on the config-driven architectures."""
import pytest
import torch

from pmetal_b200.models.architectures.generic import GenericDecoderLM, arch_config_from_hf
from pmetal_b200.models.architectures.speculative import speculative_generate, truncate_cache


def _model(layers, seed, family="gemma2"):
    cfg = dict(model_type=family, vocab_size=120, hidden_size=32, intermediate_size=64, num_hidden_layers=layers,
               num_attention_heads=4, num_key_value_heads=2, head_dim=8, max_position_embeddings=256, sliding_window=16,
               final_logit_softcapping=30.0, attn_logit_softcapping=50.0, query_pre_attn_scalar=8)
    torch.manual_seed(seed)
    return GenericDecoderLM(arch_config_from_hf(cfg)).init_weights(0.4, seed).eval()


def _greedy(model, prompt, n):
    cache = model.new_cache()
    cur, out = torch.tensor([prompt]), []
    with torch.no_grad():
        for _ in range(n):
            nxt = int(model(cur, cache)[:, -1].argmax(-1))
            out.append(nxt)
            cur = torch.tensor([[nxt]])
    return out


@pytest.mark.parametrize("k", [1, 3, 5])
def test_greedy_speculation_reproduces_the_target_exactly(k):
    target = _model(3, 0)
    prompt = [3, 17, 99, 4, 56, 8]
    want = _greedy(target, prompt, 24)
    for draft in (_model(1, 5), target):                      # an unrelated draft, and the target as its own draft
        st = speculative_generate(target, draft, prompt, 24, k=k)
        assert st.tokens == want
        assert st.proposed >= st.accepted >= 0 and st.rounds > 0
    assert st.acceptance_rate == 1.0 and st.rounds < 24        # a perfect draft: every proposal accepted, fewer target calls


def test_eos_and_budget_and_cache_roll_back():
    target = _model(2, 1)
    prompt = [9, 9, 2]
    base = _greedy(target, prompt, 12)
    stop = base[5]
    cut = base.index(stop) + 1
    st = speculative_generate(target, _model(1, 2), prompt, 12, k=4, eos_ids=[stop])
    assert st.tokens == base[:cut]
    assert len(speculative_generate(target, target, prompt, 7, k=4).tokens) == 7
    cache = target.new_cache()
    with torch.no_grad():
        target(torch.tensor([prompt + base[:4]]), cache)
        full = target(torch.tensor([[base[4]]]), cache)[:, -1]
        truncate_cache(cache, len(prompt) + 2)
        assert cache.length() == len(prompt) + 2
        again = target(torch.tensor([base[2:5]]), cache)[:, -1]
    assert torch.allclose(full, again, atol=1e-5)
    with pytest.raises(TypeError):
        truncate_cache(target.new_cache(kv_bits=8), 1)


def test_sampling_keeps_the_target_distribution():
    """First generated token after a fixed prefix, many seeds: speculative sampling and plain sampling agree in distribution."""
    target, draft = _model(2, 3), _model(1, 4)
    prompt = [5, 6, 7]
    with torch.no_grad():
        p0 = torch.softmax(target(torch.tensor([prompt]))[0, -1].float(), -1)
        first = int(p0.argmax())
        p1 = torch.softmax(target(torch.tensor([prompt + [first]]))[0, -1].float(), -1)
    counts = torch.zeros(120)
    n = 600
    g = torch.Generator().manual_seed(0)
    hits = 0
    for _ in range(n):
        st = speculative_generate(target, draft, prompt, 2, k=2, temperature=1.0, generator=g, adaptive=False)
        if st.tokens[0] == first:
            counts[st.tokens[1]] += 1
            hits += 1
    emp = counts / max(hits, 1)
    assert hits > 20
    tv = 0.5 * (emp - p1).abs().sum()
    assert float(tv) < 0.5 * (120 / hits) ** 0.5 + 0.15          # total variation within sampling noise
