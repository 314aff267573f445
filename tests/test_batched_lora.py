"""Several LoRA adapters in one batch: the grouped low-rank products against a per-row loop, whole-model generation
with per-request adapters against models that have one adapter merged, and the serving engine mixing adapters."""
import os

import pytest
import torch

from pmetal_b200.lora.batched import NO_ADAPTER, AdapterSet, BatchedLoraAdapters, batched_lora_delta, batched_lora_linear


def _store(n=3, k=32, segs=(16, 8, 8), r=4, seed=0):
    g = torch.Generator().manual_seed(seed)
    st = BatchedLoraAdapters(n, k, segs, r, torch.float32)
    facs = []
    for i in range(n):
        a = torch.randn(len(segs) * r, k, generator=g) * 0.3
        b = torch.randn(sum(segs), r, generator=g) * 0.3
        st.load_adapter(i, a, b, 0.5 + i)
        facs.append((a, b, 0.5 + i))
    return st, facs


def test_rows_pick_their_adapter():
    st, facs = _store()
    g = torch.Generator().manual_seed(1)
    x = torch.randn(11, 32, generator=g)
    ids = torch.tensor([0, 2, NO_ADAPTER, 1, 1, 0, 2, 2, NO_ADAPTER, 0, 1])
    w = torch.randn(32, 32, generator=g) * 0.2
    res = torch.randn(11, 32, generator=g)
    y = batched_lora_linear(x, w, st, ids, res)
    for t in range(11):
        ref = x[t] @ w.t() + res[t]
        if ids[t] >= 0:
            a, b, sc = facs[int(ids[t])]
            o = 0
            for s, sz in enumerate(st.seg_sizes):
                ref[o:o + sz] += sc * (b[o:o + sz] @ (a[s * 4:(s + 1) * 4] @ x[t]))
                o += sz
        assert torch.allclose(y[t], ref, atol=1e-5), t
    assert float(batched_lora_delta(x[:2], torch.tensor([NO_ADAPTER, NO_ADAPTER]), st).abs().max()) == 0.0
    with pytest.raises(IndexError):
        st.load_adapter(3, facs[0][0], facs[0][1], 1.0)
    with pytest.raises(ValueError):
        st.load_adapter(0, facs[0][0][:, :8], facs[0][1], 1.0)
    st.unload_adapter(1)
    assert float(batched_lora_delta(x[3:5], ids[3:5], st).abs().max()) == 0.0


def _tiny():
    from pmetal_b200.models.config import ModelArgs
    from pmetal_b200.models.decoder import DecoderLM
    cfg = ModelArgs(vocab_size=97, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=8)
    m = DecoderLM(cfg).init_weights(0.2, 0).eval()
    for p in m.parameters():
        p.requires_grad_(False)
    return m


def _adapter_dir(tmp_path, name, seed):
    """A trained-looking adapter written in the adapter file format."""
    from pmetal_b200.core.config import LoraConfig
    from pmetal_b200.lora import apply_lora
    from pmetal_b200.lora.adapter import save_adapter
    m = _tiny()
    cfg = LoraConfig(r=4, alpha=8.0, target_modules=["q_proj", "v_proj", "o_proj", "down_proj"])
    apply_lora(m, cfg, seed=seed)
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for _, _, fl in m.fused_linears():
            if fl.lora_b is not None:
                fl.lora_b.copy_(torch.randn(fl.lora_b.shape, generator=g) * 0.3)
    d = str(tmp_path / name)
    save_adapter(m, d, cfg)
    return d, m


def test_generation_with_per_request_adapters_matches_single_adapter_models(tmp_path):
    from pmetal_b200.models.generation import Generator
    from pmetal_b200.models.sampling import SamplingParams
    from pmetal_b200.serve.engine import ContinuousBatchEngine, Request
    d1, m1 = _adapter_dir(tmp_path, "alpha", 1)
    d2, m2 = _adapter_dir(tmp_path, "beta", 2)
    base = _tiny()
    prompts = [[5, 9, 11, 3, 60], list(range(1, 30)), [7, 7, 8]]
    want = {}
    for name, m in (("alpha", m1), ("beta", m2), (None, base)):
        want[name] = Generator(m, num_blocks=32).generate(prompts, SamplingParams.greedy(8)).tokens
    assert want["alpha"] != want[None] and want["alpha"] != want["beta"]      # the adapters do change the output
    model = _tiny()
    ads = AdapterSet(model, 4, 4)
    assert ads.load("alpha", d1) == 0 and ads.load("beta", d2) == 1
    with pytest.raises(KeyError):
        ads.index("gamma")
    eng = ContinuousBatchEngine(model, num_blocks=64, max_slots=8, adapters=ads)
    reqs = []
    for name in ("alpha", None, "beta"):
        for p in prompts:
            reqs.append((name, eng.submit(Request(list(p), SamplingParams.greedy(8), adapter=name))))
    while not all(r.done.is_set() for _, r in reqs):
        eng.tick()
    for i, (name, r) in enumerate(reqs):
        assert r.output == want[name][i % 3], (name, i)
    with pytest.raises(KeyError):
        eng.submit(Request([1, 2], SamplingParams.greedy(2), adapter="gamma"))
    ads.unload("beta")
    assert ads.names[1] is None and ads.load("beta2", d2) == 1
