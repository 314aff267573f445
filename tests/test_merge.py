import json
import os

import pytest
import torch

from pmetal_b200.merge import methods as M
from pmetal_b200.merge.merge import MergeConfig, merge_lora_into_base, run_merge
from pmetal_b200.utils import safetensors_io as st


def test_sparsify_and_consensus():
    t = torch.tensor([0.1, -0.5, 0.3, -0.05, 0.9, 0.0, -0.2, 0.4, 0.6, -0.7])
    s = M.sparsify_by_magnitude(t, 0.3)
    assert (s != 0).sum() == 3 and set(s.nonzero().flatten().tolist()) == {4, 8, 9}
    assert torch.equal(M.sparsify_by_magnitude(t, 1.0), t) and M.sparsify_by_magnitude(t, 0.0).abs().sum() == 0
    a, b, c = torch.tensor([1.0, -1.0, 2.0]), torch.tensor([2.0, 1.0, -1.0]), torch.tensor([3.0, -2.0, -1.0])
    out = M.sign_consensus([a, b, c], [1.0, 1.0, 1.0])
    assert out.tolist() == [6.0, -3.0, -2.0]


def test_basic_methods():
    a, b = torch.tensor([1.0, 0.0]), torch.tensor([0.0, 1.0])
    assert torch.allclose(M.linear([a, b], [1.0, 3.0]), torch.tensor([0.25, 0.75]))
    s = M.slerp(a, b, 0.5)
    assert torch.allclose(s, torch.tensor([0.5 ** 0.5, 0.5 ** 0.5]), atol=1e-6)
    assert torch.allclose(M.slerp(a, a * 2, 0.25), 1.25 * a)                 # colinear -> lerp
    base = torch.zeros(4)
    m1, m2 = torch.tensor([1.0, 2.0, 0.0, -1.0]), torch.tensor([1.0, -2.0, 3.0, 0.0])
    assert torch.allclose(M.task_arithmetic([m1, m2], base, [1, 1], 0.5), torch.tensor([1.0, 0.0, 1.5, -0.5]))
    t = M.ties([m1, m2], base, [1.0, 1.0], [1.0, 1.0], 1.0)
    assert t.tolist() == [2.0, 0.0, 3.0, -1.0]                               # tied sign at index 1 -> dropped
    assert torch.allclose(M.nearswap([m1, m2], base), torch.tensor([1.0, 2.0, 0.0, 0.0]))
    d = M.dare([m1], base, [1.0], [0.5], seed=0)
    assert set(d.tolist()) <= {0.0, 2.0, 4.0, -2.0, -0.0}
    big = torch.randn(2000)
    dd = M.dare([big], torch.zeros(2000), [1.0], [0.3], seed=1)
    assert abs((dd != 0).float().mean().item() - 0.3) < 0.05 and abs(dd.sum().item() - big.sum().item()) < 300
    de = M.della([big.view(20, 100)], torch.zeros(20, 100), [1.0], [0.5], seed=2)
    kept = de != 0
    mags = big.view(20, 100).abs()
    assert mags[kept].mean() > mags[~kept].mean()                              # large magnitudes survive more often
    bc = M.breadcrumbs([big], torch.zeros(2000), [1.0], top_p=0.9, bottom_p=0.2)
    assert abs((bc != 0).float().mean().item() - 0.7) < 0.02
    ms = M.model_stock([m1, m1 * 1.0], base)
    assert torch.allclose(ms, m1)
    f = M.fisher([a, b], [torch.tensor([3.0, 1.0]), torch.tensor([1.0, 1.0])])
    assert torch.allclose(f, torch.tensor([0.75, 0.5]), atol=1e-6)
    W = torch.randn(3, 4)
    G = torch.randn(10, 4); G = G.t() @ G
    assert torch.allclose(M.regmean([W, W], [G, G], 1.0), W, atol=1e-3)
    assert torch.allclose(M.multislerp([a, b], [1, 1]), torch.tensor([0.5 ** 0.5, 0.5 ** 0.5]), atol=1e-6)
    r = M.ram([m1, m2], base, [1.0, 1.0])
    assert abs(r.norm().item() - (m1.norm() + m2.norm()).item() / 2) < 1e-5


def _ckpt(d, seed, layers=2):
    os.makedirs(d, exist_ok=True)
    g = torch.Generator().manual_seed(seed)
    t = {"model.embed_tokens.weight": torch.randn(8, 4, generator=g), "model.norm.weight": torch.ones(4)}
    for i in range(layers):
        t[f"model.layers.{i}.self_attn.q_proj.weight"] = torch.randn(4, 4, generator=g)
    st.save_file(t, os.path.join(d, "model.safetensors"))
    json.dump({"num_hidden_layers": layers, "model_type": "llama"}, open(os.path.join(d, "config.json"), "w"))
    return t


def test_run_merge_yaml_and_slices(tmp_path):
    a, b, base = (_ckpt(str(tmp_path / n), s) for n, s in (("a", 1), ("b", 2), ("base", 3)))
    cfg = MergeConfig.from_dict({
        "merge_method": "ties", "base_model": str(tmp_path / "base"), "dtype": "float32",
        "output_path": str(tmp_path / "out"), "parameters": {"lambda": 1.0, "density": 0.5},
        "models": [{"model": str(tmp_path / "a"), "parameters": {"weight": 0.7}}, {"model": str(tmp_path / "b")}]})
    assert cfg.models[0].parameters.weight == 0.7 and cfg.models[1].parameters.density == 0.5
    res = run_merge(cfg, "cpu")
    out = st.load_file(str(tmp_path / "out" / "model.safetensors"))
    n = "model.layers.0.self_attn.q_proj.weight"
    exp = M.ties([a[n], b[n]], base[n], [0.7, 1.0], [0.5, 0.5], 1.0)
    assert torch.allclose(out[n], exp) and res["tensors"] == 4
    assert os.path.exists(tmp_path / "out" / "model.safetensors.index.json")
    with pytest.raises(ValueError):
        run_merge(MergeConfig.from_dict({"merge_method": "ties", "models": [{"model": str(tmp_path / "a")}],
                                         "output_path": str(tmp_path / "x")}), "cpu")
    sl = MergeConfig.from_dict({"merge_method": "passthrough", "dtype": "float32", "output_path": str(tmp_path / "s"),
                                "slices": [{"sources": [{"model": str(tmp_path / "a"), "layer_range": [0, 2]}]},
                                           {"sources": [{"model": str(tmp_path / "b"), "layer_range": [1, 2]}]}]})
    r = run_merge(sl, "cpu")
    so = st.load_file(str(tmp_path / "s" / "model.safetensors"))
    assert r["num_layers"] == 3 and torch.equal(so["model.layers.2.self_attn.q_proj.weight"], b["model.layers.1.self_attn.q_proj.weight"])
    assert json.load(open(tmp_path / "s" / "config.json"))["num_hidden_layers"] == 3


def test_fuse_lora_into_base(tmp_path):
    base = _ckpt(str(tmp_path / "base"), 5)
    ad = tmp_path / "ad"
    os.makedirs(ad)
    A, B = torch.randn(2, 4), torch.randn(4, 2)
    st.save_file({"layers.0.self_attn.q_proj.lora_a": A, "layers.0.self_attn.q_proj.lora_b": B,
                  "layers.1.self_attn.q_proj.lora_a": torch.zeros(1, 4), "layers.1.self_attn.q_proj.lora_b": torch.zeros(4, 1)},
                 str(ad / "lora_weights.safetensors"))
    json.dump({"r": 2, "alpha": 4.0, "target_modules": ["q_proj"], "use_rslora": False}, open(ad / "adapter_config.json", "w"))
    res = merge_lora_into_base(str(tmp_path / "base"), str(ad), str(tmp_path / "fused"), "float32")
    out = st.load_file(str(tmp_path / "fused" / "model.safetensors"))
    n0, n1 = "model.layers.0.self_attn.q_proj.weight", "model.layers.1.self_attn.q_proj.weight"
    assert res["fused_projections"] == 1
    assert torch.allclose(out[n0], base[n0] + 2.0 * (B @ A), atol=1e-6) and torch.equal(out[n1], base[n1])
