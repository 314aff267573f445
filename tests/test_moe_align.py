"""Expert alignment before merging mixture-of-experts checkpoints."""
import json
import os

import pytest
import torch

from pmetal_b200.merge.merge import LazyCheckpoint, MergeConfig, run_merge
from pmetal_b200.merge.moe_align import align_experts, expert_layers, hungarian_max
from pmetal_b200.utils.safetensors_io import load_file, save_file


def test_hungarian_finds_the_best_assignment():
    import itertools
    g = torch.Generator().manual_seed(0)
    for n in (1, 2, 5, 7):
        w = torch.rand(n, n, generator=g)
        got = hungarian_max(w)
        best = max(itertools.permutations(range(n)), key=lambda p: sum(float(w[i, p[i]]) for i in range(n)))
        assert sorted(got) == list(range(n))
        assert abs(sum(float(w[i, got[i]]) for i in range(n)) - sum(float(w[i, best[i]]) for i in range(n))) < 1e-9
    perm = [3, 0, 2, 1]
    assert hungarian_max(torch.eye(4)[perm]) == perm


def _moe_state(seed: int, experts: int = 4, stacked: bool = False):
    g = torch.Generator().manual_seed(seed)
    sd = {"model.embed_tokens.weight": torch.randn(16, 8, generator=g)}
    for layer in range(2):
        pre = f"model.layers.{layer}.mlp"
        sd[f"{pre}.gate.weight"] = torch.randn(experts, 8, generator=g)
        if stacked:
            sd[f"{pre}.experts.gate_up_proj"] = torch.randn(experts, 12, 8, generator=g)
            sd[f"{pre}.experts.down_proj"] = torch.randn(experts, 8, 6, generator=g)
        else:
            for e in range(experts):
                for part, shape in (("gate_proj", (6, 8)), ("up_proj", (6, 8)), ("down_proj", (8, 6))):
                    sd[f"{pre}.experts.{e}.{part}.weight"] = torch.randn(*shape, generator=g)
    return sd


def _permuted(sd, perms, stacked):
    """The same model with its experts stored in another order: new position j holds old expert perms[layer][j]."""
    out = dict(sd)
    for layer, p in perms.items():
        pre = f"model.layers.{layer}.mlp"
        out[f"{pre}.gate.weight"] = sd[f"{pre}.gate.weight"][p]
        if stacked:
            for part in ("gate_up_proj", "down_proj"):
                out[f"{pre}.experts.{part}"] = sd[f"{pre}.experts.{part}"][p]
        else:
            for j, src in enumerate(p):
                for part in ("gate_proj", "up_proj", "down_proj"):
                    out[f"{pre}.experts.{j}.{part}.weight"] = sd[f"{pre}.experts.{src}.{part}.weight"]
    return out


@pytest.mark.parametrize("stacked", [False, True])
def test_alignment_undoes_an_expert_shuffle_before_merging(tmp_path, stacked):
    base = _moe_state(0, stacked=stacked)
    tuned = {k: v + 0.01 * torch.randn(v.shape, generator=torch.Generator().manual_seed(5)) for k, v in base.items()}
    shuffle = {0: [2, 0, 3, 1], 1: [1, 3, 0, 2]}
    for name, sd in (("a", base), ("b", _permuted(tuned, shuffle, stacked))):
        os.makedirs(tmp_path / name)
        save_file({k: v.contiguous() for k, v in sd.items()}, str(tmp_path / name / "model.safetensors"))
        (tmp_path / name / "config.json").write_text(json.dumps({"model_type": "qwen3_moe"}))
    cks = [LazyCheckpoint(str(tmp_path / "a")), LazyCheckpoint(str(tmp_path / "b"))]
    assert set(expert_layers(cks[0].keys())) == {0, 1}
    al = align_experts(cks)
    inverse = {l: [p.index(i) for i in range(4)] for l, p in shuffle.items()}
    assert al.perms[0] == {0: [0, 1, 2, 3], 1: [0, 1, 2, 3]} and al.perms[1] == inverse and not al.is_identity()

    def merged(align):
        cfg = MergeConfig.from_dict({"merge_method": "linear", "dtype": "float32", "align_moe_experts": align,
                                     "models": [{"model": str(tmp_path / n), "parameters": {"weight": 0.5}} for n in "ab"]})
        cfg.output_path = str(tmp_path / f"out{int(align)}")
        rep = run_merge(cfg, "cpu")
        return rep, load_file(os.path.join(cfg.output_path, "model.safetensors"))
    rep, good = merged(True)
    assert rep["expert_alignment"] == {"layers": 2, "identity": False}
    want = {k: 0.5 * (base[k] + tuned[k]) for k in base}
    assert all(torch.allclose(good[k], want[k], atol=1e-6) for k in want)        # experts and router rows line up again
    _, bad = merged(False)
    key = "model.layers.0.mlp.experts.gate_up_proj" if stacked else "model.layers.0.mlp.experts.0.gate_proj.weight"
    assert not torch.allclose(bad[key], want[key], atol=1e-3)


def test_dense_models_need_no_alignment(tmp_path):
    os.makedirs(tmp_path / "d")
    save_file({"model.layers.0.mlp.gate_proj.weight": torch.randn(4, 4)}, str(tmp_path / "d" / "model.safetensors"))
    assert align_experts([LazyCheckpoint(str(tmp_path / "d"))]) is None


def test_merge_sanity_levels(tmp_path):
    from pmetal_b200.merge.sanity import check_tensor
    assert check_tensor("x", torch.ones(3), "off") is None
    q = check_tensor("x", torch.tensor([0.0, 1.0, -3.0, 0.0]), "quick")
    assert (q.n_elements, q.n_nan, q.n_inf, q.mean) == (4, 0, 0, None)
    f = check_tensor("x", torch.tensor([0.0, 1.0, -3.0, 0.0]), "full")
    assert f.abs_max == 3.0 and f.sparsity == 0.5 and abs(f.mean + 0.5) < 1e-6 and not f.is_outlier()
    assert check_tensor("big", torch.full((4,), 50.0), "full").is_outlier()
    for bad in (float("nan"), float("inf")):
        with pytest.raises(ValueError):
            check_tensor("x", torch.tensor([1.0, bad]), "quick")
    for name, scale in (("a", 1.0), ("b", 200.0)):
        os.makedirs(tmp_path / name)
        save_file({"model.layers.0.mlp.down_proj.weight": torch.full((4, 4), scale)}, str(tmp_path / name / "model.safetensors"))
        (tmp_path / name / "config.json").write_text("{}")
    cfg = MergeConfig.from_dict({"merge_method": "linear", "dtype": "float32", "sanity": "full",
                                 "models": [{"model": str(tmp_path / n), "parameters": {"weight": 0.5}} for n in "ab"]})
    cfg.output_path = str(tmp_path / "o")
    rep = run_merge(cfg, "cpu")
    assert rep["outliers"][0]["name"].endswith("down_proj.weight") and len(rep["tensor_reports"]) == 1
