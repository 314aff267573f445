import json
import os

import torch

from pmetal_b200.core.config import LoraConfig, TrainingConfig
from pmetal_b200.lora import apply_lora, load_adapter, lora_state_dict, save_adapter
from pmetal_b200.lora.adapter import infer_rank_from_file, load_adapter_config, merge_adapter_into_base
from pmetal_b200.models.config import preset
from pmetal_b200.models.decoder import DecoderLM
from pmetal_b200.ops import reference as ref
from pmetal_b200.trainer.checkpoint import CheckpointManager
from pmetal_b200.trainer.loop import TrainingLoop
from pmetal_b200.trainer.optimizer import FlatAdamW, classify_param
from pmetal_b200.utils import safetensors_io as st


def _tiny(seed=0):
    m = DecoderLM(preset("tiny-qwen3")).init_weights(0.02, seed)
    return m


def test_safetensors_roundtrip_and_interop(tmp_path):
    t = {"b": torch.randn(3, 4), "a": torch.arange(6, dtype=torch.int32).view(2, 3),
         "c": torch.randn(5).to(torch.bfloat16)}
    p = str(tmp_path / "x.safetensors")
    st.save_file(t, p, metadata={"format": "mlx"})
    back = st.load_file(p)
    assert all(torch.equal(back[k], t[k]) for k in t)
    assert st.load_metadata(p) == {"format": "mlx"}
    hdr, base = st.read_header(p)
    assert base % 8 == 0 and hdr["a"]["data_offsets"][0] == 0
    try:
        from safetensors.torch import load_file, save_file
    except ImportError:
        return
    other = load_file(p)
    assert all(torch.equal(other[k], t[k]) for k in t)
    q = str(tmp_path / "y.safetensors")
    save_file({k: v.contiguous() for k, v in t.items()}, q)
    again = st.load_file(q)
    assert all(torch.equal(again[k], t[k]) for k in t)


def test_adapter_file_contract(tmp_path):
    m = _tiny()
    cfg = LoraConfig(r=8, alpha=16)
    apply_lora(m, cfg)
    d = str(tmp_path / "out")
    save_adapter(m, d, cfg, base_model="base")
    sd = st.load_file(os.path.join(d, "lora_weights.safetensors"))
    assert len(sd) == 2 * 7 * 2
    assert sd["layers.0.self_attn.q_proj.lora_a"].shape == (8, 256)
    assert sd["layers.0.self_attn.q_proj.lora_b"].shape == (256, 8)
    assert sd["layers.1.self_attn.k_proj.lora_b"].shape == (128, 8)
    assert sd["layers.0.mlp.gate_proj.lora_a"].shape == (1, 256)      # rank-0 placeholder
    assert sd["layers.0.mlp.down_proj.lora_b"].shape == (256, 1)
    assert all(v.dtype == torch.float32 for v in sd.values())
    assert not any(k.startswith("model.") for k in sd)
    ac = json.load(open(os.path.join(d, "adapter_config.json")))
    assert ac == {"r": 8, "alpha": 16, "target_modules": ["q_proj", "k_proj", "v_proj", "o_proj"],
                  "use_rslora": False, "base_model": "base"}
    assert infer_rank_from_file(d) == 8 and load_adapter_config(d).r == 8
    # B starts at zero, A within +-sqrt(3/in)
    a = sd["layers.0.self_attn.q_proj.lora_a"]
    assert sd["layers.0.self_attn.q_proj.lora_b"].abs().max() == 0 and a.abs().max() <= (3 / 256) ** 0.5
    m2 = _tiny()
    apply_lora(m2, cfg, seed=7)
    assert load_adapter(m2, d) == 2 * 4 * 2
    assert all(torch.equal(v, lora_state_dict(m2)[k]) for k, v in sd.items())


def test_lora_forward_equals_merged_weights():
    m = _tiny()
    apply_lora(m, LoraConfig(r=4, alpha=8, target_modules=["q_proj", "v_proj", "down_proj"]))
    with torch.no_grad():
        for _, _, fl in m.fused_linears():
            if fl.lora_b is not None:
                fl.lora_b.normal_(0, 0.1)
    ids = torch.randint(0, 1024, (2, 17))
    out = m(ids)
    merge_adapter_into_base(m)
    assert torch.allclose(out, m(ids), atol=1e-4)


def test_packed_equals_separate_documents():
    m = _tiny()
    g = torch.Generator().manual_seed(0)
    a, b = torch.randint(0, 1024, (9,), generator=g), torch.randint(0, 1024, (14,), generator=g)
    packed = m(torch.cat([a, b]), cu_seqlens=torch.tensor([0, 9, 23], dtype=torch.int32))
    assert torch.allclose(packed[:9], m(a[None])[0], atol=1e-4)
    assert torch.allclose(packed[9:], m(b[None])[0], atol=1e-4)


def test_adamw_reference_semantics():
    p = torch.tensor([1.0, -2.0]); g = torch.tensor([0.5, 0.25])
    m = torch.zeros(2); v = torch.zeros(2)
    ref.adamw_step(p, g, m, v, 1, 0.1, 0.9, 0.999, 1e-8, 0.01)
    # step 1: m_hat = g, v_hat = g^2 -> p - lr*sign(g), then decay on the updated value
    exp = torch.tensor([1.0 - 0.1, -2.0 - 0.1])
    exp = exp - 0.01 * 0.1 * exp
    assert torch.allclose(p, exp, atol=1e-6)
    assert classify_param("layers.0.self_attn.q_proj.lora_b") == "lora_b"
    assert classify_param("model.norm.weight") == "no_decay" and classify_param("embed_tokens") == "embedding"
    assert classify_param("layers.0.mlp.up_proj.lora_a") == "regular"


def test_flat_adamw_matches_per_tensor(tmp_path):
    torch.manual_seed(0)
    ps = [("x.lora_a", torch.nn.Parameter(torch.randn(5, 7))), ("x.lora_b", torch.nn.Parameter(torch.randn(3, 5))),
          ("n.norm", torch.nn.Parameter(torch.randn(11)))]
    copies = [p.detach().clone() for _, p in ps]
    opt = FlatAdamW(ps, lr=1e-2, weight_decay=0.1, loraplus_ratio=4.0, max_grad_norm=0.0)
    ms = [torch.zeros_like(c) for c in copies]; vs = [torch.zeros_like(c) for c in copies]
    for step in (1, 2, 3):
        opt.zero_grad()
        gs = [torch.randn_like(c) for c in copies]
        for (_, p), g in zip(ps, gs):
            p.grad.copy_(g)
        opt.step()
        for c, g, m, v, (lr, wd) in zip(copies, gs, ms, vs, [(1e-2, 0.1), (4e-2, 0.1), (1e-2, 0.0)]):
            ref.adamw_step(c, g, m, v, step, lr, 0.9, 0.999, 1e-8, wd)
    for (_, p), c in zip(ps, copies):
        assert torch.allclose(p.detach(), c, atol=1e-6)


def test_flat_adamw_without_bias_correction():
    """The plain variant uses the running moments as they are: after one step m = (1 - b1) g and v = (1 - b2) g^2."""
    torch.manual_seed(1)
    p = torch.nn.Parameter(torch.randn(6, 5))
    start = p.detach().clone()
    opt = FlatAdamW([("x.lora_a", p)], lr=1e-2, weight_decay=0.0, max_grad_norm=0.0, bias_correction=False)
    g = torch.randn(6, 5)
    p.grad.copy_(g)
    opt.step()
    want = start - 1e-2 * (0.1 * g) / ((0.001 * g * g).sqrt() + 1e-8)
    assert torch.allclose(p.detach(), want, atol=1e-6)
    m, v = torch.zeros(2), torch.zeros(2)
    q = torch.tensor([1.0, -1.0])
    ref.adamw_step(q, torch.tensor([0.5, 0.5]), m, v, 0, 0.1, 0.9, 0.999, 1e-8, 0.0)
    assert torch.allclose(q, torch.tensor([1.0, -1.0]) - 0.1 * 0.05 / (0.00025 ** 0.5 + 1e-8), atol=1e-6)


def test_grad_clip_and_accumulation():
    m = _tiny(); apply_lora(m, LoraConfig(r=4, alpha=8))
    loop = TrainingLoop(m, TrainingConfig(gradient_accumulation_steps=2, warmup_steps=0, max_grad_norm=1e-3,
                                          lr_scheduler="constant", learning_rate=1e-2))
    ids = torch.randint(0, 1024, (2, 16))
    l1, g1 = loop.train_step({"input_ids": ids, "labels": ids})
    assert g1 is None and loop.state.step == 0
    l2, g2 = loop.train_step({"input_ids": ids, "labels": ids})
    assert g2 is not None and loop.state.step == 1


def test_config1_tiny_sft_loss_decreases_and_checkpoint(tmp_path):
    m = _tiny(); cfg = LoraConfig(r=8, alpha=16); apply_lora(m, cfg)
    ck = CheckpointManager(str(tmp_path / "checkpoints"), keep=2, async_write=True)
    loop = TrainingLoop(m, TrainingConfig(gradient_accumulation_steps=1, warmup_steps=0, lr_scheduler="constant",
                                          learning_rate=2e-4, save_steps=5), checkpoint_manager=ck)
    ids = torch.randint(0, 1024, (4, 128), generator=torch.Generator().manual_seed(1))
    losses = []
    for i in range(20):
        loss, _ = loop.train_step({"input_ids": ids, "labels": ids})
        losses.append(float(loss))
        if loop.state.step % 5 == 0:
            loop.save_checkpoint()
    ck.wait()
    assert losses[-1] < losses[0] - 0.05
    steps = sorted(d for d in os.listdir(ck.dir) if d.startswith("step_"))
    assert steps == ["step_15", "step_20"] and open(os.path.join(ck.dir, "latest")).read() == "step_20"
    meta = json.load(open(os.path.join(ck.dir, "step_20", "metadata.json")))
    assert meta["step"] == 20 and set(meta) >= {"epoch", "running_loss", "learning_rate", "seed", "timestamp"}
    m2 = _tiny(); apply_lora(m2, cfg, seed=3)
    loop2 = TrainingLoop(m2, TrainingConfig(gradient_accumulation_steps=1, warmup_steps=0))
    loop2.resume(ck.latest_path())
    assert loop2.state.step == 20
    a, b = lora_state_dict(m), lora_state_dict(m2)
    assert all(torch.equal(a[k], b[k]) for k in a)
    save_adapter(m, str(tmp_path / "final"), cfg)


def test_dora_row_norms_without_the_merged_weight_and_their_cache():
    from pmetal_b200.lora.dora import attach_dora, merged_dora_weight, row_norms
    m = _tiny()
    apply_lora(m, LoraConfig(r=8, alpha=16, target_modules=["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj",
                                                            "up_proj", "down_proj"]))
    g = torch.Generator().manual_seed(3)
    with torch.no_grad():
        for _, _, fl in m.fused_linears():
            fl.lora_b.copy_(torch.randn(fl.lora_b.shape, generator=g) * 0.1)
    assert attach_dora(m) == 8
    for _, _, fl in m.fused_linears():
        want = fl.merged_weight().float().norm(dim=1)
        got = row_norms(fl)
        assert torch.allclose(got, want, rtol=1e-4, atol=1e-5)
        assert row_norms(fl) is got                      # unchanged factors: the cached tensor comes back
        with torch.no_grad():
            fl.lora_b.mul_(1.5)                          # an optimizer step bumps the version
        again = row_norms(fl)
        assert again is not got and torch.allclose(again, fl.merged_weight().float().norm(dim=1), rtol=1e-4, atol=1e-5)
    # forward of the decomposed form equals a plain linear with the merged DoRA weight
    fl = m.layers[0].self_attn.qkv_proj
    x = torch.randn(5, fl.in_features, generator=g)
    assert torch.allclose(fl.forward(x), x @ merged_dora_weight(fl).t(), rtol=1e-4, atol=1e-4)
