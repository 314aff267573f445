"""MLX-layout affine group quantisation: packing, round trip, edge exactness, bit allocation, checkpoint round trip."""
import json

import pytest
import torch

from pmetal_b200.quant import mlx_affine as Q


@pytest.mark.parametrize("bits", [2, 3, 4, 6, 8])
def test_pack_unpack_and_round_trip(bits):
    torch.manual_seed(bits)
    q = torch.randint(0, 1 << bits, (5, 128))
    p = Q.pack_bits(q, bits)
    assert p.dtype == torch.int32 and p.shape == (5, 128 * bits // 32)
    assert torch.equal(Q.unpack_bits(p, bits, 128), q)
    if bits == 4:                                      # eight nibbles per word, first element in the low nibble
        assert int(p[0, 0]) & 0xF == int(q[0, 0]) and (int(p[0, 0]) >> 4) & 0xF == int(q[0, 1])
    w = torch.randn(16, 128)
    packed, s, b = Q.quantize_affine(w, bits, 64)
    assert s.dtype == torch.float16 and s.shape == (16, 2) == b.shape
    r = Q.dequantize_affine(packed, s, b, bits, 64)
    step = (w.reshape(16, 2, 64).amax(-1) - w.reshape(16, 2, 64).amin(-1)) / ((1 << bits) - 1)
    assert ((r - w).abs().reshape(16, 2, 64).amax(-1) <= 1.01 * step + 2e-3).all()       # re-derived scale: < one step
    # the edge of every group (largest magnitude end of its range) is reproduced up to the fp16 rounding of the scale
    g = w.reshape(16, 2, 64)
    edge = torch.where(g.amin(-1).abs() > g.amax(-1).abs(), g.amin(-1), g.amax(-1))
    pos = (g - edge[..., None]).abs().argmin(-1)
    got = r.reshape(16, 2, 64).gather(-1, pos[..., None]).squeeze(-1)
    assert torch.allclose(got, edge, rtol=2e-3, atol=2e-3)


def test_scores_fall_with_bits_and_quantized_matmul():
    torch.manual_seed(0)
    w = torch.randn(64, 256) * 0.05
    scores = [Q.reconstruction_score(w, b, 64) for b in (2, 3, 4, 6, 8)]
    assert all(a > b for a, b in zip(scores, scores[1:])) and scores[-1] < 0.02
    x = torch.randn(3, 256)
    p, s, b = Q.quantize_affine(w, 8, 64)
    y = Q.quantized_matmul(x, p, s, b, 8, 64)
    assert torch.allclose(y, x @ w.t(), atol=0.02)
    with pytest.raises(ValueError):
        Q.quantize_affine(torch.randn(4, 100), 4, 64)


def test_critical_tensors_and_allocation():
    for name in ("model.norm.weight", "model.layers.0.input_layernorm.weight", "model.layers.3.self_attn.q_norm.weight",
                 "model.layers.1.mlp.gate.weight", "model.layers.1.mlp.experts.3.up_proj.weight", "lm_head.weight",
                 "model.layers.0.linear_attn.A_log", "model.layers.0.linear_attn.conv1d.weight"):
        assert Q.is_critical_tensor(name), name
    for name in ("model.layers.0.self_attn.q_proj.weight", "model.layers.0.mlp.gate_proj.weight"):
        assert not Q.is_critical_tensor(name), name
    torch.manual_seed(1)
    sd = {"model.embed_tokens.weight": torch.randn(64, 128), "model.layers.0.self_attn.q_proj.weight": torch.randn(128, 128),
          "model.layers.0.mlp.down_proj.weight": torch.randn(128, 256) * torch.linspace(0.1, 3, 256),   # harder to quantise
          "model.layers.0.input_layernorm.weight": torch.ones(128)}
    scores = Q.evaluate_tensor_quality(sd, 64)
    assert [len(s) for _, _, s in scores] == [5, 5, 5, 0]
    low = {t.name: t.bits for t in Q.allocate_bits_for_bpw(scores, 2.0, 64)}
    assert low["model.embed_tokens.weight"] == 8 and low["model.layers.0.self_attn.q_proj.weight"] == 2
    mid = {t.name: t.bits for t in Q.allocate_bits_for_bpw(scores, 5.0, 64)}
    assert mid["model.layers.0.mlp.down_proj.weight"] >= mid["model.layers.0.self_attn.q_proj.weight"] > 2
    high = {t.name: t.bits for t in Q.allocate_bits_for_bpw(scores, 16.0, 64)}
    assert set(high.values()) == {8}


def test_checkpoint_round_trip(tmp_path):
    from pmetal_b200.models.config import preset
    from pmetal_b200.models.decoder import DecoderLM
    from pmetal_b200.utils.safetensors_io import load_file, save_file
    cfg = preset("tiny-qwen3")
    m = DecoderLM(cfg).init_weights(0.05, 0)
    src = tmp_path / "src"
    src.mkdir()
    save_file({k: v.contiguous() for k, v in m.hf_state_dict().items()}, str(src / "model.safetensors"))
    (src / "config.json").write_text(json.dumps(cfg.to_hf_dict()))
    rep = Q.quantize_model(str(src), str(tmp_path / "q"), target_bpw=5.0)
    assert 4.0 < rep["effective_bpw"] < 9.0 and rep["tensors"] > 0
    qcfg = json.loads((tmp_path / "q" / "config.json").read_text())["quantization"]
    assert qcfg["group_size"] == 64 and "bits" in qcfg
    qsd = load_file(str(tmp_path / "q" / "model.safetensors"))
    assert "model.layers.0.self_attn.q_proj.scales" in qsd and qsd["model.layers.0.self_attn.q_proj.weight"].dtype == torch.int32
    dense = Q.load_quantized_state_dict(qsd, qcfg, torch.float32)
    ref = m.hf_state_dict()
    assert set(dense) == set(ref)
    w, r = ref["model.layers.0.mlp.down_proj.weight"].float(), dense["model.layers.0.mlp.down_proj.weight"]
    assert float((w - r).norm() / w.norm()) < 0.2
    assert torch.equal(dense["model.layers.0.input_layernorm.weight"], ref["model.layers.0.input_layernorm.weight"])
    # the model loader expands such a checkpoint on the fly
    from pmetal_b200.models.loader import load_pretrained
    m2, _, _ = load_pretrained(str(tmp_path / "q"), dtype=torch.float32)
    ids = torch.randint(0, cfg.vocab_size, (1, 12), generator=torch.Generator().manual_seed(3))
    m3 = DecoderLM(cfg)
    m3.load_hf_state_dict(dense)                      # the same dequantised weights, loaded explicitly
    with torch.no_grad():
        a, b, c = m(ids[0]), m2(ids[0]), m3(ids[0])
    assert torch.allclose(b, c, atol=1e-5)
    assert torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0) > 0.8


def test_gather_qmm_matches_per_row_dense_products():
    import torch
    from pmetal_b200.quant.mlx_affine import dequantize_affine, gather_qmm, quantize_affine
    torch.manual_seed(0)
    E, N, K, R = 5, 24, 128, 17
    w = torch.randn(E, N, K)
    packed, scales, biases = quantize_affine(w, 4, 64)
    x = torch.randn(R, K)
    idx = torch.tensor([4, 0, 0, 3, 1, 4, 4, 2, 0, 1, 3, 3, 2, 0, 4, 1, 2])
    got = gather_qmm(x, packed, scales, biases, idx, 4, 64)
    dense = dequantize_affine(packed, scales, biases, 4, 64)
    want = torch.stack([x[i] @ dense[idx[i]].t() for i in range(R)])
    assert got.shape == (R, N) and torch.allclose(got, want, atol=1e-4)
    assert (dense - w).abs().max() < 0.6                          # 4-bit groups of 64 on N(0,1) data
