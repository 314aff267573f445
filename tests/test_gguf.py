"""GGUF: block codecs against plain numpy restatements, file round trips, recipe, imatrix, reader hardening."""
import io
import json
import os
import struct

import numpy as np
import pytest
import torch

from pmetal_b200.gguf import native
from pmetal_b200.gguf.convert import gguf_to_hf_name, hf_to_gguf_name, quantize_model
from pmetal_b200.gguf.imatrix import IMatrix
from pmetal_b200.gguf.reader import GgufError, GgufFile
from pmetal_b200.gguf.recipe import DynamicConfig, DynamicQuantizer, tensor_type, use_more_bits
from pmetal_b200.gguf.types import BLOCK_GEOMETRY, GgmlType, tensor_nbytes
from pmetal_b200.gguf.writer import GgufWriter

T = GgmlType


def _rnd(v):      # round half away from zero, as the quantisers do
    return np.sign(v) * np.floor(np.abs(v) + 0.5)


def _data(n=256 * 12, seed=0, scale=0.05):
    return (np.random.default_rng(seed).standard_normal(n) * scale).astype(np.float32)


def test_q8_0_matches_numpy_restatement():
    x = _data(32 * 7 + 5)                      # ragged tail is zero-padded
    raw = native.quantize(x, T.Q8_0)
    assert raw.size == 8 * 34
    xp = np.concatenate([x, np.zeros(27, np.float32)]).reshape(8, 32)
    amax = np.abs(xp).max(1)
    d = (amax / np.float32(127)).astype(np.float16)
    inv = np.where(amax == 0, 0, np.float32(127) / amax).astype(np.float32)
    q = np.clip(_rnd(xp * inv[:, None]), -127, 127).astype(np.int8)
    blocks = raw.reshape(8, 34)
    assert np.array_equal(blocks[:, :2].copy().view(np.float16).reshape(-1), d)
    assert np.array_equal(blocks[:, 2:].view(np.int8), q)
    y = native.dequantize(raw, T.Q8_0, x.size)
    assert np.allclose(y, (q * d.astype(np.float32)[:, None]).reshape(-1)[:x.size])


def test_q4_0_layout_and_signed_scale():
    x = np.zeros(32, np.float32)
    x[3] = -2.0                                 # largest magnitude is negative -> d = -2 / -8 = 0.25
    x[20] = 1.0
    raw = native.quantize(x, T.Q4_0)
    assert raw[:2].view(np.float16)[0] == np.float16(0.25)
    qs = raw[2:]
    assert qs[3] & 15 == 1                      # round(-2/0.25 + 8.5) = round(0.5) = 1 (half away from zero)
    assert qs[4] >> 4 == 13                     # element 20 sits in the high nibble of byte 4: round(4 + 8.5) = 13
    y = native.dequantize(raw, T.Q4_0, 32)
    assert abs(y[3] - (1 - 8) * 0.25) < 1e-6


@pytest.mark.parametrize("t,tol", [(T.Q4_0, 0.25), (T.Q4_1, 0.12), (T.Q5_0, 0.13), (T.Q5_1, 0.06), (T.Q8_0, 0.01),
                                   (T.Q8_1, 0.01), (T.Q2K, 0.40), (T.Q3K, 0.22), (T.Q4K, 0.11), (T.Q5K, 0.06),
                                   (T.Q6K, 0.03), (T.Q8K, 0.012), (T.MXFP4, 0.18), (T.F16, 1e-3), (T.BF16, 5e-3)])
def test_round_trip_error(t, tol):
    x = _data()
    raw = native.quantize(x, t)
    assert raw.size == tensor_nbytes(t, x.size)
    y = native.dequantize(raw, t, x.size)
    assert np.linalg.norm(y - x) / np.linalg.norm(x) < tol
    # deterministic and independent of the thread count
    assert np.array_equal(raw, native.quantize(x, t, threads=3))


def test_k_quant_ragged_tail_is_zero_and_constant_block():
    x = _data(256 + 100)
    raw = native.quantize(x, T.Q4K)
    assert raw.size == 2 * 144 and not raw[144:].any()
    const = np.full(256, 0.5, np.float32)       # max == min in every sub-block -> all scales zero
    y = native.dequantize(native.quantize(const, T.Q4K), T.Q4K, 256)
    assert not y.any()
    z = native.dequantize(native.quantize(np.zeros(256, np.float32), T.Q6K), T.Q6K, 256)
    assert not z.any() and np.isfinite(z).all()


def test_q6k_block_fields():
    x = _data(256, seed=3)
    raw = native.quantize(x, T.Q6K)
    sc = raw[192:208].view(np.int8)
    d = raw[208:210].view(np.float16)[0]
    assert np.abs(sc).max() in (127, 128 - 1) or np.abs(sc).max() > 100      # scales use the int8 range
    assert d != 0


def test_iq4_and_unknown_types():
    blk = np.zeros(18, np.uint8)
    blk[:2] = np.frombuffer(np.float16(2.0).tobytes(), np.uint8)
    blk[2] = 0x0F                               # element 0 -> code 15 (113), element 16 -> code 0 (-127)
    y = native.dequantize(blk, T.IQ4_NL, 32)
    assert y[0] == 226.0 and y[16] == -254.0
    with pytest.raises(NotImplementedError):
        native.quantize(_data(256), T.IQ4_XS)
    with pytest.raises(NotImplementedError):
        native.quantize(_data(256), T.IQ2_XXS)


IQ_GRID_TYPES = ["IQ2_XXS", "IQ2_XS", "IQ2_S", "IQ3_XXS", "IQ3_S", "IQ1_S", "IQ1_M"]


def _random_iq_blocks(name, nb, seed):
    from pmetal_b200.gguf.types import BLOCK_GEOMETRY
    nbytes = BLOCK_GEOMETRY[T[name]][1]
    blocks = np.random.default_rng(seed).integers(0, 256, size=(nb, nbytes), dtype=np.uint8)
    if name == "IQ1_M":                          # the f16 scale is spread over the top nibbles of four words
        sc = blocks[:, 48:56].view("<u2")
        sc[:, 3] = (sc[:, 3] & 0x0FFF) | 0x2000
    else:
        blocks[:, 0:2] = np.array([0.01 * (i + 1) for i in range(nb)], dtype="<f2").view(np.uint8).reshape(nb, 2)
    return blocks


@pytest.mark.parametrize("name", IQ_GRID_TYPES)
def test_grid_iquant_decoders_match_gguf_py(name):
    """Random block bytes decode to exactly what the gguf Python package gives."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    blocks = _random_iq_blocks(name, 9, seed=len(name))
    want = quants.dequantize(blocks, getattr(gguf.GGMLQuantizationType, name)).reshape(-1)
    got = native.dequantize(blocks.reshape(-1), T[name], 9 * 256)
    np.testing.assert_array_equal(got, want.astype(np.float32))
    assert native.can_dequantize(T[name]) and not native.can_quantize(T[name])
    with pytest.raises(ValueError):
        native.dequantize(blocks.reshape(-1)[:-1], T[name], 9 * 256)


def test_grid_iquant_structure_without_the_oracle():
    """Format facts that hold for any block: IQ2_XXS magnitudes come from the grid, signs have even parity, the scale
    nibble multiplies a whole group of 32, and IQ1_S values are scale * ({-1, 0, 1} +- 1/8)."""
    from pmetal_b200.gguf import iq_quants
    from pmetal_b200.gguf.iq_grids import KSIGNS, grid
    assert all(bin(int(v)).count("1") % 2 == 0 for v in KSIGNS) and [int(v) & 127 for v in KSIGNS] == list(range(128))
    assert grid("IQ2XXS").shape == (256, 8) and grid("IQ2XS").shape == (512, 8) and grid("IQ2S").shape == (1024, 8)
    assert grid("IQ3XXS").shape == (256, 4) and grid("IQ3S").shape == (512, 4) and grid("IQ1S").shape == (2048, 8)
    assert set(np.unique(grid("IQ2XXS"))) <= {8, 25, 43} and set(np.unique(grid("IQ1S"))) == {-1, 0, 1}
    blk = np.zeros(66, np.uint8)
    blk[0:2] = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)
    blk[2:6] = [5, 0, 0, 0]                                  # grid entries of the first four groups
    blk[6:10] = np.frombuffer(np.uint32((3 << 28) | 1).tobytes(), np.uint8)   # scale 3; first group: sign index 1
    y = iq_quants.dequantize(blk, T.IQ2_XXS, 256)
    db = (0.5 + 3) * 0.25
    sign = 1.0 - 2.0 * ((int(KSIGNS[1]) >> np.arange(8)) & 1)
    np.testing.assert_allclose(y[:8], db * grid("IQ2XXS")[5] * sign)
    np.testing.assert_allclose(y[8:16], db * grid("IQ2XXS")[0])
    np.testing.assert_allclose(y[32:40], 0.5 * 0.25 * grid("IQ2XXS")[0])     # next group of 32: scale nibble 0
    b1 = np.zeros(50, np.uint8)
    b1[0:2] = np.frombuffer(np.float16(2.0).tobytes(), np.uint8)
    b1[34:36] = np.frombuffer(np.uint16((2 << 12) | 0x8000).tobytes(), np.uint8)      # scale 2*2+1 = 5, negative offset
    y1 = iq_quants.dequantize(b1, T.IQ1_S, 256)
    np.testing.assert_allclose(y1[:8], 2.0 * 5 * (grid("IQ1S")[0] - 0.125))
    np.testing.assert_allclose(y1[32:40], 2.0 * 1 * (grid("IQ1S")[0] + 0.125))


def test_ternary_one_bit_and_nvfp4_codecs():
    # ternary inputs survive TQ1_0 / TQ2_0 exactly up to the f16 scale, including a ragged (padded) tail
    tern = np.random.default_rng(3).integers(-1, 2, 256 * 3 + 40).astype(np.float32) * 0.75
    for t, blk in ((T.TQ1_0, 54), (T.TQ2_0, 66)):
        q = native.quantize(tern, t)
        assert q.size == 4 * blk
        assert np.abs(native.dequantize(q, t, tern.size) - tern).max() < 1e-3
    # TQ2_0 layout: element m + 32 k of each 128-half sits in bits 2k of byte m; the scale is the last f16
    x = np.zeros(256, np.float32)
    x[0], x[32], x[64], x[96] = 1.0, -1.0, 0.0, 1.0
    q = native.quantize(x, T.TQ2_0)
    assert q[0] == (2 | (0 << 2) | (1 << 4) | (2 << 6)) and q[1] == 0x55
    assert np.frombuffer(q[64:66].tobytes(), np.float16)[0] == 1.0
    # TQ1_0: five trits base 3, most significant first, stored as ceil(v * 256 / 243)
    x = np.zeros(256, np.float32)
    x[0], x[32], x[64], x[96], x[128] = 1.0, 1.0, -1.0, 0.0, 1.0           # trits 2 2 0 1 2 -> 221
    q = native.quantize(x, T.TQ1_0)
    assert q[0] == -(-(221 * 256) // 243)
    # Q1_0: scale = mean |x| over the 128-element block, one sign bit per element (zero counts as positive)
    x = _data(128, seed=5)
    q = native.quantize(x, T.Q1_0)
    assert q.size == 18
    d = np.frombuffer(q[:2].tobytes(), np.float16)[0]
    assert abs(float(d) - np.abs(x).mean()) < 1e-3 * np.abs(x).mean() + 1e-4
    bits = np.unpackbits(q[2:], bitorder="little").astype(bool)
    assert (bits == (x >= 0)).all()
    y = native.dequantize(q, T.Q1_0, 128)
    assert np.allclose(np.abs(y), float(d)) and (np.sign(y) == np.where(x >= 0, 1, -1)).all()
    # NVFP4: 4 sub-blocks of 16 with an unsigned e4m3 scale each (decoded with a factor one half)
    x = _data(64 * 5 + 9, seed=6)
    q = native.quantize(x, T.NVFP4)
    assert q.size == 6 * 36
    y = native.dequantize(q, T.NVFP4, x.size)
    assert np.linalg.norm(y - x) / np.linalg.norm(x) < 0.13
    one = np.zeros(64, np.float32)
    one[:16] = 6.0                                         # amax / 6 = 1.0 -> e = 7, m = 0; decodes to 0.5 x code 7 (12)
    q = native.quantize(one, T.NVFP4)
    assert q[0] == (7 << 3) and q[1] == 0 and q[4] == 0x77
    assert np.allclose(native.dequantize(q, T.NVFP4, 64)[:16], 6.0)


def test_writer_layout_and_reader_round_trip(tmp_path):
    w = GgufWriter()
    w.add_string("general.architecture", "qwen3").add_u32("qwen3.block_count", 2).add_f32("qwen3.rope.freq_base", 1e6)
    w.add_array("tokenizer.ggml.tokens", 8, ["<a>", "b", "c"])
    a = _data(64 * 256).reshape(64, 256)
    w.add_tensor_f32("blk.0.attn_q.weight", a, T.Q4K)
    w.add_tensor_f32("output_norm.weight", a[0], T.F32)
    w.add_tensor_f32("blk.0.ffn_down.weight", a[:3, :96], T.F16)      # 576 bytes: last tensor is not padded
    p = str(tmp_path / "m.gguf")
    n = w.write_to(p)
    assert os.path.getsize(p) == n
    raw = open(p, "rb").read()
    magic, ver, nt, nkv = struct.unpack_from("<IIQQ", raw, 0)
    assert (magic, ver, nt, nkv) == (0x46554747, 3, 3, 6)
    # metadata keys appear in sorted order
    first_key_len = struct.unpack_from("<Q", raw, 24)[0]
    assert raw[32:32 + first_key_len] == b"general.alignment"
    with GgufFile(p) as f:
        assert f.metadata["qwen3.block_count"] == 2 and f.metadata["tokenizer.ggml.tokens"] == ["<a>", "b", "c"]
        assert f.data_start % 32 == 0
        assert f.tensors["blk.0.attn_q.weight"].shape == (64, 256)
        assert f.tensors["output_norm.weight"].offset % 32 == 0
        assert np.array_equal(f.tensor_f32("output_norm.weight"), a[0])
        q = f.tensor_f32("blk.0.attn_q.weight")
        assert np.linalg.norm(q - a) / np.linalg.norm(a) < 0.11
        assert f.tensor_f32("blk.0.ffn_down.weight").shape == (3, 96)
        assert f.data_start + f.tensors["blk.0.ffn_down.weight"].offset + 576 == len(raw)


def test_reader_rejects_malformed_files():
    w = GgufWriter()
    w.add_tensor_f32("t", _data(256), T.Q8_0)
    b = io.BytesIO()
    w.write(b)
    good = b.getvalue()
    GgufFile.from_bytes(good)
    with pytest.raises(GgufError):
        GgufFile.from_bytes(b"GGML" + good[4:])
    with pytest.raises(GgufError):
        GgufFile.from_bytes(good[:8] + struct.pack("<Q", 1 << 40) + good[16:])       # absurd tensor count
    with pytest.raises(GgufError):
        GgufFile.from_bytes(good[:-50])                                              # tensor data cut short
    with pytest.raises(GgufError):
        GgufFile.from_bytes(good[:24] + struct.pack("<Q", 1 << 60) + good[32:])      # string length overflow
    rng = np.random.default_rng(1)
    for _ in range(200):                                                             # random corruption never crashes
        m = bytearray(good)
        for _ in range(4):
            m[rng.integers(0, min(len(m), 200))] = rng.integers(0, 256)
        try:
            GgufFile.from_bytes(bytes(m))
        except (GgufError, UnicodeDecodeError, struct.error, OverflowError, MemoryError, ValueError):
            pass


def test_name_mapping_and_recipe():
    assert hf_to_gguf_name("model.layers.7.self_attn.q_proj.weight") == "blk.7.attn_q.weight"
    assert hf_to_gguf_name("model.embed_tokens.weight") == "token_embd.weight"
    assert hf_to_gguf_name("model.layers.1.mlp.experts.down_proj.weight") == "blk.1.ffn_down_exps.weight"
    assert gguf_to_hf_name("blk.3.attn_k_norm.weight") == "model.layers.3.self_attn.k_norm.weight"
    assert gguf_to_hf_name(hf_to_gguf_name("model.layers.0.mlp.up_proj.weight")) == "model.layers.0.mlp.up_proj.weight"
    cfg = {"num_hidden_layers": 32, "num_attention_heads": 32, "num_key_value_heads": 8}
    assert [use_more_bits(i, 32) for i in (0, 3, 4, 5, 6, 26, 28)] == [True, True, False, False, True, False, True]
    assert tensor_type("q4_k_m", "blk.0.attn_v.weight", (1024, 4096), cfg) == T.Q6K
    assert tensor_type("q4_k_m", "blk.5.attn_v.weight", (1024, 4096), cfg) == T.Q4K
    assert tensor_type("q4_k_m", "output.weight", (32000, 4096), cfg) == T.Q6K
    assert tensor_type("q2_k", "blk.9.attn_v.weight", (1024, 4096), cfg) == T.Q4K       # n_gqa >= 4
    assert tensor_type("q3_k_m", "blk.1.ffn_down.weight", (4096, 11008), cfg) == T.Q5K
    assert tensor_type("q4_k_m", "blk.2.attn_norm.weight", (4096,), cfg) == T.F16
    assert tensor_type("q8_0", "token_embd.weight", (32000, 4096), cfg) == T.Q8_0
    assert tensor_type("mxfp4", "token_embd.weight", (32000, 4096), cfg) == T.F16
    assert tensor_type("f16", "blk.0.attn_q.weight", (8, 8), cfg) == T.F16


def test_imatrix_round_trip_and_dynamic(tmp_path):
    im = IMatrix()
    im.accumulate("blk.0.attn_q.weight", np.ones((4, 8), np.float32) * 3)
    im.accumulate("blk.0.attn_q.weight", np.ones((4, 8), np.float32))
    im.accumulate("blk.1.ffn_up.weight", np.ones((2, 8), np.float32) * 0.1)
    for i in range(2, 10):
        im.accumulate(f"blk.{i}.ffn_up.weight", np.ones((2, 8), np.float32) * 0.01)
    p = str(tmp_path / "im.dat")
    im.save(p)
    back = IMatrix.load(p)
    assert back.ncalls["blk.0.attn_q.weight"] == 2
    assert np.allclose(back.data["blk.0.attn_q.weight"], 5.0)
    dq = DynamicQuantizer(DynamicConfig(), back)
    assert dq.propose("blk.0.attn_q.weight") == T.Q6K           # top 20 % by importance
    assert dq.propose("blk.5.ffn_up.weight") == T.Q4K
    assert dq.propose("output.weight") == T.Q6K                 # critical -> fallback
    assert DynamicQuantizer(DynamicConfig()).propose("blk.0.attn_q.weight") == T.Q4K
    with pytest.raises(ValueError):
        IMatrix.from_bytes(struct.pack("<i", -1))
    x = _data(4096)
    t = DynamicQuantizer(DynamicConfig(kl_calibrate=True, error_budget=0.05)).calibrate("blk.0.x.weight", x)
    assert t in (T.Q5K, T.Q6K)
    plan = {"a": (T.Q6K, 1000, 5.0), "b": (T.Q6K, 1000, 1.0), "output.weight": (T.Q6K, 10, 9.0)}
    out = DynamicQuantizer(DynamicConfig(target_bpw=5.6)).fit_target_bpw(plan)
    assert out["output.weight"] == T.Q6K and out["b"] != T.Q6K


def test_quantize_model_and_load_back(tmp_path):
    from pmetal_b200.models.config import ModelArgs
    from pmetal_b200.models.decoder import DecoderLM
    from pmetal_b200.models.loader import load_pretrained, save_pretrained
    cfg = ModelArgs(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                    num_attention_heads=2, num_key_value_heads=1, head_dim=128, tie_word_embeddings=False)
    m = DecoderLM(cfg).init_weights(0.05, 0)
    src = str(tmp_path / "hf")
    save_pretrained(m, src)
    out = str(tmp_path / "m.gguf")
    info = quantize_model(src, out, "q8_0")
    assert info["architecture"] == "qwen3" and info["types"]["Q8_0"] >= 14
    with GgufFile(out) as f:
        assert f.metadata["general.name"] == "quantized-model"
        assert f.metadata["qwen3.block_count"] == 2 and f.metadata["qwen3.attention.head_count_kv"] == 1
        assert f.tensors["blk.0.attn_norm.weight"].dtype == T.F32
        names = f.tensor_order
        assert names == sorted(names, key=lambda n: gguf_to_hf_name(n))        # plain tensors in HF-name order
    m2, args2, _ = load_pretrained(out, dtype=torch.float32)
    assert args2.num_hidden_layers == 2 and args2.head_dim == 128
    ids = torch.randint(0, 512, (1, 16))
    with torch.no_grad():
        a = m.float().loss(ids, ids.clone())
        b = m2.loss(ids, ids.clone())
    assert abs(float(a) - float(b)) < 0.05
    info2 = quantize_model(src, str(tmp_path / "k.gguf"), "q4_k_m")
    assert info2["types"].get("Q6K", 0) >= 1 and info2["compression"] > 3


@pytest.mark.parametrize("t", ["Q2K", "Q3K", "Q4K", "Q5K", "Q6K", "Q8K"])
def test_integer_vec_dot_equals_dequantised_dot(t):
    """The integer dot product with a Q8_K activation row equals the float dot product of the two dequantised rows."""
    from pmetal_b200.gguf import native
    from pmetal_b200.gguf.types import GgmlType
    ty = GgmlType[t]
    rng = np.random.default_rng(3)
    n = 1024
    x = rng.standard_normal(n).astype(np.float32)
    y = rng.standard_normal(n).astype(np.float32) * 2.0
    xb, yb = native.quantize(x, ty), native.quantize(y, GgmlType.Q8K)
    got = native.vec_dot_q8k(xb, ty, yb, n)
    want = float(np.dot(native.dequantize(xb, ty, n).astype(np.float64), native.dequantize(yb, GgmlType.Q8K, n).astype(np.float64)))
    assert abs(got - want) <= 1e-4 * max(1.0, abs(want)) + 1e-3
    with pytest.raises(ValueError):
        native.vec_dot_q8k(xb, ty, yb, 100)
    with pytest.raises(NotImplementedError):
        native.vec_dot_q8k(xb, GgmlType.Q4_0, yb, n)


def test_quantised_matvec_close_to_float():
    from pmetal_b200.gguf import native
    from pmetal_b200.gguf.types import GgmlType
    rng = np.random.default_rng(4)
    rows, n = 37, 512
    w = rng.standard_normal((rows, n)).astype(np.float32)
    y = rng.standard_normal(n).astype(np.float32)
    wb = native.quantize(w, GgmlType.Q6K)
    out = native.matvec_q8k(wb, GgmlType.Q6K, rows, n, y, threads=3)
    ref = w @ y
    assert np.abs(out - ref).max() / np.abs(ref).max() < 0.03
    wd = native.dequantize(wb, GgmlType.Q6K, rows * n).reshape(rows, n)
    yd = native.dequantize(native.quantize(y, GgmlType.Q8K), GgmlType.Q8K, n)
    np.testing.assert_allclose(out, wd @ yd, rtol=1e-4, atol=1e-3)


def test_gguf_file_with_iquant_tensor_reads_back(tmp_path):
    """A tensor stored in an i-quant type comes out of the reader as float32 through the same decoders."""
    from pmetal_b200.gguf.reader import GgufFile
    from pmetal_b200.gguf.writer import GgufWriter
    blocks = _random_iq_blocks("IQ3_S", 8, seed=2)           # 8 blocks = a [4, 512] matrix
    w = GgufWriter()
    w.add_string("general.architecture", "llama")
    w.add_tensor_bytes("blk.0.ffn_up.weight", [4, 512], T.IQ3_S, blocks.tobytes())
    path = tmp_path / "iq.gguf"
    w.write_to(str(path))
    with GgufFile(str(path)) as f:
        arr = f.tensor_f32("blk.0.ffn_up.weight")
    assert arr.shape == (4, 512)
    np.testing.assert_array_equal(arr.reshape(-1), native.dequantize(blocks.reshape(-1), T.IQ3_S, 8 * 256))
