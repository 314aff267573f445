"""Small parts: secret strings, MXFP8 block quantisation, fuzzing of the GGUF reader."""
import copy
import dataclasses
import io
import json
import pickle

import numpy as np
import pytest
import torch


def test_secret_string_never_prints():
    from pmetal_b200.core.config import ModelConfig
    from pmetal_b200.core.secrets import REDACTED, SecretString, expose
    s = SecretString("hf_abc123")
    assert str(s) == REDACTED and "hf_abc123" not in repr(s) and f"{s}" == REDACTED and f"{s:>12}" == f"{REDACTED:>12}"
    assert s.expose_secret() == "hf_abc123" and len(s) == 9 and not s.is_empty() and s == "hf_abc123" and s == SecretString(s)
    assert SecretString.from_option(None) is None and SecretString("").is_empty() and expose(None) is None
    with pytest.raises(TypeError):
        pickle.dumps(s)
    with pytest.raises(AttributeError):
        s.other = 1
    cfg = ModelConfig(model_id="m", hf_token="hf_abc123")
    assert isinstance(cfg.hf_token, SecretString) and expose(cfg.hf_token) == "hf_abc123"
    dumped = dataclasses.asdict(cfg)
    assert "hf_abc123" not in repr(dumped) and "hf_abc123" not in repr(cfg) and "hf_abc123" not in json.dumps(dumped, default=str)
    assert copy.deepcopy(cfg).hf_token.expose_secret() == "hf_abc123"


def test_full_config_dump_drops_the_token():
    from pmetal_b200.core.config import FullTrainingConfig
    cfg = FullTrainingConfig.from_dict({"model": {"model_id": "x", "hf_token": "hf_secret"}})
    d = cfg.to_dict()
    assert "hf_token" not in d["model"] and "hf_secret" not in json.dumps(d, default=str)


def test_mxfp8_round_trip_and_layout():
    from pmetal_b200.quant.mxfp8 import dequantize_mxfp8, quantize_mode, quantize_mxfp8
    torch.manual_seed(0)
    w = torch.randn(6, 128) * torch.logspace(-3, 3, 6)[:, None]
    codes, scales = quantize_mxfp8(w)
    assert codes.dtype == torch.uint8 and codes.shape == (6, 128) and scales.shape == (6, 4) and scales.dtype == torch.uint8
    back = dequantize_mxfp8(codes, scales)
    rel = ((back - w).abs().amax(-1) / w.abs().amax(-1))
    assert rel.max() < 0.07                              # 3 mantissa bits: half an ulp at the top of the block's range
    blocks = back.reshape(6, 4, 32).abs().amax(-1)       # the scale keeps every block inside the E4M3 range
    assert (blocks / torch.exp2(scales.float() - 127) <= 448).all()
    exact = torch.tensor([[0.0] * 31 + [1.5]]) * 2.0 ** 5
    c, s = quantize_mxfp8(exact)
    assert torch.equal(dequantize_mxfp8(c, s), exact)    # powers of two times E4M3 values are exact
    z, zs = quantize_mxfp8(torch.zeros(1, 32))
    assert int(zs[0, 0]) == 0 and torch.equal(dequantize_mxfp8(z, zs), torch.zeros(1, 32))
    assert len(quantize_mode(w, "mxfp8")) == 2 and len(quantize_mode(w, "affine", 4, 64)) == 3
    with pytest.raises(ValueError):
        quantize_mxfp8(torch.zeros(3, 33))
    with pytest.raises(ValueError):
        quantize_mode(w, "nope")


def _valid_gguf() -> bytes:
    from pmetal_b200.gguf.types import GgmlType
    from pmetal_b200.gguf.writer import GgufWriter
    w = GgufWriter()
    w.add_string("general.architecture", "llama")
    w.add_u32("llama.block_count", 2)
    w.add_array("tokenizer.ggml.tokens", __import__("pmetal_b200.gguf.types", fromlist=["ValueType"]).ValueType.STRING,
                ["a", "b", "c"])
    w.add_tensor_f32("token_embd.weight", np.arange(64, dtype=np.float32).reshape(2, 32))
    w.add_tensor_f32("blk.0.attn_q.weight", np.ones((2, 32), np.float32), GgmlType.Q8_0)
    buf = io.BytesIO()
    w.write(buf)
    return buf.getvalue()


def test_gguf_reader_survives_mutated_files():
    """Counterpart of the reference's cargo-fuzz target (fuzz/fuzz_targets/gguf_reader.rs): any byte string either parses
    or raises ``GgufError``; it never raises anything else, hangs or allocates by an attacker-chosen length."""
    hyp = pytest.importorskip("hypothesis")
    from hypothesis import HealthCheck, given, settings
    from hypothesis import strategies as st
    from pmetal_b200.gguf.reader import GgufError, GgufFile
    good = _valid_gguf()
    with GgufFile.from_bytes(good) as f:
        assert f.tensor_f32("token_embd.weight").shape == (2, 32)

    def parse(data: bytes):
        try:
            with GgufFile.from_bytes(data) as f:
                for name in list(f.tensors)[:4]:
                    f.tensor_f32(name)
        except GgufError:
            pass

    @settings(max_examples=300, deadline=None, suppress_health_check=list(HealthCheck))
    @given(st.lists(st.tuples(st.integers(0, len(good) - 1), st.integers(0, 255)), min_size=1, max_size=8),
           st.integers(0, len(good)))
    def mutate(edits, cut):
        b = bytearray(good)
        for pos, val in edits:
            b[pos] = val
        parse(bytes(b[:cut]) if cut % 3 == 0 else bytes(b))

    @settings(max_examples=200, deadline=None, suppress_health_check=list(HealthCheck))
    @given(st.binary(max_size=256))
    def garbage(tail):
        parse(b"GGUF" + tail)
        parse(tail)

    mutate()
    garbage()
