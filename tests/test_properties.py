"""Property-based tests (hypothesis) of host-side invariants: packing, gradient codecs, learning-rate schedules, streamed
decoding, the safetensors reader / writer and the stop-suffix detector."""
import math

import numpy as np
import pytest
import torch

hyp = pytest.importorskip("hypothesis")
from hypothesis import HealthCheck, given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402

FAST = settings(max_examples=60, deadline=None, suppress_health_check=list(HealthCheck))


@FAST
@given(st.lists(st.integers(1, 40), min_size=1, max_size=30), st.integers(8, 48), st.sampled_from(["ffd", "greedy"]))
def test_packer_keeps_every_token_once_and_respects_the_length(lengths, max_len, algorithm):
    from pmetal_b200.data.packing import PackerConfig, Sample, SequencePacker
    samples = [Sample(list(range(i * 100, i * 100 + n)), list(range(i * 100, i * 100 + n))) for i, n in enumerate(lengths)]
    packs = SequencePacker(PackerConfig(max_length=max_len, algorithm=algorithm, max_seq_length=max_len)).pack(samples)
    seen = []
    for p in packs:
        assert p.total_tokens() <= max_len and p.cu_seqlens[0] == 0 and p.cu_seqlens[-1] == p.total_tokens()
        assert all(b > a for a, b in zip(p.cu_seqlens, p.cu_seqlens[1:])) and len(p.cu_seqlens) == p.num_sequences + 1
        for a, b in zip(p.cu_seqlens, p.cu_seqlens[1:]):
            assert p.position_ids[a:b] == list(range(b - a))                 # positions restart in every document
            seen.append(tuple(p.input_ids[a:b]))
    want = sorted(tuple(s.input_ids[:max_len]) for s in samples)                # long documents are cut, none is dropped
    assert sorted(seen) == want


@FAST
@given(st.lists(st.floats(-50, 50, allow_nan=False, width=32), min_size=1, max_size=200),
       st.sampled_from(["none", "fp16", "bf16", "int8", "onebit", "topk", "random"]))
def test_gradient_codecs_round_trip_through_bytes_with_bounded_error(values, strategy):
    from pmetal_b200.parallel.compression import GradientCompressor, deserialize, serialize
    g = np.asarray(values, dtype=np.float32)
    comp = GradientCompressor(strategy, ratio=0.25, use_error_feedback=True)
    c = comp.compress(g)
    back = GradientCompressor.decompress(deserialize(serialize(c)))
    assert back.shape == g.shape and np.isfinite(back).all()
    amax = float(np.abs(g).max())
    if strategy == "none":
        assert np.array_equal(back, g)
    elif strategy in ("fp16", "bf16"):
        assert np.abs(back - g).max() <= 2 ** (-7 if strategy == "bf16" else -10) * max(amax, 1e-3) + 1e-6
    elif strategy == "int8":
        assert np.abs(back - g).max() <= amax / 127.0 + 1e-6
    elif strategy == "topk":
        kept = back != 0
        assert kept.sum() <= max(int(g.size * 0.25), 1) and np.array_equal(back[kept], g[kept])
        if comp.error is not None:                                            # what was not sent is remembered exactly
            assert np.allclose(comp.error + back, g, atol=1e-6)
    elif strategy == "onebit":
        assert set(np.unique(np.abs(back)).tolist()) <= {float(np.float32(c.scale))}


@FAST
@given(st.sampled_from(["constant", "linear", "cosine", "cosine_with_restarts", "polynomial", "wsd"]),
       st.integers(1, 400), st.integers(0, 80), st.floats(1e-6, 1e-2), st.floats(0.0, 0.5))
def test_learning_rate_schedules_stay_in_range_and_warm_up(kind, total, warmup, base, min_frac):
    from pmetal_b200.core.scheduler import LearningRateScheduler
    warmup = min(warmup, total)
    s = LearningRateScheduler(base, total, warmup, kind, min_lr=base * min_frac, num_restarts=2)
    lrs = [s.get_lr(i) for i in range(total + 5)]
    assert all(math.isfinite(x) and -1e-12 <= x <= base * (1 + 1e-9) for x in lrs)
    if warmup > 1:
        ramp = lrs[:warmup]
        assert all(b >= a - 1e-15 for a, b in zip(ramp, ramp[1:])) and abs(ramp[0] - base * min_frac) < 1e-12     # from min_lr up
    if kind == "constant" and total > warmup:
        assert abs(lrs[warmup] - base) < 1e-12


@FAST
@given(st.text(alphabet=st.characters(min_codepoint=32, max_codepoint=0x2FFF, blacklist_categories=("Cs",)), max_size=40))
def test_streamed_decoding_concatenates_to_the_full_text(text):
    from pmetal_b200.data.tokenizer import ByteTokenizer, StreamDecoder
    tok = ByteTokenizer()
    ids = tok.encode(text)
    dec = StreamDecoder(tok)
    pieces = "".join(dec.push(i) for i in ids)
    assert pieces == tok.decode(ids) and "�" not in pieces


@FAST
@given(specs=st.lists(st.tuples(st.sampled_from(["float32", "bfloat16", "int64", "uint8", "float16"]),
                                st.lists(st.integers(0, 5), min_size=0, max_size=3)), min_size=1, max_size=6))
def test_safetensors_round_trip_any_shapes_and_types(tmp_path_factory, specs):
    from pmetal_b200.utils.safetensors_io import load_file, load_file_parallel, save_file
    g = torch.Generator().manual_seed(0)
    tensors = {}
    for i, (dt, shape) in enumerate(specs):
        dtype = getattr(torch, dt)
        t = torch.randint(0, 100, tuple(shape), generator=g)
        tensors[f"t{i}"] = t.to(dtype)
    path = str(tmp_path_factory.mktemp("st") / "x.safetensors")
    save_file(tensors, path, metadata={"format": "pt"})
    for loader in (load_file, lambda p: load_file_parallel(p, threads=2)):
        back = loader(path)
        assert set(back) == set(tensors)
        for k, v in tensors.items():
            assert back[k].dtype == v.dtype and back[k].shape == v.shape and torch.equal(back[k], v)


@FAST
@given(st.lists(st.integers(97, 122), min_size=0, max_size=20), st.lists(st.integers(97, 122), min_size=1, max_size=4))
def test_stop_suffix_detector_agrees_with_string_search(prefix, stop):
    from pmetal_b200.serve.engine import detect_stop_suffix
    decode = lambda ids: "".join(chr(i) for i in ids)                      # noqa: E731
    gen = prefix + stop
    cut = detect_stop_suffix(decode, gen, [decode(stop)])
    assert cut == len(stop) and decode(gen[len(gen) - cut:]) == decode(stop)      # one character per token here
    longer = decode(prefix[-1:] + stop) if prefix else decode(stop)
    assert detect_stop_suffix(decode, gen, [decode(stop), longer]) == len(longer)    # the longest stop that ends the text
    assert detect_stop_suffix(decode, prefix, ["~~"]) == 0 and detect_stop_suffix(decode, [], [decode(stop)]) == 0
