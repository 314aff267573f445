"""Serving the config-driven architectures: the sequential engine behind the same HTTP routes."""
import json
import threading

import pytest
import torch

from pmetal_b200.models.sampling import SamplingParams
from pmetal_b200.serve.engine import Request
from pmetal_b200.serve.portable_engine import PortableEngine


def _gemma():
    from pmetal_b200.models.architectures.generic import GenericDecoderLM, arch_config_from_hf
    cfg = dict(model_type="gemma2", vocab_size=300, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
               num_attention_heads=4, num_key_value_heads=2, head_dim=8, max_position_embeddings=256, sliding_window=16,
               final_logit_softcapping=30.0, attn_logit_softcapping=50.0, query_pre_attn_scalar=8)
    torch.manual_seed(0)
    return GenericDecoderLM(arch_config_from_hf(cfg)).init_weights(0.3, 0).eval()


def _greedy(model, prompt, n):
    cache = model.new_cache()
    cur, out = torch.tensor([prompt]), []
    with torch.no_grad():
        for _ in range(n):
            nxt = int(model(cur, cache)[:, -1].argmax(-1))
            out.append(nxt)
            cur = torch.tensor([[nxt]])
    return out


def test_engine_matches_the_models_own_greedy_decoding_with_chunked_prefill():
    m = _gemma()
    prompts = [[5, 9, 200, 17, 3, 44, 8], [7], list(range(20, 60))]
    eng = PortableEngine(m, max_slots=2, prefill_chunk=16)          # the 40-token prompt takes three chunks
    reqs = [eng.submit(Request(p, SamplingParams.greedy(6))) for p in prompts]
    while not all(r.done.is_set() for r in reqs):
        eng.tick()
    for p, r in zip(prompts, reqs):
        assert r.output == _greedy(m, p, 6) and r.finish_reason == "length"
    st = eng.stats.as_dict()
    assert st["requests_done"] == 3 and st["generated_tokens"] == 18 and st["prompt_tokens"] == 48 and not eng.slots


def test_stops_logprobs_penalties_and_cancellation():
    m = _gemma()
    base = _greedy(m, [1, 2, 3], 8)
    eos = base[3]
    cut = base.index(eos) + 1                                    # a tiny random model may repeat itself: first occurrence
    eng = PortableEngine(m, eos_ids=[eos])
    r = eng.generate([1, 2, 3], SamplingParams.greedy(8))
    assert r.output == base[:cut] and r.finish_reason == "stop"
    eng = PortableEngine(m)
    seq = base[1:3]
    n = next(i for i in range(2, 9) if base[i - 2:i] == seq)
    r = eng.generate([1, 2, 3], SamplingParams.greedy(8), stop_sequences=[seq], want_logprobs=True, top_logprobs=3)
    assert r.output == base[:n] and len(r.logprobs) == n and len(r.top_entries) == n and r.top_entries[0][0][0] == base[0]
    assert all(lp <= 0 for lp in r.logprobs)
    rep = eng.generate([1, 2, 3], SamplingParams(temperature=0.0, max_tokens=8, repetition_penalty=50.0))
    assert len(set(rep.output)) == len(rep.output)               # a strong penalty never repeats a token
    with pytest.raises(KeyError):
        eng.submit(Request([1], SamplingParams(), adapter="x"))
    eng.start()
    slow = eng.submit(Request([1, 2], SamplingParams(temperature=0.0, max_tokens=100000)))
    eng.shutdown()
    assert slow.done.is_set() and slow.finish_reason in ("cancelled", "length", "stop")


def test_http_routes_on_a_portable_model():
    pytest.importorskip("fastapi")
    from fastapi.testclient import TestClient
    from pmetal_b200.data.tokenizer import ByteTokenizer
    from pmetal_b200.serve.server import ServerState, create_app
    m = _gemma()
    eng = PortableEngine(m, max_slots=4)
    eng.start()
    try:
        app = create_app(ServerState(eng, ByteTokenizer(), model_name="tiny-gemma"))
        with TestClient(app) as c:
            assert c.get("/v1/models").json()["data"][0]["id"] == "tiny-gemma"
            r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 5,
                                                     "temperature": 0, "logprobs": True, "top_logprobs": 2})
            j = r.json()
            assert r.status_code == 200 and j["usage"]["completion_tokens"] <= 5
            assert len(j["choices"][0]["logprobs"]["content"][0]["top_logprobs"]) == 2
            results = []

            def ask(i):
                rr = c.post("/v1/completions", json={"prompt": "abc" * (i + 1), "max_tokens": 6, "temperature": 0})
                results.append(rr.status_code)
            ts = [threading.Thread(target=ask, args=(i,)) for i in range(5)]
            [t.start() for t in ts]
            [t.join() for t in ts]
            assert results == [200] * 5
            e = c.post("/v1/embeddings", json={"input": "hello"}).json()["data"][0]["embedding"]
            assert abs(sum(x * x for x in e) - 1) < 1e-3
            with c.stream("POST", "/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}],
                                                                   "max_tokens": 4, "temperature": 0, "stream": True}) as s:
                lines = [l for l in s.iter_lines() if l.startswith("data: ")]
            assert lines[-1] == "data: [DONE]" and json.loads(lines[0][6:])["choices"][0]["delta"]["role"] == "assistant"
            mt = c.get("/v1/metrics").json()
            assert mt["requests_done"] >= 7 and mt["free_kv_blocks"] == 4
    finally:
        eng.shutdown()
