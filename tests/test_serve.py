"""Continuous-batching engine, prefix cache and the HTTP routes (CPU, tiny random model, byte tokenizer)."""
import json
import threading

import pytest
import torch

from pmetal_b200.models.sampling import SamplingParams
from pmetal_b200.serve.engine import ContinuousBatchEngine, Request


def tiny():
    from pmetal_b200.models.config import ModelArgs
    from pmetal_b200.models.decoder import DecoderLM
    cfg = ModelArgs(vocab_size=300, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2,
                    num_key_value_heads=1, head_dim=16)
    m = DecoderLM(cfg).init_weights(0.1, 0).eval()
    for p in m.parameters():
        p.requires_grad_(False)
    return m


def test_engine_matches_plain_generation_and_batches():
    from pmetal_b200.models.generation import Generator
    m = tiny()
    prompts = [[1, 2, 3, 4, 5], list(range(10, 90)), [7, 7, 7]]
    ref = Generator(m, num_blocks=64).generate(prompts, SamplingParams.greedy(12))
    eng = ContinuousBatchEngine(m, max_slots=2, num_blocks=64, prefill_chunk=32)
    reqs = [eng.submit(Request(p, SamplingParams.greedy(12), want_logprobs=True)) for p in prompts]
    ticks = 0
    while not all(r.done.is_set() for r in reqs):
        assert eng.tick() or all(r.done.is_set() for r in reqs)
        ticks += 1
        assert ticks < 500
    for r, want in zip(reqs, ref.tokens):
        assert r.output == want and r.finish_reason == "length" and len(r.logprobs) == 12
    assert eng.stats.requests_done == 3 and eng.stats.generated_tokens == 36
    assert eng.cache.num_free() + sum(len(eng.cache.seqs[s].blocks) for s in eng.cache.seqs) >= 0
    eng.shutdown()
    assert eng.cache.num_free() == 64


def test_stop_sequences_eos_and_prefix_cache_reuse():
    m = tiny()
    eng = ContinuousBatchEngine(m, max_slots=4, num_blocks=64)
    base = eng.generate(list(range(5, 140)), SamplingParams.greedy(8))
    assert base.cached_tokens == 0
    again = eng.generate(list(range(5, 140)) + [1, 2], SamplingParams.greedy(8))
    assert again.cached_tokens == 128                      # two whole 64-token blocks shared
    fresh = ContinuousBatchEngine(m, max_slots=4, num_blocks=64, prefix_cache=False)
    want = fresh.generate(list(range(5, 140)) + [1, 2], SamplingParams.greedy(8))
    assert again.output == want.output                      # cached prefix gives identical tokens
    stop_seq = base.output[2:4]
    r = eng.generate(list(range(5, 140)), SamplingParams.greedy(8), stop_sequences=[stop_seq])
    assert r.finish_reason == "stop" and r.output[-2:] == stop_seq and r.output == base.output[:len(r.output)]
    eng2 = ContinuousBatchEngine(m, eos_ids=[base.output[1]], max_slots=4, num_blocks=64)
    r2 = eng2.generate(list(range(5, 140)), SamplingParams.greedy(8))
    first = base.output.index(base.output[1])
    assert r2.finish_reason == "stop" and r2.output == base.output[:first + 1]
    big = eng.submit(Request(list(range(200)) * 30, SamplingParams.greedy(4)))
    while not big.done.is_set():
        eng.tick()
    assert big.finish_reason == "error:too_long"


def test_background_thread_and_concurrent_submitters():
    m = tiny()
    eng = ContinuousBatchEngine(m, max_slots=8, num_blocks=128)
    eng.start()
    outs = {}

    def worker(i):
        outs[i] = eng.generate([i + 1, i + 2, i + 3], SamplingParams.greedy(6)).output
    ts = [threading.Thread(target=worker, args=(i,)) for i in range(6)]
    [t.start() for t in ts]
    [t.join(30) for t in ts]
    eng.shutdown()
    assert len(outs) == 6 and all(len(v) == 6 for v in outs.values())


def test_http_routes():
    fastapi = pytest.importorskip("fastapi")
    from fastapi.testclient import TestClient
    from pmetal_b200.data.tokenizer import ByteTokenizer
    from pmetal_b200.serve.server import ServerState, create_app
    m = tiny()
    eng = ContinuousBatchEngine(m, max_slots=4, num_blocks=128)
    eng.start()
    try:
        app = create_app(ServerState(eng, ByteTokenizer(), model_name="tiny"))
        with TestClient(app) as c:
            assert c.get("/health").json()["status"] == "ok"
            assert c.get("/v1/models").json()["data"][0]["id"] == "tiny"
            r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 5,
                                                     "temperature": 0, "logprobs": True})
            j = r.json()
            assert r.status_code == 200 and j["choices"][0]["finish_reason"] in ("stop", "length")
            assert j["usage"]["completion_tokens"] <= 5 and len(j["choices"][0]["logprobs"]["content"]) == j["usage"]["completion_tokens"]
            r = c.post("/v1/completions", json={"prompt": "abc", "max_tokens": 4, "temperature": 0})
            assert r.status_code == 200 and r.json()["usage"]["prompt_tokens"] == 3
            r = c.post("/v1/embeddings", json={"input": ["hello", "world!"]})
            e = r.json()["data"]
            assert len(e) == 2 and abs(sum(x * x for x in e[0]["embedding"]) - 1) < 1e-3
            r = c.post("/v1/messages", json={"system": "be brief", "messages": [{"role": "user", "content": [{"type": "text", "text": "yo"}]}],
                                             "max_tokens": 4, "temperature": 0})
            assert r.status_code == 200 and r.json()["content"][0]["type"] == "text" and r.json()["stop_reason"] in ("end_turn", "max_tokens")
            assert c.post("/v1/messages", json={"messages": [{"role": "user", "content": "x"}]}).status_code == 400
            with c.stream("POST", "/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}],
                                                                   "max_tokens": 4, "temperature": 0, "stream": True}) as s:
                lines = [l for l in s.iter_lines() if l.startswith("data: ")]
            assert lines[-1] == "data: [DONE]"
            chunks = [json.loads(l[6:]) for l in lines[:-1]]
            assert chunks[0]["choices"][0]["delta"]["role"] == "assistant" and chunks[-1]["choices"][0]["finish_reason"] in ("stop", "length")
            with c.stream("POST", "/v1/messages", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3,
                                                        "temperature": 0, "stream": True}) as s:
                evs = [l for l in s.iter_lines() if l.startswith("event: ")]
            assert evs[0] == "event: message_start" and evs[-1] == "event: message_stop"
            assert c.post("/v1/chat/completions", json={"messages": []}).status_code == 400
            assert c.post("/v1/chat/completions", content=b"x" * (2 * 1024 * 1024 + 10)).status_code == 413
            assert c.get("/v1/metrics").json()["requests_done"] >= 4
    finally:
        eng.shutdown()
