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


def test_stop_suffix_detection_follows_token_boundaries():
    from pmetal_b200.serve.engine import detect_stop_suffix
    words = {1: "alpha", 2: " beta", 3: " gamma", 4: " be", 5: "ta"}
    dec = lambda ids: "".join(words[i] for i in ids)      # noqa: E731
    assert detect_stop_suffix(dec, [1, 2, 3], ["beta gamma"]) == 0          # " beta gamma" != "beta gamma": no boundary
    assert detect_stop_suffix(dec, [1, 2, 3], [" beta gamma"]) == 2
    assert detect_stop_suffix(dec, [1, 2, 3], [" gamma", " beta gamma"]) == 2   # the longest match wins
    assert detect_stop_suffix(dec, [1, 4, 5], [" beta"]) == 2               # a stop string spread over two tokens
    assert detect_stop_suffix(dec, [1, 2], ["delta"]) == 0 and detect_stop_suffix(dec, [], ["x"]) == 0


def test_stop_strings_cut_the_output_and_penalties_change_sampling():
    from pmetal_b200.data.tokenizer import ByteTokenizer
    m = tiny()
    tok = ByteTokenizer()
    eng = ContinuousBatchEngine(m, max_slots=4, num_blocks=64)
    base = eng.generate([1, 2, 3, 4, 5], SamplingParams.greedy(24))
    text = tok.decode(base.output)
    # pick a stop string from the middle of the greedy answer (byte tokenizer: one token per byte)
    i = max(3, len(base.output) // 2)
    stop = tok.decode(base.output[i:i + 2])
    r = eng.generate([1, 2, 3, 4, 5], SamplingParams.greedy(24), stop_strings=[stop], decode=tok.decode,
                     want_logprobs=True)
    first = text.find(stop)
    assert r.finish_reason == "stop" and tok.decode(r.output) == text[:first]
    assert len(r.logprobs) == len(r.output)
    # a greedy answer of a tiny random model repeats itself; penalties over the generated tokens change that
    greedy = SamplingParams.greedy(24)
    pen = SamplingParams.greedy(24)
    pen.repetition_penalty, pen.frequency_penalty, pen.presence_penalty = 1.8, 0.6, 0.4
    a = eng.generate([9, 9, 9], greedy).output
    b = eng.generate([9, 9, 9], pen).output
    assert a != b and len(set(b)) > len(set(a))
    assert sorted(eng._free_rows) == list(range(4))          # count-table rows go back to the pool
    # the penalised request does not disturb an unpenalised one decoded in the same batch
    r1 = eng.submit(Request([9, 9, 9], greedy))
    r2 = eng.submit(Request([9, 9, 9], pen))
    while not (r1.done.is_set() and r2.done.is_set()):
        eng.tick()
    assert r1.output == a and r2.output == b
    eng.shutdown()


def test_http_logprob_alternatives_stop_holdback_and_tool_calls():
    fastapi = pytest.importorskip("fastapi")
    from fastapi.testclient import TestClient
    from pmetal_b200.data.tokenizer import ByteTokenizer
    from pmetal_b200.serve.server import ServerState, create_app, try_parse_tool_calls
    calls = try_parse_tool_calls(' {"name": "get_weather", "arguments": {"city": "Oslo"}} ')
    assert calls and calls[0]["function"]["name"] == "get_weather" and json.loads(calls[0]["function"]["arguments"]) == {"city": "Oslo"}
    calls = try_parse_tool_calls('{"tool_calls": [{"id": "c1", "function": {"name": "f", "arguments": "{}"}}, {"nofunction": 1}]}')
    assert len(calls) == 1 and calls[0]["id"] == "c1" and calls[0]["type"] == "function"
    assert try_parse_tool_calls("sure, here you go") is None and try_parse_tool_calls("{broken") is None
    assert try_parse_tool_calls('{"answer": 42}') is None
    m = tiny()
    eng = ContinuousBatchEngine(m, max_slots=4, num_blocks=128)
    eng.start()
    try:
        tok = ByteTokenizer()
        app = create_app(ServerState(eng, tok, model_name="tiny"))
        with TestClient(app) as c:
            msg = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 12, "temperature": 0}
            j = c.post("/v1/chat/completions", json={**msg, "logprobs": True, "top_logprobs": 3}).json()
            content = j["choices"][0]["logprobs"]["content"]
            assert len(content) == j["usage"]["completion_tokens"]
            for e in content:
                assert len(e["top_logprobs"]) == 3 and e["top_logprobs"][0]["logprob"] >= e["top_logprobs"][1]["logprob"]
                assert abs(e["top_logprobs"][0]["logprob"] - e["logprob"]) < 1e-3      # greedy: the choice is the top entry
            full = j["choices"][0]["message"]["content"]
            # stop string taken from the answer: non-streaming and streaming both end right before it
            stop = full[4:6]
            cut = full[:full.find(stop)]
            j2 = c.post("/v1/chat/completions", json={**msg, "stop": [stop]}).json()
            assert j2["choices"][0]["message"]["content"] == cut and j2["choices"][0]["finish_reason"] == "stop"
            with c.stream("POST", "/v1/chat/completions", json={**msg, "stop": stop, "stream": True}) as s:
                lines = [l for l in s.iter_lines() if l.startswith("data: ") and l != "data: [DONE]"]
            pieces = "".join(json.loads(l[6:])["choices"][0]["delta"].get("content") or "" for l in lines)
            assert pieces == cut                                                         # nothing of the stop string leaked
            j3 = c.post("/v1/completions", json={"prompt": "abc", "max_tokens": 4, "temperature": 0, "logprobs": 2}).json()
            lp = j3["choices"][0]["logprobs"]
            # (alternatives are keyed by their text: two byte tokens that decode to the same replacement character share a key)
            assert len(lp["tokens"]) == len(lp["token_logprobs"]) == len(lp["top_logprobs"]) and 1 <= len(lp["top_logprobs"][0]) <= 2
    finally:
        eng.shutdown()
