"""End-to-end CLI runs on CPU with a tiny random checkpoint written to a temp directory."""
import json
import os

import pytest
import torch

from pmetal_b200.cli.main import main


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    from pmetal_b200.models.config import ModelArgs
    from pmetal_b200.models.decoder import DecoderLM
    from pmetal_b200.models.loader import save_pretrained
    d = str(tmp_path_factory.mktemp("m"))
    cfg = ModelArgs(vocab_size=300, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                    num_key_value_heads=1, head_dim=64, tie_word_embeddings=False)
    save_pretrained(DecoderLM(cfg).init_weights(0.05, 0), d)
    return d


def _json_out(capsys):
    return json.loads(capsys.readouterr().out.strip().splitlines()[-1])


def test_infer_eval_and_speculative(model_dir, capsys, tmp_path):
    assert main(["infer", "-m", model_dir, "-p", "hello", "--max-tokens", "5", "--greedy", "--json", "--device", "cpu"]) == 0
    j = _json_out(capsys)
    assert j["generated_tokens"] == 5 and j["prompt_tokens"] == 5
    assert main(["infer", "-m", model_dir, "-p", "hi", "--chat", "--system", "s", "--max-tokens", "3", "--greedy", "--device", "cpu"]) == 0
    capsys.readouterr()
    assert main(["infer", "-m", model_dir, "-p", "hello", "--max-tokens", "6", "--greedy", "--json", "--draft-model", model_dir,
                 "--speculative-k", "3", "--device", "cpu"]) == 0
    j2 = _json_out(capsys)
    assert j2["acceptance_rate"] == 1.0 and j2["tokens"] == 6          # draft == target -> everything accepted
    data = tmp_path / "d.jsonl"
    data.write_text("\n".join(json.dumps({"text": "the quick brown fox " * 3}) for _ in range(3)))
    assert main(["eval", "-m", model_dir, "-d", str(data), "--device", "cpu"]) == 0
    e = _json_out(capsys)
    assert e["samples"] == 3 and e["perplexity"] > 1


def test_quantize_merge_fuse_ollama(model_dir, capsys, tmp_path):
    gg = str(tmp_path / "m.gguf")
    assert main(["quantize", "-m", model_dir, "-o", gg, "--method", "q8_0"]) == 0
    q = _json_out(capsys)
    assert q["tensors"] > 10 and os.path.getsize(gg) == q["bytes"]
    assert main(["infer", "-m", gg, "-p", "hello", "--max-tokens", "3", "--greedy", "--json", "--device", "cpu"]) == 0
    assert _json_out(capsys)["generated_tokens"] == 3
    out = str(tmp_path / "merged")
    assert main(["merge", "--models", model_dir, model_dir, "--method", "linear", "-o", out, "--dtype", "float32"]) == 0
    capsys.readouterr()
    from pmetal_b200.models.loader import read_state_dict
    a, b = read_state_dict(model_dir), read_state_dict(out)
    k = "model.layers.0.mlp.down_proj.weight"
    assert torch.allclose(a[k].float(), b[k].float(), atol=1e-3)
    fp8 = str(tmp_path / "fp8")
    assert main(["quantize", "-m", model_dir, "-o", fp8, "--format", "fp8"]) == 0
    f = _json_out(capsys)
    assert f["quantized_tensors"] > 0
    from pmetal_b200.models.fp8 import dequantize_fp8_state_dict
    from pmetal_b200.utils.safetensors_io import load_file
    back = dequantize_fp8_state_dict(load_file(os.path.join(fp8, "model.safetensors")), torch.float32)
    assert (back[k] - a[k].float()).abs().max() < 0.07 * a[k].float().abs().max()
    mf = str(tmp_path / "Modelfile")
    assert main(["ollama", "modelfile", "--gguf", gg, "-o", mf, "--template", "chatml", "--system", "be nice"]) == 0
    assert main(["ollama", "create", "--name", "me/tiny:v1", "--base", gg, "-o", mf + "2", "--num-ctx", "4096"]) == 0
    assert "ollama create me/tiny:v1" in capsys.readouterr().out and "num_ctx 4096" in open(mf + "2").read()
    assert main(["ollama", "create", "--name", "x; rm -rf /", "--base", gg, "-o", mf + "3"]) == 2
    text = open(mf).read()
    assert text.startswith("FROM ") and 'SYSTEM """be nice"""' in text and "PARAMETER stop" in text
    assert main(["download", "/nonexistent/x"]) == 1


def test_distill_and_grpo_commands(model_dir, capsys, tmp_path):
    data = tmp_path / "p.jsonl"
    data.write_text("\n".join(json.dumps({"prompt": f"question {i} about things"}) for i in range(4)))
    out = str(tmp_path / "dist")
    assert main(["distill", "--teacher", model_dir, "--student", model_dir, "-d", str(data), "-o", out, "--max-steps", "2",
                 "--lora-r", "4", "--device", "cpu"]) == 0
    assert os.path.exists(os.path.join(out, "lora_weights.safetensors"))
    capsys.readouterr()
    out2 = str(tmp_path / "grpo")
    assert main(["grpo", "-m", model_dir, "-d", str(data), "-o", out2, "--max-steps", "1", "--num-generations", "2",
                 "--max-completion-length", "4", "--lora-r", "4", "--device", "cpu", "--reward", "length"]) == 0
    assert os.path.exists(os.path.join(out2, "adapter_config.json"))
    assert main(["cluster", "status"]) == 0


def test_new_subcommands(tmp_path, capsys):
    import json

    import torch

    from pmetal_b200.cli import commands
    from pmetal_b200.cli.main import main
    # dashboard folds an event file
    ev = tmp_path / "events.jsonl"
    ev.write_text("\n".join(json.dumps(e) for e in [
        {"event": "started", "job_id": "j1", "kind": "train", "ts": 1},
        {"event": "metric", "job_id": "j1", "payload": {"kind": "step", "step": 3, "loss": 1.5, "tokens_per_s": 10.0}},
        {"event": "finished", "job_id": "j1"}]) + "\n")
    assert main(["dashboard", str(ev), "--once"]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out == {"job": "j1", "state": "finished", "kind": "train", "step": 3, "loss": 1.5, "tokens_per_s": 10.0}
    # pack-experts: per-layer binary files with fixed-size expert records, both checkpoint layouts
    torch.manual_seed(0)
    sd = {"model.embed_tokens.weight": torch.randn(8, 64),
          "model.layers.0.mlp.experts.gate_up_proj": torch.randn(3, 256, 64), "model.layers.0.mlp.experts.down_proj": torch.randn(3, 64, 128)}
    for e in range(3):
        sd[f"model.layers.2.mlp.experts.{e}.gate_proj.weight"] = torch.randn(128, 64)
        sd[f"model.layers.2.mlp.experts.{e}.up_proj.weight"] = torch.randn(128, 64)
        sd[f"model.layers.2.mlp.experts.{e}.down_proj.weight"] = torch.randn(64, 128)
    lay = commands.pack_experts(sd, str(tmp_path / "packed"), bits=4, group_size=64, model_name="toy")
    assert lay["moe_layer_indices"] == [0, 2] and lay["num_experts"] == 3 and lay["bits"] == "Four"
    rec = lay["record"]
    assert rec["gate_weight"] == {"offset": 0, "size": 128 * 8 * 4, "shape": [128, 8]} and rec["gate_scales"]["shape"] == [128, 1]
    assert lay["expert_size"] == rec["down_biases"]["offset"] + rec["down_biases"]["size"]
    assert (tmp_path / "packed" / "layer_02.bin").stat().st_size == 3 * lay["expert_size"]
    one = commands.read_packed_expert(str(tmp_path / "packed"), 0, 2)
    ref = sd["model.layers.0.mlp.experts.gate_up_proj"][2, 128:]
    assert one["up"].shape == (128, 64) and float((one["up"] - ref).norm() / ref.norm()) < 0.15
    two = commands.read_packed_expert(str(tmp_path / "packed"), 2, 1)
    ref = sd["model.layers.2.mlp.experts.1.down_proj.weight"]
    assert float((two["down"] - ref).norm() / ref.norm()) < 0.15
    # offline search, native call overhead, delta-rule micro-benchmark, DFlash on a random target
    assert main(["search", "nothing-matches-this"]) == 0 and json.loads(capsys.readouterr().out)["results"] == []
    assert main(["bench-ffi", "--calls", "2000"]) == 0 and json.loads(capsys.readouterr().out)["ns_per_call"] > 0
    assert main(["bench-gdn", "--tokens", "48", "--heads", "2", "--device", "cpu"]) == 0
    assert json.loads(capsys.readouterr().out)["max_abs_diff"] < 1e-3
    assert main(["dflash", "-m", "random:tiny-qwen3", "--draft", "random", "--max-tokens", "12", "--device", "cpu"]) == 0
    res = json.loads(capsys.readouterr().out)
    assert len(res["tokens"]) == 12 and res["avg_acceptance_length"] >= 1


def test_infer_benchmark_profile_tools_and_repetition(model_dir, capsys, tmp_path):
    from pmetal_b200.cli.commands import cut_repetition
    assert cut_repetition(list(range(30))) is None
    assert cut_repetition([1, 2, 3] + [7] * 30) == 4                               # one copy of the repeated token stays
    assert cut_repetition([9, 9] + [4, 5, 6] * 10) == 5 and cut_repetition([4, 5, 6] * 3) is None
    assert main(["infer", "-m", model_dir, "-p", "x", "--max-tokens", "4", "--greedy", "--benchmark", "--benchmark-iters", "1",
                 "--benchmark-prompt-tokens", "16", "--device", "cpu"]) == 0
    b = _json_out(capsys)
    assert b["prompt_tokens"] == 16 and b["new_tokens"] == 4 and b["decode_tok_per_s"] > 0 and b["prefill_tok_per_s"] > 0
    prof = tmp_path / "layers.json"
    assert main(["infer", "-m", model_dir, "-p", "hello world", "--profile-layers", "--profile-output", str(prof),
                 "--device", "cpu"]) == 0
    rep = json.load(open(prof))
    assert [r["layer"] for r in rep["layers"]] == [0, 1] and rep["total_ms"] > 0
    tools = tmp_path / "tools.json"
    tools.write_text(json.dumps([{"type": "function", "function": {"name": "get_time", "description": "now", "parameters": {}}}]))
    assert main(["infer", "-m", model_dir, "-p", "time?", "--tools", str(tools), "--max-tokens", "2", "--greedy", "--json",
                 "--backend", "standard", "--kv-quant", "--detect-repetition", "--device", "cpu"]) == 0
    out = capsys.readouterr()
    # --kv-quant selects the int8 paged cache; the tool block is in the prompt
    assert "kv cache: int8 (explicit)" in out.err and json.loads(out.out.strip().splitlines()[-1])["prompt_tokens"] > 20


def test_quantize_with_adapter_and_bits(model_dir, capsys, tmp_path):
    from pmetal_b200.lora import apply_lora
    from pmetal_b200.core.config import LoraConfig
    from pmetal_b200.lora.adapter import save_adapter
    from pmetal_b200.models.loader import load_pretrained
    m, _, _ = load_pretrained(model_dir, dtype=torch.float32)
    cfg = LoraConfig(r=4, alpha=8.0)
    apply_lora(m, cfg)
    for n, p in m.named_parameters():
        if "lora_b" in n:
            torch.nn.init.normal_(p, std=0.05)
    ad = str(tmp_path / "adapter")
    save_adapter(m, ad, cfg)
    assert main(["quantize", "-m", model_dir, "-o", str(tmp_path / "q.gguf"), "--method", "q8_0", "--lora", ad]) == 0
    a = _json_out(capsys)
    assert main(["quantize", "-m", model_dir, "-o", str(tmp_path / "p.gguf"), "--method", "q8_0"]) == 0
    b = _json_out(capsys)
    assert a["tensors"] == b["tensors"]
    assert open(tmp_path / "q.gguf", "rb").read() != open(tmp_path / "p.gguf", "rb").read()      # the adapter changed the weights
    assert main(["quantize", "-m", model_dir, "-o", str(tmp_path / "mlx"), "--format", "mlx", "--bits", "6"]) == 0
    r = _json_out(capsys)
    assert 5.0 < r["effective_bpw"] < 8.5


def test_grpo_epochs_checkpoints_resume_and_metrics(model_dir, capsys, tmp_path):
    data = tmp_path / "p.jsonl"
    data.write_text("".join(json.dumps({"question": f"what is {i}+1?", "answer": str(i + 1)}) + "\n" for i in range(3)))
    out = str(tmp_path / "g")
    common = ["grpo", "-m", model_dir, "-d", str(data), "-o", out, "--num-generations", "2", "--max-completion-length", "4",
              "--prompt-column", "question", "--reasoning-rewards", "--async-rewards", "--device", "cpu"]
    assert main(common + ["--epochs", "1", "--checkpoint-every", "2", "--log-metrics", str(tmp_path / "m.jsonl")]) == 0
    j = _json_out(capsys)
    assert j["steps"] == 3 and j["resumed_from"] == 0
    assert os.path.isdir(os.path.join(out, "checkpoints", "step_2")) and not os.path.isdir(os.path.join(out, "checkpoints", "step_3"))
    lines = [json.loads(l) for l in open(tmp_path / "m.jsonl")]
    assert [l["step"] for l in lines] == [1, 2, 3]
    assert main(common + ["--max-steps", "4", "--resume"]) == 0
    j = _json_out(capsys)
    assert j["resumed_from"] == 2 and j["steps"] == 4


def test_distill_offline_rationale_and_checkpoints(model_dir, capsys, tmp_path):
    data = tmp_path / "d.jsonl"
    data.write_text("".join(json.dumps({"prompt": f"question {i} about several things"}) + "\n" for i in range(3)))
    cache = str(tmp_path / "cache")
    base = ["distill", "--teacher", model_dir, "--student", model_dir, "-d", str(data), "--device", "cpu"]
    assert main(base + ["--offline-generate", "--offline-cache", cache, "--offline-top-k", "16"]) == 0
    assert _json_out(capsys)["sequences"] == 3 and os.path.exists(os.path.join(cache, "metadata.json"))
    out = str(tmp_path / "o")
    assert main(base + ["--offline", "--offline-cache", cache, "-o", out, "--epochs", "1", "--lora-r", "4",
                        "--checkpoint-every", "2", "--log-metrics", str(tmp_path / "m.jsonl"), "--eval-dataset", str(data)]) == 0
    j = _json_out(capsys)
    assert j["steps"] == 3 and j["eval_samples"] == 3 and os.path.isdir(os.path.join(out, "checkpoints", "step_2"))
    assert len(open(tmp_path / "m.jsonl").read().splitlines()) == 3
    assert main(base + ["-o", out, "--max-steps", "4", "--lora-r", "4", "--resume", "--rationale", "--rationale-weight", "2.0"]) == 0
    assert _json_out(capsys)["resumed_from"] == 2
    assert main(base + ["--offline", "-o", out]) == 2                       # offline needs a cache directory


def test_rationale_loss_weights_uncertain_tokens():
    from pmetal_b200.distill import losses as L
    torch.manual_seed(0)
    s, t = torch.randn(6, 50), torch.randn(6, 50)
    t[:3] *= 8                                                              # confident teacher rows: low entropy
    plain = L.kl_divergence(s, t, 1.0) 
    lt, ls = torch.log_softmax(t, -1), torch.log_softmax(s, -1)
    kl = (lt.exp() * (lt - ls)).sum(-1)
    ent = -(lt.exp() * lt).sum(-1)
    w = 1 + 2.0 * ent / ent.max()
    assert torch.allclose(L.rationale_kl(s, t, 1.0, None, 2.0), (kl * w).sum() / w.sum(), atol=1e-6)
    assert torch.allclose(L.rationale_kl(s, t, 1.0, None, 0.0), plain, atol=1e-6)        # weight 0: the plain mean KL
    toks = torch.tensor([5, 1, 7, 8, 2, 9])
    assert L.reasoning_mask(toks, 1, 2).tolist() == [0, 1, 1, 1, 0, 0]
    only = L.rationale_kl(s, t, 1.0, None, 0.0, L.reasoning_mask(toks, 1, 2))
    assert torch.allclose(only, kl[1:4].mean(), atol=1e-6)


def test_tokenize_shards_then_pretrain_with_eval_and_resume(tmp_path, capsys):
    corpus = tmp_path / "c.jsonl"
    corpus.write_text("".join(json.dumps({"body": "the quick brown fox jumps over the lazy dog " * 6}) + "\n" for _ in range(25)))
    shards = str(tmp_path / "shards")
    assert main(["tokenize", "--tokenizer", "random:tiny-qwen3", "-i", str(corpus), "-o", shards, "--text-column", "body",
                 "--docs-per-shard", "10"]) == 0
    j = _json_out(capsys)
    assert j["shards"] == 3 and j["documents"] == 25 and sorted(os.listdir(shards))[0] == "shard_00000.bin"
    assert main(["tokenize", "-m", "random:tiny-qwen3", "--text", "hi"]) == 0 and _json_out(capsys)["count"] == 2
    out = str(tmp_path / "pt")
    base = ["pretrain", "--arch", "tiny-qwen3", "--shards", shards + "/shard_0000[01].bin", "--eval-shards",
            shards + "/shard_00002.bin", "-o", out, "--seq-len", "32", "--batch-size", "2", "--gradient-accumulation-steps", "2",
            "--learning-rate", "1e-3", "--warmup-steps", "1", "--eval-batches", "2", "--log-every", "2", "--device", "cpu"]
    assert main(base + ["--steps", "4", "--checkpoint-every", "2", "--eval-every", "2"]) == 0
    a = _json_out(capsys)
    assert a["step"] == 4 and a["eval_batches"] == 2 and a["tokens"] == 4 * 2 * 2 * 32 and os.path.isdir(os.path.join(out, "step_4"))
    assert main(base + ["--steps", "6", "--resume"]) == 0
    b = _json_out(capsys)
    assert b["resumed_from"].endswith("step_4") and b["step"] == 6


def test_fuse_merge_eval_embed_flag_forms(model_dir, capsys, tmp_path):
    from pmetal_b200.core.config import LoraConfig
    from pmetal_b200.lora import apply_lora
    from pmetal_b200.lora.adapter import save_adapter
    from pmetal_b200.models.loader import load_pretrained
    from pmetal_b200.utils.safetensors_io import load_file
    m, _, _ = load_pretrained(model_dir, dtype=torch.float32)
    cfg = LoraConfig(r=4, alpha=8.0)
    apply_lora(m, cfg)
    for n, p in m.named_parameters():
        if "lora_b" in n:
            torch.nn.init.normal_(p, std=0.05)
    ad = str(tmp_path / "ad")
    save_adapter(m, ad, cfg)
    outs = {}
    for name, extra in (("a", []), ("b", ["--low-memory"]), ("c", ["--fast"]), ("d", ["--alpha", "16"])):
        assert main(["fuse", "-m", model_dir, "-l", ad, "-o", str(tmp_path / name), "--dtype", "float32"] + extra) == 0
        outs[name] = load_file(str(tmp_path / name / "model.safetensors"))["model.layers.0.self_attn.q_proj.weight"]
    assert _json_out(capsys)["scale"] == 4.0                                       # alpha 16 / r 4
    base = load_file(os.path.join(model_dir, "model.safetensors"))["model.layers.0.self_attn.q_proj.weight"]
    assert torch.equal(outs["a"], outs["b"]) and torch.allclose(outs["a"], outs["c"], atol=1e-5)
    assert torch.allclose(outs["d"] - base, 2 * (outs["a"] - base), atol=1e-5)
    assert main(["merge", "--model-a", model_dir, "--model-b", str(tmp_path / "a"), "--method", "slerp", "--t", "0.0",
                 "-o", str(tmp_path / "s0"), "--dtype", "float32"]) == 0
    s0 = load_file(str(tmp_path / "s0" / "model.safetensors"))["model.layers.0.self_attn.q_proj.weight"]
    assert torch.allclose(s0, base, atol=1e-5)                                     # t = 0 returns model a
    assert main(["merge", "--model-a", model_dir, "--model-b", str(tmp_path / "a"), "--weight-a", "0.25", "--weight-b", "0.75",
                 "-o", str(tmp_path / "lin"), "--dtype", "float32"]) == 0
    lin = load_file(str(tmp_path / "lin" / "model.safetensors"))["model.layers.0.self_attn.q_proj.weight"]
    assert torch.allclose(lin, 0.25 * base + 0.75 * outs["a"], atol=1e-5)
    capsys.readouterr()
    data = tmp_path / "e.jsonl"
    data.write_text("".join(json.dumps({"text": "some words to score " * 4}) + "\n" for _ in range(5)))
    assert main(["eval", "-m", model_dir, "-d", str(data), "--num-samples", "2", "--json", "--device", "cpu"]) == 0
    assert _json_out(capsys)["samples"] == 2
    pairs = tmp_path / "pairs.jsonl"
    pairs.write_text("".join(json.dumps({"anchor": f"query {i}", "positive": f"answer {i}", "negative": f"other {i}"}) + "\n"
                             for i in range(6)))
    assert main(["embed-train", "-m", model_dir, "-d", str(pairs), "-o", str(tmp_path / "emb"), "--loss", "triplet", "--margin", "0.3",
                 "--epochs", "1", "--batch-size", "3", "--pooling", "last", "--no-normalize", "--weight-decay", "0.01",
                 "--log-every", "1", "--lora-r", "4", "--device", "cpu"]) == 0
    assert _json_out(capsys)["steps"] == 2


def test_cluster_flags_after_the_action_are_applied(monkeypatch):
    from pmetal_b200.parallel import cluster_cli
    seen = {}
    monkeypatch.setattr(cluster_cli, "run", lambda a: seen.update(vars(a)) or 0)
    assert main(["cluster", "pipeline-bench", "--gpus", "2", "--hidden-dim", "2048", "--tokens", "4096", "--mb", "8"]) == 0
    assert (seen["gpus"], seen["hidden_dim"], seen["tokens"], seen["mb"], seen["rest"]) == (2, 2048, 4096, 8, [])
    assert main(["cluster", "--gpus", "4", "bench", "--iters", "5"]) == 0
    assert (seen["gpus"], seen["iters"]) == (4, 5)
    assert main(["cluster", "train", "--", "-m", "x", "--gpus", "2"]) == 0           # flags of the launched command stay
    assert seen["rest"] == ["--", "-m", "x", "--gpus", "2"] or seen["rest"] == ["-m", "x", "--gpus", "2"]


def test_serve_over_two_ranks_answers_http(tmp_path):
    """``serve --tp 2`` starts one process per rank; rank 0 answers HTTP while rank 1 repeats its model calls."""
    import json
    import signal
    import subprocess
    import sys
    import time
    import urllib.request
    port = 18431
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.Popen([sys.executable, "-m", "pmetal_b200.cli.main", "serve", "-m", "random:tiny-qwen3-moe", "--tp", "2",
                          "--device", "cpu", "--port", str(port), "--kv-blocks", "64", "--max-slots", "4"], cwd=root,
                         start_new_session=True, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    try:
        up = False
        for _ in range(240):
            try:
                urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=1).read()
                up = True
                break
            except Exception:
                if p.poll() is not None:
                    break
                time.sleep(0.5)
        assert up, "server did not come up"
        outs = []
        for _ in range(2):
            req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/completions",
                                         data=json.dumps({"prompt": "hello world", "max_tokens": 8, "temperature": 0}).encode(),
                                         headers={"Content-Type": "application/json"})
            outs.append(json.loads(urllib.request.urlopen(req, timeout=120).read()))
        assert outs[0]["usage"]["completion_tokens"] == 8
        assert outs[0]["choices"][0]["text"] == outs[1]["choices"][0]["text"]
    finally:
        os.killpg(p.pid, signal.SIGINT)
        try:
            p.communicate(timeout=60)
        except subprocess.TimeoutExpired:
            os.killpg(p.pid, signal.SIGKILL)
            p.communicate()


def test_column_options_select_the_text_of_a_record():
    from types import SimpleNamespace as NS
    from pmetal_b200.cli.commands import record_text
    rec = {"q": "why?", "ctx": "because", "a": "so", "text": "plain"}
    assert record_text(rec) == "plain"
    assert record_text(rec, NS(text_column="ctx")) == "because"
    assert record_text(rec, NS(text_columns="q, ctx", column_separator=" | ")) == "why? | because"
    assert record_text(rec, NS(prompt_column="q", response_column="a")) == "why?"                      # rollout prompt only
    assert record_text(rec, NS(prompt_column="q", response_column="a", column_separator="\n"), with_response=True) == "why?\nso"
    assert record_text({"question": "x", "answer": "y"}, with_response=True) == "x\n\ny"
    assert record_text("bare") == "bare"


def test_grpo_takes_the_reference_flags(model_dir, capsys, tmp_path):
    data = tmp_path / "p.jsonl"
    data.write_text("".join(json.dumps({"a": f"part {i}", "b": "and more words to make the prompt long enough"}) + "\n" for i in range(2)))
    out = str(tmp_path / "g")
    from pmetal_b200.ops.functional import set_force_reference
    try:
        assert main(["grpo", "-m", model_dir, "-d", str(data), "-o", out, "--num-generations", "2", "--max-completion-length", "4",
                     "--text-columns", "a,b", "--column-separator", " ", "--max-seq-len", "8", "--no-flash-attention",
                     "--reward-model", model_dir, "--reward-model-max-length", "16",
                     "--reward-model-template", "Q: {prompt} A: {completion}", "--max-steps", "1", "--device", "cpu"]) == 0
    finally:
        set_force_reference(False)                     # the switch is process-wide
    assert _json_out(capsys)["steps"] == 1
    with pytest.raises(SystemExit):
        main(["grpo", "-m", model_dir, "-d", str(data), "-o", out, "--max-completion-length", "4", "--max-seq-len", "4",
              "--device", "cpu"])


def test_cluster_status_flags(capsys):
    assert main(["cluster", "status", "--json", "--no-discovery", "--result-port", "7"]) == 0
    doc = json.loads(capsys.readouterr().out.strip())
    assert doc["cluster"]["ports"]["results"] == 7
    assert main(["cluster", "up", "--wait", "0.25", "--status-interval", "0.1", "--json"]) == 0
    assert len(capsys.readouterr().out.strip().splitlines()) >= 2
    assert main(["cluster", "status", "--min-peers", "64"]) == 1


def test_bench_commands_take_the_reference_options(tmp_path, capsys):
    data = tmp_path / "d.jsonl"
    data.write_text("".join(json.dumps({"prompt": f"question number {i} " * 3, "response": "an answer " * 4}) + "\n" for i in range(6)))
    out = tmp_path / "w.json"
    assert main(["bench-workload", "-m", "random:tiny-qwen3", "--device", "cpu", "--dataset", str(data), "--prompt-samples", "2",
                 "--max-prompt-tokens", "24", "--decode-steps", "3", "--inference-warmup-passes", "1",
                 "--inference-session-repeats", "2", "--inference-repeats", "2", "--inference-context", "prompt",
                 "--train-samples", "2", "--train-steps", "1", "--max-seq-len", "64", "--json", "-o", str(out)]) == 0
    doc = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    g = doc["generation"]
    assert g["batch"] == 2 and g["decode_steps"] == 3 and g["sessions"] == 2 and g["warmup_passes"] == 1 and g["timed_passes"] == 4
    assert max(g["prompt_tokens"]) <= 24 and doc["inference_context"] == "prompt"
    assert doc["training"]["steps"] == 1 and doc["training"]["samples_per_step"] == 2
    assert json.load(open(out))["generation"]["batch"] == 2
    assert main(["bench-gen", "-m", "random:tiny-qwen3", "--device", "cpu", "--preset", "quick"]) == 0
    doc = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert doc["preset"] == "quick" and doc["generation"]["decode_steps"] == 8 and "training" not in doc
    for stage in ("prefill", "input-proj", "out-proj"):
        assert main(["bench-gdn", "--stage", stage, "--seq-len", "16", "--heads", "2", "--device", "cpu", "--warmup-iterations", "0",
                     "--benchmark-iterations", "1", "-o", str(tmp_path / "g.json")]) == 0
        assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["stage"] == stage
    assert json.load(open(tmp_path / "g.json"))["stage"] == "out-proj"


def test_dashboard_follows_a_metrics_file_and_modelfile_carries_a_license(tmp_path, capsys):
    m = tmp_path / "m.jsonl"
    m.write_text('{"step": 1, "loss": 2.5}\n{"step": 2, "loss": 2.25, "reward": 0.5}\n')
    assert main(["dashboard", "--metrics-file", str(m), "--once"]) == 0
    row = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert row["job"] == "metrics" and row["step"] == 2 and row["loss"] == 2.25 and row["reward"] == 0.5
    assert main(["dashboard", "--once"]) == 2
    capsys.readouterr()
    mf = tmp_path / "Modelfile"
    assert main(["ollama", "modelfile", "--gguf", str(tmp_path / "x.gguf"), "--license", "Apache-2.0", "-o", str(mf)]) == 0
    assert 'LICENSE """Apache-2.0"""' in mf.read_text()
