"""The package-level Python interface: names the reference's bindings export, and the pieces added on top."""
import json
import os

import pytest
import torch

import pmetal_b200 as pm


def test_every_exported_name_resolves():
    for name in ("LoraConfig", "TrainingConfig", "GenerationConfig", "DataLoaderConfig", "Dtype", "Quantization", "LoraBias",
                 "LrSchedulerType", "OptimizerType", "DatasetFormat", "ModelArchitecture", "download_model", "download_file",
                 "Model", "DFlashGenerator", "Tokenizer", "Trainer", "ProgressCallback", "LoggingCallback",
                 "MetricsJsonCallback", "finetune", "infer"):
        assert getattr(pm, name) is not None, name
    assert set(pm.__all__) >= {"Model", "Trainer", "DFlashGenerator"}


def test_dflash_generator_equals_plain_greedy_decoding():
    g = pm.DFlashGenerator("random:tiny-qwen3", "random", device="cpu")
    try:
        prompt = [5, 6, 7, 8]
        toks, metrics = g.generate(prompt, max_new_tokens=10)
        assert toks[:4] == prompt and len(toks) == 14 and metrics["generated_tokens"] == 10
        assert metrics["steps"] >= 1 and 0.0 <= metrics["acceptance_rate"] <= 1.0
        # plain greedy decoding of the target
        cache = g.target.new_cache()
        cur, want = torch.tensor([prompt]), []
        with torch.no_grad():
            for _ in range(10):
                nxt = int(g.target(cur, cache)[0, -1].argmax())
                want.append(nxt)
                cur = torch.tensor([[nxt]])
        assert toks[4:] == want
        tree, _ = g.generate(prompt, max_new_tokens=10, tree_budget=6)
        assert tree == toks
        stopped, _ = g.generate(prompt, max_new_tokens=10, stop_tokens=[want[2]])
        assert stopped[4:] == want[:want.index(want[2]) + 1]
        with pytest.raises(ValueError):
            g.generate(prompt, temperature=0.7)
        assert "DFlashGenerator" in repr(g)
    finally:
        g.close()


def test_tokenizer_from_pretrained_and_special_ids(tmp_path):
    from tokenizers import Tokenizer as HfTok
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace
    tok = HfTok(WordLevel({"<unk>": 0, "<s>": 1, "</s>": 2, "hello": 3, "world": 4}, unk_token="<unk>"))
    tok.pre_tokenizer = Whitespace()
    tok.save(str(tmp_path / "tokenizer.json"))
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"bos_token": "<s>", "eos_token": {"content": "</s>"}}))
    t = pm.Tokenizer.from_pretrained(str(tmp_path))
    assert (t.bos_token_id, t.eos_token_id, t.unk_token_id) == (1, 2, 0)
    assert t.pad_token_id == 2 and t.vocab_size == 5
    assert t.encode("hello there world") == [3, 0, 4] and t.decode([3, 4]) == "hello world"
    t2 = pm.Tokenizer.from_pretrained(str(tmp_path / "tokenizer.json"))
    assert t2.encode("world") == [4] and t2.unk_token_id == 0


def test_model_reports_its_architecture():
    m = pm.Model.load("random:tiny-qwen3", device="cpu")
    assert m.architecture == "qwen3"
