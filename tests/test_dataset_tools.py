"""``pmetal dataset`` actions: validate, preview, filter, split, merge, sample, template, prepare, formats."""
import json

import pytest

from pmetal_b200.cli.main import main
from pmetal_b200.data import tools as dt
from pmetal_b200.data.tokenizer import ByteTokenizer


def _write(path, rows):
    path.write_text("".join((r if isinstance(r, str) else json.dumps(r)) + "\n" for r in rows))
    return str(path)


def _read(path):
    return [json.loads(l) for l in open(path) if l.strip()]


ROWS = [{"instruction": "add", "input": "1 2", "output": "3", "kind": "math"},
        {"conversations": [{"from": "human", "value": "hi"}, {"from": "gpt", "value": "hello there"}], "kind": "chat"},
        {"messages": [{"role": "user", "content": "q"}, {"role": "assistant", "content": ""}], "kind": "chat"},
        {"text": "plain text sample", "kind": "text"},
        {"text": "plain text sample", "kind": "text"},
        {"prompt": "p", "response": "a longer response " * 20, "kind": "math"}]


def test_validate_counts_problems(tmp_path):
    path = _write(tmp_path / "d.jsonl", ROWS[:2] + ["{not json", {"other": 1}, {"text": "   "}, {"text": "x" * 100}])
    rep = dt.validate(path, ByteTokenizer(), max_seq_len=50)
    assert (rep["total"], rep["valid"], rep["parse_errors"], rep["empty"], rep["too_long"]) == (6, 2, 1, 2, 1)
    assert not rep["ok"] and any("JSON parse error" in i for i in rep["issues"])
    good = _write(tmp_path / "g.jsonl", ROWS[:2])
    assert dt.validate(good)["ok"]
    assert main(["dataset", "validate", good]) == 0 and main(["dataset", "validate", "-p", path]) == 1


def test_filter_split_merge_sample():
    tok = ByteTokenizer()
    kept, rep = dt.filter_records(ROWS, tok, min_tokens=5, max_tokens=200, dedup=True, complete_only=True)
    assert rep["removed"] == {"length": 1, "duplicate": 1, "pattern": 0, "incomplete": 1, "no_text": 0} and len(kept) == 3
    assert len(dt.filter_records(ROWS, pattern="plain")[0]) == 2
    assert len(dt.filter_records(ROWS, pattern="plain", invert=True)[0]) == 4
    with pytest.raises(ValueError):
        dt.filter_records(ROWS, None, min_tokens=3)
    many = [{"text": f"t{i}", "kind": "a" if i % 4 else "b"} for i in range(200)]
    parts = dt.split_records(many, 0.1, 0.1, seed=1, stratify="kind")
    assert (len(parts["train"]), len(parts["val"]), len(parts["test"])) == (160, 20, 20)
    assert sum(r["kind"] == "b" for r in parts["val"]) == 5                      # 50 of 200 are "b": 10 % of them
    assert sorted(r["text"] for p in parts.values() for r in p) == sorted(r["text"] for r in many)
    assert parts == dt.split_records(many, 0.1, 0.1, seed=1, stratify="kind")   # deterministic
    a, b = [{"text": f"a{i}"} for i in range(4)], [{"text": f"b{i}"} for i in range(2)]
    assert [r["text"] for r in dt.merge_records([a, b], interleave=True)] == ["a0", "b0", "a1", "b1", "a2", "a3"]
    assert len(dt.merge_records([a, b], weights=[0.5, 2.0])) == 2 + 4
    assert len(dt.sample_records(many, 7, seed=3)) == 7 and dt.sample_records(many, 7, 3) == dt.sample_records(many, 7, 3)


def test_template_and_prepare(tmp_path):
    out, rep = dt.apply_template(ROWS[:2] + [ROWS[3], {"junk": 1}], "chatml", system="be brief", mask_prompt=True)
    assert rep == {"input": 4, "formatted": 3, "skipped": 1, "template": "chatml"}
    assert out[0]["text"].startswith("<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\nadd\n\n1 2<|im_end|>")
    assert out[0]["text"].startswith(out[0]["prompt"]) and out[0]["text"][len(out[0]["prompt"]):].startswith("3")
    assert "hello there" in out[1]["text"] and out[2] == {"text": "plain text sample"}
    raw, _ = dt.apply_template(ROWS[:1], "raw")
    assert raw[0]["text"] == "add\n\n1 2\n\n3"
    llama, _ = dt.apply_template(ROWS[:1], "llama3", add_generation_prompt=True)
    assert "<|start_header_id|>user<|end_header_id|>" in llama[0]["text"]
    src = _write(tmp_path / "src.jsonl", [{"problem": f"q{i}", "solution": f"a{i}"} for i in range(40)] +
                 [{"problem": "q0", "solution": "a0"}, {"problem": "long", "solution": "z" * 5000}])
    rep = dt.prepare(src, str(tmp_path / "out"), ByteTokenizer(), None, "chatml", 512, 0.1, 0, True,
                     "instruction=problem,output=solution")
    assert rep["read"] == 42 and rep["removed"]["duplicate"] == 1 and rep["removed"]["length"] == 1
    assert rep["train"] + rep["val"] == 40 and rep["val"] == 4
    rows = _read(rep["files"]["train"])
    assert all(set(r) == {"text", "prompt"} for r in rows) and json.load(open(tmp_path / "out" / "prepare_report.json"))["train"] == 36


def test_cli_round_trip(tmp_path, capsys):
    src = _write(tmp_path / "d.jsonl", ROWS)
    assert main(["dataset", "filter", "-i", src, "-o", str(tmp_path / "f.jsonl"), "--dedup"]) == 0
    assert len(_read(tmp_path / "f.jsonl")) == 5
    assert main(["dataset", "filter", "-i", src, "-o", str(tmp_path / "x.jsonl"), "--min-tokens", "3"]) == 2
    assert main(["dataset", "split", "-i", src, "-o", str(tmp_path / "s"), "--val-ratio", "0.34"]) == 0
    assert len(_read(tmp_path / "s" / "train.jsonl")) + len(_read(tmp_path / "s" / "val.jsonl")) == 6
    assert main(["dataset", "merge", "-i", src, str(tmp_path / "f.jsonl"), "-o", str(tmp_path / "m.jsonl"), "--shuffle"]) == 0
    assert len(_read(tmp_path / "m.jsonl")) == 11
    assert main(["dataset", "sample", "-i", src, "-o", str(tmp_path / "p.jsonl"), "-n", "2"]) == 0
    assert len(_read(tmp_path / "p.jsonl")) == 2
    assert main(["dataset", "template", "-i", src, "-o", str(tmp_path / "t.jsonl"), "--template", "gemma"]) == 0
    assert "<start_of_turn>" in _read(tmp_path / "t.jsonl")[0]["text"]
    capsys.readouterr()
    assert main(["dataset", "preview", src, "-n", "2"]) == 0
    pv = json.loads(capsys.readouterr().out)
    assert len(pv["samples"]) == 2 and "instruction" in pv["columns"]
    assert main(["dataset", "prepare", src, "-o", str(tmp_path / "prep"), "-m", "random:tiny-qwen3", "--val-ratio", "0.2"]) == 0
    assert main(["dataset", "formats"]) == 0 and "chatml" in capsys.readouterr().out
    assert main(["dataset", "preview", "org/not-local"]) == 2
