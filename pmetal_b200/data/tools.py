"""Dataset utilities behind ``pmetal dataset <action>``: validate, preview, filter, split, merge, sample, template,
prepare and formats (crates/pmetal/src/commands/dataset.rs:464-1600; argument definitions in
crates/pmetal/src/main.rs:586-870). Everything works on JSONL records (dicts); reading other containers goes through
``dataset.read_records``. Each function returns a small report dict that the command line prints as JSON."""
from __future__ import annotations

import hashlib
import json
import os
import random
import re
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

from . import dataset as ds
from .chat_templates import ChatTemplate, Message

TEMPLATE_CHOICES = ("chatml", "llama3", "llama2", "mistral", "qwen", "phi", "gemma", "raw", "auto")
_TEMPLATE_ALIAS = {"phi": "phi3", "qwen": "chatml"}


def write_jsonl(records: Iterable[dict], path: str) -> int:
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    n = 0
    with open(path, "w", encoding="utf-8") as fh:
        for r in records:
            fh.write(json.dumps(r, ensure_ascii=False) + "\n")
            n += 1
    return n


def record_text(rec: dict) -> Optional[str]:
    """All the text of a record, for length checks, pattern matching and de-duplication; None when the record has no
    recognisable text field."""
    if isinstance(rec.get("text"), str):
        return rec["text"]
    for key, field in (("conversations", "value"), ("messages", "content")):
        turns = rec.get(key)
        if isinstance(turns, list):
            return " ".join(str(t.get(field, "")) for t in turns if isinstance(t, dict))
    if isinstance(rec.get("instruction"), str):
        return " ".join(str(rec.get(k) or "") for k in ("instruction", "input", "output"))
    if isinstance(rec.get("prompt"), str):
        return " ".join(str(rec.get(k) or "") for k in ("prompt", "response", "completion", "chosen"))
    return None


def record_turns(rec: dict) -> Optional[List[Tuple[str, str]]]:
    """(role, content) turns of a conversation-style or instruction-style record."""
    roles = {"human": "user", "gpt": "assistant", "bot": "assistant"}
    if isinstance(rec.get("conversations"), list):
        return [(roles.get(str(t.get("from", "")), str(t.get("from", ""))), str(t.get("value", "")))
                for t in rec["conversations"] if isinstance(t, dict)]
    if isinstance(rec.get("messages"), list):
        return [(str(t.get("role", "")), str(t.get("content", ""))) for t in rec["messages"] if isinstance(t, dict)]
    if isinstance(rec.get("instruction"), str):
        user = rec["instruction"] + (("\n\n" + rec["input"]) if rec.get("input") else "")
        return [("user", user), ("assistant", str(rec.get("output", "")))]
    if isinstance(rec.get("prompt"), str):
        return [("user", rec["prompt"]), ("assistant", str(rec.get("response") or rec.get("completion") or ""))]
    return None


# ------------------------------------------------------------------------------------------------ validate / preview
def validate(path: str, tokenizer=None, max_seq_len: int = 2048) -> dict:
    """Line-by-line check of a JSONL file: JSON syntax, a recognisable non-empty text field and (with a tokenizer) the
    token count against ``max_seq_len``. Samples that are too long do not make the dataset invalid (they are
    truncated in training); parse errors and empty samples do."""
    total = valid = too_long = empty = parse_errors = 0
    issues: List[str] = []
    with open(path, "r", encoding="utf-8", errors="replace") as fh:
        for no, line in enumerate(fh, 1):
            if not line.strip():
                continue
            total += 1
            try:
                rec = json.loads(line)
            except ValueError as e:
                parse_errors += 1
                issues.append(f"line {no}: JSON parse error: {e}")
                continue
            text = record_text(rec) if isinstance(rec, dict) else None
            if text is None:
                empty += 1
                issues.append(f"line {no}: no recognisable text field")
                continue
            if not text.strip():
                empty += 1
                issues.append(f"line {no}: empty text content")
                continue
            if tokenizer is not None:
                n = len(tokenizer.encode(text))
                if n > max_seq_len:
                    too_long += 1
                    issues.append(f"line {no}: token length {n} exceeds max_seq_len {max_seq_len}")
                    continue
            valid += 1
    return {"path": path, "total": total, "valid": valid, "parse_errors": parse_errors, "empty": empty,
            "too_long": too_long, "max_seq_len": max_seq_len, "ok": parse_errors == 0 and empty == 0,
            "issues": issues[:10], "more_issues": max(len(issues) - 10, 0)}


def preview(path: str, num: int = 5) -> dict:
    recs = ds.read_records(path, max_samples=num)
    return {"path": path, "format": ds.detect_format(recs[0]) if recs else None,
            "columns": sorted({k for r in recs for k in r}), "samples": recs[:num]}


# ------------------------------------------------------------------------------------------------ filter / split
def filter_records(records: Sequence[dict], tokenizer=None, min_tokens: Optional[int] = None,
                   max_tokens: Optional[int] = None, dedup: bool = False, pattern: Optional[str] = None,
                   invert: bool = False, complete_only: bool = False) -> Tuple[List[dict], dict]:
    """Keep the records that pass every active criterion; the report counts what each criterion removed."""
    if (min_tokens is not None or max_tokens is not None) and tokenizer is None:
        raise ValueError("token-count filters need a tokenizer (--model)")
    rx = re.compile(pattern) if pattern else None
    seen = set()
    kept: List[dict] = []
    removed = {"length": 0, "duplicate": 0, "pattern": 0, "incomplete": 0, "no_text": 0}
    for rec in records:
        text = record_text(rec)
        if text is None:
            removed["no_text"] += 1
            continue
        if complete_only:
            turns = record_turns(rec)
            if turns is not None:
                speakers = [r for r, _ in turns if r != "system"]
                if not speakers or speakers[-1] != "assistant" or any(not c.strip() for _, c in turns):
                    removed["incomplete"] += 1
                    continue
        if rx is not None and (rx.search(text) is None) != invert:
            removed["pattern"] += 1
            continue
        if tokenizer is not None and (min_tokens is not None or max_tokens is not None):
            n = len(tokenizer.encode(text))
            if (min_tokens is not None and n < min_tokens) or (max_tokens is not None and n > max_tokens):
                removed["length"] += 1
                continue
        if dedup:
            h = hashlib.sha1(text.encode("utf-8")).digest()
            if h in seen:
                removed["duplicate"] += 1
                continue
            seen.add(h)
        kept.append(rec)
    return kept, {"input": len(records), "kept": len(kept), "removed": removed}


def split_records(records: Sequence[dict], val_ratio: float = 0.1, test_ratio: float = 0.0, seed: int = 42,
                  stratify: Optional[str] = None) -> Dict[str, List[dict]]:
    """Shuffled train / validation / test split; with ``stratify`` every value of that field is split with the same
    ratios, so the class mix of each part matches the whole."""
    if val_ratio < 0 or test_ratio < 0 or val_ratio + test_ratio >= 1:
        raise ValueError("val_ratio + test_ratio must be in [0, 1)")
    rnd = random.Random(seed)
    groups: Dict[str, List[dict]] = {}
    for r in records:
        groups.setdefault(str(r.get(stratify)) if stratify else "", []).append(r)
    out = {"train": [], "val": [], "test": []}
    for key in sorted(groups):
        g = list(groups[key])
        rnd.shuffle(g)
        n_val, n_test = int(round(len(g) * val_ratio)), int(round(len(g) * test_ratio))
        out["val"] += g[:n_val]
        out["test"] += g[n_val:n_val + n_test]
        out["train"] += g[n_val + n_test:]
    for part in out.values():
        rnd.shuffle(part)
    return out


# ------------------------------------------------------------------------------------------------ merge / sample
def merge_records(datasets: Sequence[Sequence[dict]], shuffle: bool = False, seed: int = 42, interleave: bool = False,
                  weights: Optional[Sequence[float]] = None) -> List[dict]:
    """Concatenate (default), alternate (``interleave``: round-robin until every input is exhausted) or resample by
    weight (``weights``: input i contributes ``round(len_i * w_i)`` records, drawn with replacement only when the
    weight is above 1)."""
    rnd = random.Random(seed)
    parts = [list(d) for d in datasets]
    if weights is not None:
        if len(weights) != len(parts):
            raise ValueError("one weight per input dataset is required")
        scaled = []
        for d, w in zip(parts, weights):
            n = int(round(len(d) * float(w)))
            if n <= len(d):
                scaled.append(rnd.sample(d, n))
            else:
                scaled.append(d * (n // max(len(d), 1)) + rnd.sample(d, n % max(len(d), 1)) if d else [])
        parts = scaled
    if interleave:
        out, i = [], 0
        while any(i < len(p) for p in parts):
            out.extend(p[i] for p in parts if i < len(p))
            i += 1
    else:
        out = [r for p in parts for r in p]
    if shuffle:
        rnd.shuffle(out)
    return out


def sample_records(records: Sequence[dict], num: int, seed: int = 42) -> List[dict]:
    return random.Random(seed).sample(list(records), min(num, len(records)))


# ------------------------------------------------------------------------------------------------ template / prepare
def _template_for(name: str, model_dir: Optional[str]) -> Optional[ChatTemplate]:
    if name == "raw":
        return None
    if name == "auto":
        if not model_dir:
            raise ValueError("--template auto needs --model (the tokenizer's own chat template)")
        return ChatTemplate.from_model_dir(model_dir)
    return ChatTemplate(_TEMPLATE_ALIAS.get(name, name))


def apply_template(records: Sequence[dict], template: str = "chatml", system: Optional[str] = None,
                   model_dir: Optional[str] = None, add_generation_prompt: bool = False,
                   mask_prompt: bool = False) -> Tuple[List[dict], dict]:
    """Conversation / instruction records -> ``{"text": formatted}``; with ``mask_prompt`` the output also carries
    ``"prompt"`` (everything before the last assistant turn) so that training computes the loss on the response only.
    Records that already are plain text pass through."""
    tpl = _template_for(template, model_dir)
    out, skipped = [], 0
    for rec in records:
        turns = record_turns(rec)
        if turns is None:
            if isinstance(rec.get("text"), str):
                out.append({"text": rec["text"]})
            else:
                skipped += 1
            continue
        if system and not any(r == "system" for r, _ in turns):
            turns = [("system", system)] + turns
        elif system:
            turns = [(r, system if r == "system" else c) for r, c in turns]
        if tpl is None:
            text = "\n\n".join(c for _, c in turns)
            start = len(text) - len(turns[-1][1]) if turns and turns[-1][0] == "assistant" else len(text)
        else:
            fc = tpl.apply([Message(r, c) for r, c in turns])
            text, start = fc.text, fc.response_start
            if add_generation_prompt:
                text += tpl.generation_prefix()
        row = {"text": text}
        if mask_prompt:
            row["prompt"] = text[:start]
        out.append(row)
    return out, {"input": len(records), "formatted": len(out), "skipped": skipped, "template": template}


def remap_columns(records: Sequence[dict], mapping: Optional[str]) -> List[dict]:
    """``"target=source,target=source"``: copy source columns to the standard names."""
    if not mapping:
        return list(records)
    pairs = [p.split("=", 1) for p in mapping.split(",") if "=" in p]
    return [{**r, **{t.strip(): r[s.strip()] for t, s in pairs if s.strip() in r}} for r in records]


def prepare(source: str, output_dir: str, tokenizer, model_dir: Optional[str] = None, template: str = "chatml",
            max_seq_len: int = 2048, val_ratio: float = 0.05, seed: int = 42, dedup: bool = True,
            columns: Optional[str] = None) -> dict:
    """The whole pipeline: read -> remap columns -> apply the chat template -> de-duplicate -> drop samples longer
    than ``max_seq_len`` tokens -> split -> write ``train.jsonl`` / ``val.jsonl`` and ``prepare_report.json``."""
    recs = remap_columns(ds.read_records(source), columns)
    formatted, trep = apply_template(recs, template, None, model_dir, False, True)
    kept, frep = filter_records(formatted, tokenizer, None, max_seq_len, dedup)
    parts = split_records(kept, val_ratio, 0.0, seed)
    os.makedirs(output_dir, exist_ok=True)
    files = {}
    for name in ("train", "val"):
        if parts[name] or name == "train":
            files[name] = os.path.join(output_dir, f"{name}.jsonl")
            write_jsonl(parts[name], files[name])
    rep = {"source": source, "read": len(recs), "formatted": trep["formatted"], "skipped": trep["skipped"],
           "removed": frep["removed"], "train": len(parts["train"]), "val": len(parts["val"]), "files": files,
           "template": template, "max_seq_len": max_seq_len}
    with open(os.path.join(output_dir, "prepare_report.json"), "w", encoding="utf-8") as fh:
        json.dump(rep, fh, indent=2)
    return rep


def formats() -> dict:
    return {"input_containers": ["jsonl", "json", "parquet", "csv"],
            "record_formats": {"text": '{"text": ...}', "alpaca": '{"instruction", "input", "output"}',
                               "sharegpt": '{"conversations": [{"from", "value"}]}',
                               "messages": '{"messages": [{"role", "content"}]}',
                               "prompt_response": '{"prompt", "response" | "completion"}',
                               "custom": "--text-column / --text-columns / --prompt-column + --response-column"},
            "templates": list(TEMPLATE_CHOICES)}
