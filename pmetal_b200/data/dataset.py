"""Dataset loading and tokenisation.

Formats and their detection by the first JSONL record follow the reference
(crates/pmetal-data/src/dataset.rs:563-590): ``text`` → simple, ``instruction`` → Alpaca,
``conversations`` → ShareGPT, ``messages`` → OpenAI, ``problem``/``thinking`` → reasoning;
plus custom column mapping with optional prompt/response masking (dataset.rs:112-165,
631-727). Tokenisation keeps special tokens, truncates to ``max_seq_len`` and produces
*unshifted* labels with the prompt prefix set to −100 (dataset.rs:938-972).
JSONL, JSON arrays, CSV and Parquet inputs are accepted.
"""
from __future__ import annotations

import csv
import json
import os
import random
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence

from .chat_templates import ChatTemplate, Message
from .packing import IGNORE_INDEX, Sample

FORMATS = ("auto", "simple", "alpaca", "sharegpt", "openai", "reasoning", "custom")


@dataclass
class TextSample:
    text: str
    prompt: Optional[str] = None


@dataclass
class CustomColumns:
    text_column: str = "text"
    text_columns: Optional[List[str]] = None
    column_separator: str = "\n"
    prompt_column: Optional[str] = None
    response_column: Optional[str] = None


def detect_format(record: dict) -> str:
    if "text" in record:
        return "simple"
    if "instruction" in record:
        return "alpaca"
    if "conversations" in record:
        return "sharegpt"
    if "messages" in record:
        return "openai"
    if "problem" in record or "thinking" in record:
        return "reasoning"
    raise ValueError("Could not detect dataset format. Expected 'text', 'instruction', 'conversations', "
                     "'messages', or 'problem' field.")


def _extract_text(val) -> str:
    if isinstance(val, str):
        return val
    if isinstance(val, list):
        parts = []
        for item in val:
            if isinstance(item, dict):
                c = item.get("content", item.get("value"))
                if isinstance(c, str):
                    role = item.get("role", item.get("from"))
                    parts.append(f"{role}: {c}" if isinstance(role, str) else c)
        return "\n".join(parts) if parts else json.dumps(val)
    if isinstance(val, bool):
        return "true" if val else "false"
    if isinstance(val, (int, float)):
        return str(val)
    return json.dumps(val)


def _basic_chat(pairs) -> TextSample:
    names = {"human": "User", "user": "User", "gpt": "Assistant", "assistant": "Assistant", "system": "System"}
    text, prompt_end = "", 0
    for role, content in pairs:
        text += f"{names.get(role, role)}: {content}\n\n"
        if role in ("human", "user", "system"):
            prompt_end = len(text)
    return TextSample(text, text[:prompt_end] if prompt_end > 0 else None)


def parse_record(rec: dict, fmt: str, template: Optional[ChatTemplate] = None,
                 custom: Optional[CustomColumns] = None) -> TextSample:
    if fmt == "simple":
        return TextSample(rec["text"])
    if fmt == "alpaca":
        inp = rec.get("input", "") or ""
        prompt = (f"### Instruction:\n{rec['instruction']}\n\n### Response:\n" if not inp else
                  f"### Instruction:\n{rec['instruction']}\n\n### Input:\n{inp}\n\n### Response:\n")
        return TextSample(prompt + rec.get("output", ""), prompt)
    if fmt in ("sharegpt", "openai"):
        if fmt == "sharegpt":
            pairs = [(m.get("from", ""), m.get("value", "")) for m in rec["conversations"]]
            norm = [("assistant" if r in ("gpt", "assistant") else r, c) for r, c in pairs]
        else:
            pairs = norm = [(m.get("role", ""), m.get("content", "") or "") for m in rec["messages"]]
        if template is not None:
            f = template.apply([Message("user" if r == "human" else r, c) for r, c in norm])
            return TextSample(f.text, f.prompt())
        return _basic_chat(pairs)
    if fmt == "reasoning":
        problem, thinking, solution = rec.get("problem", ""), rec.get("thinking", ""), rec.get("solution", "")
        resp = solution if not thinking else f"<think>\n{thinking}\n</think>\n\n{solution}"
        return TextSample(f"{problem}\n\n{resp}", problem)
    if fmt == "custom":
        c = custom or CustomColumns()
        if c.text_columns:
            parts = [_extract_text(rec[k]) for k in c.text_columns if k in rec]
            if not parts:
                raise ValueError(f"None of the requested columns {c.text_columns} were present")
            text = c.column_separator.join(parts)
            if c.prompt_column:
                p = rec.get(c.prompt_column)
                p = p if isinstance(p, str) else None
                if p is not None and c.prompt_column not in c.text_columns:
                    return TextSample(f"{p}{c.column_separator}{text}", p)
                return TextSample(text, p)
            return TextSample(text)
        if c.prompt_column and c.response_column:
            p, r = rec.get(c.prompt_column) or "", rec.get(c.response_column) or ""
            return TextSample(str(p) + str(r), str(p))
        if c.text_column not in rec:
            raise ValueError(f"Column '{c.text_column}' not found")
        p = rec.get(c.prompt_column) if c.prompt_column else None
        return TextSample(_extract_text(rec[c.text_column]), p if isinstance(p, str) else None)
    raise ValueError(f"unknown format {fmt}")


def read_records(path: str, max_samples: Optional[int] = None) -> List[dict]:
    low = path.lower()
    out: List[dict] = []
    if low.endswith(".parquet"):
        import pyarrow.parquet as pq
        out = pq.read_table(path).to_pylist()
    elif low.endswith(".csv"):
        with open(path, newline="", encoding="utf-8") as fh:
            out = list(csv.DictReader(fh))
    elif low.endswith(".json"):
        with open(path, "r", encoding="utf-8") as fh:
            data = json.load(fh)
        out = data if isinstance(data, list) else data.get("data", [data])
    else:
        with open(path, "r", encoding="utf-8") as fh:
            for i, line in enumerate(fh):
                line = line.strip()
                if not line:
                    continue
                try:
                    out.append(json.loads(line))
                except json.JSONDecodeError as e:
                    raise ValueError(f"Line {i + 1}: {e}") from e
                if max_samples and len(out) >= max_samples:
                    break
    return out[:max_samples] if max_samples else out


def tokenize_sample(ts: TextSample, tokenizer, max_length: int) -> Sample:
    ids = tokenizer.encode_with_special_tokens(ts.text)[:max_length]
    labels = list(ids)
    if ts.prompt is not None:
        n = min(len(tokenizer.encode_with_special_tokens(ts.prompt)), len(ids))
        labels[:n] = [IGNORE_INDEX] * n
    return Sample(ids, labels, [1] * len(ids))


class TrainingDataset:
    def __init__(self, samples: List[Sample], fmt: str = "simple"):
        self.samples, self.format = samples, fmt

    def __len__(self):
        return len(self.samples)

    def __getitem__(self, i):
        return self.samples[i]

    @classmethod
    def from_file_tokenized(cls, path: str, tokenizer, max_seq_len: int, fmt: str = "auto",
                            template: Optional[ChatTemplate] = None, custom: Optional[CustomColumns] = None,
                            max_samples: Optional[int] = None, shuffle: bool = False,
                            seed: int = 42) -> "TrainingDataset":
        recs = read_records(path, max_samples)
        if not recs:
            raise ValueError(f"dataset {path} is empty")
        if fmt == "auto":
            fmt = detect_format(recs[0])
        samples = [tokenize_sample(parse_record(r, fmt, template, custom), tokenizer, max_seq_len) for r in recs]
        samples = [s for s in samples if len(s) > 0]
        if shuffle:
            random.Random(seed).shuffle(samples)
        return cls(samples, fmt)

    from_jsonl_tokenized = from_file_tokenized

    def split(self, eval_fraction: float, seed: int = 42):
        idx = list(range(len(self.samples)))
        random.Random(seed).shuffle(idx)
        n_eval = int(len(idx) * eval_fraction)
        ev = [self.samples[i] for i in idx[:n_eval]]
        tr = [self.samples[i] for i in idx[n_eval:]]
        return TrainingDataset(tr, self.format), TrainingDataset(ev, self.format)

    def stats(self) -> Dict[str, float]:
        lens = sorted(len(s) for s in self.samples)
        if not lens:
            return {"num_samples": 0}
        trainable = sum(sum(1 for l in s.labels if l != IGNORE_INDEX) for s in self.samples if s.labels)
        return {"num_samples": len(lens), "total_tokens": sum(lens), "trainable_tokens": trainable,
                "min_len": lens[0], "max_len": lens[-1], "mean_len": sum(lens) / len(lens),
                "p50": lens[len(lens) // 2], "p95": lens[min(int(len(lens) * 0.95), len(lens) - 1)],
                "p99": lens[min(int(len(lens) * 0.99), len(lens) - 1)]}
