"""Tokenizer wrapper.

Loads ``tokenizer.json`` with the Hugging Face ``tokenizers`` library (the same engine
the reference wraps, crates/pmetal-data/src/tokenizer.rs:28-270) and exposes
``encode`` / ``encode_with_special_tokens`` / ``decode`` plus pad/eos/bos ids read
from ``tokenizer_config.json`` / ``config.json``. ``ByteTokenizer`` is a dependency-free
byte-level fallback used for random-init models and tests.
"""
from __future__ import annotations

import json
import os
from typing import List, Optional


class Tokenizer:
    def __init__(self, tok, bos_id=None, eos_id=None, pad_id=None, eos_token: Optional[str] = None):
        self._tok = tok
        self.bos_token_id, self.eos_token_id = bos_id, eos_id
        self.pad_token_id = pad_id if pad_id is not None else (eos_id if eos_id is not None else 0)
        self.eos_token = eos_token

    @classmethod
    def from_file(cls, path: str) -> "Tokenizer":
        from tokenizers import Tokenizer as HfTok
        return cls(HfTok.from_file(path))

    @classmethod
    def from_model_dir(cls, model_dir: str) -> "Tokenizer":
        tj = os.path.join(model_dir, "tokenizer.json")
        if not os.path.exists(tj):
            return ByteTokenizer()
        from tokenizers import Tokenizer as HfTok
        tok = HfTok.from_file(tj)
        bos = eos = pad = None
        eos_s = None
        tc = os.path.join(model_dir, "tokenizer_config.json")
        if os.path.exists(tc):
            with open(tc, "r", encoding="utf-8") as fh:
                c = json.load(fh)

            def tid(key):
                v = c.get(key)
                v = v.get("content") if isinstance(v, dict) else v
                return (tok.token_to_id(v), v) if v else (None, None)
            (bos, _), (eos, eos_s), (pad, _) = tid("bos_token"), tid("eos_token"), tid("pad_token")
        cj = os.path.join(model_dir, "config.json")
        if os.path.exists(cj) and eos is None:
            with open(cj, "r", encoding="utf-8") as fh:
                c = json.load(fh)
            e = c.get("eos_token_id")
            eos = e[0] if isinstance(e, list) else e
            bos = c.get("bos_token_id", bos)
        return cls(tok, bos, eos, pad, eos_s)

    @classmethod
    def from_pretrained(cls, model_id: str) -> "Tokenizer":
        """From a model directory, a ``tokenizer.json`` path, or a hub id that is in the local cache (or can be fetched)."""
        if os.path.isfile(model_id):
            return cls.from_file(model_id)
        if os.path.isdir(model_id):
            return cls.from_model_dir(model_id)
        from ..models.loader import resolve_model_path
        return cls.from_model_dir(resolve_model_path(model_id))

    @property
    def unk_token_id(self) -> Optional[int]:
        if self._tok is None:
            return None
        unk = getattr(getattr(self._tok, "model", None), "unk_token", None)
        return self._tok.token_to_id(unk) if unk else None

    @property
    def vocab_size(self) -> int:
        return self._tok.get_vocab_size(with_added_tokens=True)

    def encode(self, text: str) -> List[int]:
        return self._tok.encode(text, add_special_tokens=False).ids

    def encode_with_special_tokens(self, text: str) -> List[int]:
        return self._tok.encode(text, add_special_tokens=True).ids

    def decode(self, ids: List[int], skip_special_tokens: bool = True) -> str:
        return self._tok.decode(list(ids), skip_special_tokens=skip_special_tokens)

    def token_to_id(self, token: str) -> Optional[int]:
        return self._tok.token_to_id(token)

    def id_to_token(self, i: int) -> Optional[str]:
        return self._tok.id_to_token(i)


class ByteTokenizer(Tokenizer):
    """ids 0..255 are bytes, 256 = <bos>, 257 = <eos>, 258 = <pad>."""

    def __init__(self):
        self.bos_token_id, self.eos_token_id, self.pad_token_id = 256, 257, 258
        self.eos_token = "<eos>"
        self._tok = None

    @property
    def vocab_size(self) -> int:
        return 259

    def encode(self, text: str) -> List[int]:
        return list(text.encode("utf-8"))

    def encode_with_special_tokens(self, text: str) -> List[int]:
        return self.encode(text)

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        return bytes(i for i in ids if i < 256).decode("utf-8", errors="replace")

    def token_to_id(self, token):
        return {"<bos>": 256, "<eos>": 257, "<pad>": 258}.get(token)

    def id_to_token(self, i):
        return chr(i) if i < 256 else {256: "<bos>", 257: "<eos>", 258: "<pad>"}.get(i)


class StreamDecoder:
    """Incremental detokeniser that only emits text at UTF-8-safe boundaries."""

    def __init__(self, tok: Tokenizer):
        self.tok, self.ids, self.emitted = tok, [], 0

    def push(self, token_id: int) -> str:
        self.ids.append(token_id)
        text = self.tok.decode(self.ids)
        if text.endswith("�"):
            return ""
        out, self.emitted = text[self.emitted:], len(text)
        return out
