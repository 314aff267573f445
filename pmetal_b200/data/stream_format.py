"""Streaming output formatter for chat models with a reasoning channel.

Reasoning models wrap their chain of thought in marker tokens (``<think>…</think>`` for Qwen 3 / DeepSeek-R1 distills,
``<|channel>…<channel|>`` for Gemma 4). Printed raw, the reasoning is indistinguishable from the answer. The formatter
resolves the marker ids once, tracks whether the stream is inside the channel, and either hides the reasoning body or
labels it (``[thinking]`` / ``[answer]``). Marker tokens and hidden tokens never enter the incremental detokeniser, so no
marker text leaks and multi-byte characters are only emitted when complete
(crates/pmetal-data/src/stream_format.rs:30-151)."""
from __future__ import annotations

from typing import List

OPEN_MARKERS = ("<|channel>", "<think>")
CLOSE_MARKERS = ("<channel|>", "</think>")


class StreamFormatter:
    def __init__(self, tokenizer, show_thinking: bool = True):
        self.tok = tokenizer
        self.open_ids = [i for i in (tokenizer.token_to_id(m) for m in OPEN_MARKERS) if i is not None]
        self.close_ids = [i for i in (tokenizer.token_to_id(m) for m in CLOSE_MARKERS) if i is not None]
        self.show_thinking = show_thinking
        self.ids: List[int] = []
        self.emitted = 0
        self.in_thinking = False
        self._label_thinking = self._label_answer = False

    def push(self, token_id: int) -> str:
        """Text to print for this token (may be empty, may carry a label)."""
        if token_id in self.open_ids and not self.in_thinking:
            self.in_thinking = True
            if self.show_thinking and not self._label_thinking:
                self._label_thinking = True
                return ("\n" if self.emitted else "") + "[thinking]\n"
            return ""
        if token_id in self.close_ids and self.in_thinking:
            self.in_thinking = False
            if self.show_thinking and not self._label_answer:
                self._label_answer = True
                return "\n\n[answer]\n"
            if not self._label_answer and self.emitted:
                self._label_answer = True
                return "\n"
            return ""
        if self.in_thinking and not self.show_thinking:
            return ""
        self.ids.append(token_id)
        text = self.tok.decode(self.ids)
        if text.endswith("�"):                 # an incomplete multi-byte character: wait for the next token
            return ""
        out, self.emitted = text[self.emitted:], len(text)
        return out
