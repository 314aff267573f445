"""Serving engine for the config-driven architectures (Gemma, Phi, Cohere, Granite, DeepSeek, GPT-OSS, Llama 4, ...).

These models keep a contiguous per-sequence key/value cache and take a ``[1, T]`` batch, so they cannot share the paged,
ragged-batch engine of the fast decoder. This engine gives them the same front: the ``Request`` objects, stop handling,
log-probabilities, penalties, statistics and the background thread of ``ContinuousBatchEngine``, with requests
interleaved token by token (every active request advances by one token per round, prompts are prefilled in chunks
between decode rounds), so that streams stay responsive under concurrency. Counterpart of the reference's engine for
models without the fused batch path (crates/pmetal-serve/src/engine.rs: one session per request, serial decode)."""
from __future__ import annotations

import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional, Sequence

import torch

from ..models.sampling import Sampler, SamplingParams
from .engine import EngineStats, Request, detect_stop_suffix

PREFILL_CHUNK = 2048


@dataclass
class _Session:
    req: Request
    cache: object
    sampler: Sampler
    pos: int = 0                         # prompt tokens already in the cache
    last_token: int = -1
    state: str = "prefill"
    counts: Optional[torch.Tensor] = None            # [1, vocab] int32 occurrences (penalties)
    tokens: int = 0


class _CacheView:
    """What the metrics route asks of a cache: free capacity, here in sessions."""

    def __init__(self, engine: "PortableEngine"):
        self.engine = engine

    def num_free(self) -> int:
        return max(self.engine.max_slots - len(self.engine.slots), 0)


class PortableEngine:
    def __init__(self, model, eos_ids: Sequence[int] = (), max_slots: int = 8, max_queue: int = 1024,
                 prefill_chunk: int = PREFILL_CHUNK, cache_options: Optional[dict] = None):
        if not hasattr(model, "new_cache"):
            raise ValueError("this architecture has no text-generation cache")
        self.model = model
        self.adapters = None
        self.eos = set(eos_ids)
        self.max_slots, self.max_queue, self.prefill_chunk = max_slots, max_queue, prefill_chunk
        self.cache_options = dict(cache_options or {})
        self.device = next(model.parameters()).device
        self.queue: Deque[Request] = deque()
        self.slots: List[_Session] = []
        self.cache = _CacheView(self)
        self.stats = EngineStats()
        self._lock = threading.Lock()
        self._wake = threading.Event()
        self._stop = False
        self._thread: Optional[threading.Thread] = None
        self._next_req = 0

    # ------------------------------------------------------------------ submission (same contract as the paged engine)
    def submit(self, req: Request) -> Request:
        if req.adapter:
            raise KeyError(f"no adapters are loaded (request asked for {req.adapter!r})")
        with self._lock:
            if len(self.queue) >= self.max_queue:
                raise RuntimeError("queue full")
            req.id = self._next_req
            self._next_req += 1
            req.t_submit = time.perf_counter()
            self.queue.append(req)
            self.stats.requests_total += 1
        self._wake.set()
        return req

    def generate(self, prompt: Sequence[int], params: Optional[SamplingParams] = None, **kw) -> Request:
        req = self.submit(Request(list(prompt), params or SamplingParams(), **kw))
        if self._thread is None:
            while not req.done.is_set():
                self.tick()
        else:
            req.done.wait()
        return req

    # ------------------------------------------------------------------ one round
    def _admit(self) -> None:
        with self._lock:
            while self.queue and len(self.slots) < self.max_slots:
                req = self.queue.popleft()
                if not req.prompt:
                    req.prompt = [0]
                s = _Session(req, self.model.new_cache(**self.cache_options), Sampler(req.params, self.device))
                p = req.params
                if p.repetition_penalty != 1.0 or getattr(p, "frequency_penalty", 0.0) or getattr(p, "presence_penalty", 0.0):
                    vocab = self._vocab()
                    s.counts = torch.zeros(1, vocab, dtype=torch.int32, device=self.device)
                    idx = torch.tensor(req.prompt, device=self.device, dtype=torch.int64).clamp(0, vocab - 1)
                    s.counts[0].index_add_(0, idx, torch.ones_like(idx, dtype=torch.int32))
                self.stats.prompt_tokens += len(req.prompt)
                self.slots.append(s)

    def _vocab(self) -> int:
        c = getattr(self.model, "c", None)
        v = int(getattr(c, "vocab_size", 0) or 0)
        if v:
            return v
        with torch.no_grad():                      # no configuration to ask: one token through the model tells
            return int(self.model(torch.zeros(1, 1, dtype=torch.int64, device=self.device)).shape[-1])

    def _finish(self, s: _Session, reason: str) -> None:
        req = s.req
        self.slots.remove(s)
        s.cache = None
        req.finish_reason = reason
        req.t_done = time.perf_counter()
        self.stats.requests_done += 1
        req.done.set()
        if req.on_done:
            req.on_done(req)

    def _emit(self, s: _Session, tok: int, lp: Optional[float]) -> bool:
        req = s.req
        req.output.append(tok)
        if lp is not None:
            req.logprobs.append(lp)
        if not req.t_first:
            req.t_first = time.perf_counter()
        self.stats.generated_tokens += 1
        if s.counts is not None and 0 <= tok < s.counts.shape[1]:
            s.counts[0, tok] += 1
        if req.on_token:
            req.on_token(tok, lp)
        if tok in self.eos or tok in req.params.stop_token_ids:
            self._finish(s, "stop")
            return True
        for ss in req.stop_sequences:
            if ss and len(req.output) >= len(ss) and req.output[-len(ss):] == ss:
                self._finish(s, "stop")
                return True
        if req.stop_strings and req.decode is not None:
            cut = detect_stop_suffix(req.decode, req.output, req.stop_strings)
            if cut:
                del req.output[-cut:]
                del req.logprobs[len(req.output):]
                del req.top_entries[len(req.output):]
                self._finish(s, "stop")
                return True
        if len(req.output) >= req.params.max_tokens:
            self._finish(s, "length")
            return True
        s.last_token = tok
        return False

    def _pick(self, s: _Session, logits: torch.Tensor) -> None:
        """Sample from ``logits`` [1, V], record alternatives if asked for, and emit."""
        req = s.req
        lg = logits.float()
        want_lp = req.want_logprobs or req.top_logprobs > 0
        if want_lp:
            ids, lps = s.sampler.sample(lg, s.counts, return_logprobs=True)
            lp = float(lps[0])
        else:
            ids, lp = s.sampler.sample(lg, s.counts), None
        if req.top_logprobs > 0:
            full = torch.log_softmax(lg[0], -1)
            top = torch.topk(full, min(req.top_logprobs, full.numel()))
            req.top_entries.append([(int(i), float(v)) for v, i in zip(top.values, top.indices)])
        self._emit(s, int(ids[0]), lp)

    @torch.no_grad()
    def tick(self) -> bool:
        """Admit, give the oldest unfinished prompt one prefill chunk, then advance every decoding request by one token.
        Returns False when there was nothing to do."""
        self._admit()
        if not self.slots:
            return False
        pre = next((s for s in self.slots if s.state == "prefill"), None)
        if pre is not None:
            t0 = time.perf_counter()
            ids = pre.req.prompt[pre.pos:pre.pos + self.prefill_chunk]
            logits = self.model(torch.tensor([ids], device=self.device), pre.cache)[:, -1]
            pre.pos += len(ids)
            self.stats.prefill_seconds += time.perf_counter() - t0
            if pre.pos >= len(pre.req.prompt):
                pre.state = "decode"
                self._pick(pre, logits)
        dec = [s for s in self.slots if s.state == "decode" and s is not pre]
        if dec:
            t0 = time.perf_counter()
            for s in dec:
                logits = self.model(torch.tensor([[s.last_token]], device=self.device), s.cache)[:, -1]
                self._pick(s, logits)
            self.stats.decode_steps += 1
            self.stats.decode_seconds += time.perf_counter() - t0
        return True

    # ------------------------------------------------------------------ background thread
    def _run(self) -> None:
        while not self._stop:
            if not self.tick():
                self._wake.wait(0.05)
                self._wake.clear()

    def start(self) -> None:
        if self._thread is None:
            self._stop = False
            self._thread = threading.Thread(target=self._run, name="pmetal-portable-engine", daemon=True)
            self._thread.start()

    def shutdown(self) -> None:
        self._stop = True
        self._wake.set()
        if self._thread is not None:
            self._thread.join(timeout=10)
            self._thread = None
        for s in list(self.slots):
            self._finish(s, "cancelled")
        with self._lock:
            while self.queue:
                req = self.queue.popleft()
                req.finish_reason = "cancelled"
                req.done.set()
