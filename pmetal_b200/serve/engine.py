"""Continuous-batching inference engine.

Scheduling follows the reference pump (crates/pmetal-serve/src/continuous_pump.rs:289-406, continuous_batch.rs:87-549):
a fixed pool of slots, a FIFO queue with block-budget admission, serial chunked prefill of one request per tick (first
token sampled right after its last chunk, prompt parked in the prefix cache), and one batched decode step per tick for
all active slots with per-slot sampling parameters, stop sequences, log-probabilities and retirement. Where the
reference keeps a dense [slots, heads, max_seq, D] cache and slices it, this engine decodes straight from the paged
cache with the block-table attention kernel, and samples every slot in one fused kernel launch.

Sampling state per slot: repetition / frequency / presence penalties see the tokens generated so far (a device table
of per-token counts, one row per slot, updated by a kernel after every step; crates/pmetal-models/src/generation.rs:
813-838). Stop strings are matched on the decoded text after every token and the tokens that spell the match are cut
from the output (crates/pmetal-serve/src/engine.rs:225-250)."""
from __future__ import annotations

import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional, Sequence

import torch

from ..models.generation import PREFILL_CHUNK, Generator
from ..models.kv_cache import BLOCK
from ..models.sampling import Sampler, SamplingParams
from .prefix_cache import PrefixCache


def detect_stop_suffix(decode: Callable[[List[int]], str], generated: Sequence[int], stops: Sequence[str]) -> int:
    """Number of trailing tokens of ``generated`` whose decoding is exactly the longest stop string that the decoded
    output ends with; 0 when no stop string ends the text or the match does not start on a token boundary."""
    stops = [s for s in stops if s]
    if not generated or not stops:
        return 0
    longest = max(len(s) for s in stops)
    # a token decodes to at least one character in practice; a generous window keeps the check O(stop length)
    window = list(generated[-(2 * longest + 8):])
    text = decode(window)
    hit = [s for s in stops if text.endswith(s)]
    if not hit:
        return 0
    match = max(hit, key=len)
    for n in range(1, len(window) + 1):
        if decode(window[-n:]) == match:
            return n
    return 0


@dataclass
class Request:
    prompt: List[int]
    params: SamplingParams = field(default_factory=SamplingParams)
    stop_sequences: List[List[int]] = field(default_factory=list)
    want_logprobs: bool = False
    stop_strings: List[str] = field(default_factory=list)                   # matched on decoded text (needs ``decode``)
    decode: Optional[Callable[[List[int]], str]] = None
    top_logprobs: int = 0                                                   # alternatives recorded per generated token
    top_entries: List[List[tuple]] = field(default_factory=list)            # per token: [(token id, logprob), ...]
    adapter: Optional[str] = None                                           # LoRA adapter of this request (multi-adapter serving)
    on_token: Optional[Callable[[int, Optional[float]], None]] = None       # called from the engine thread
    on_done: Optional[Callable[["Request"], None]] = None
    # filled by the engine
    id: int = -1
    output: List[int] = field(default_factory=list)
    logprobs: List[float] = field(default_factory=list)
    finish_reason: Optional[str] = None
    t_submit: float = 0.0
    t_first: float = 0.0
    t_done: float = 0.0
    cached_tokens: int = 0
    done: threading.Event = field(default_factory=threading.Event)


@dataclass
class _Slot:
    req: Request
    seq: int
    prefill_pos: int = 0
    last_token: int = -1
    state: str = "prefill"       # prefill | decode
    row: int = -1                # row of the penalty count table (-1: the request uses no penalty)


@dataclass
class EngineStats:
    requests_total: int = 0
    requests_done: int = 0
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefix_hits: int = 0
    decode_steps: int = 0
    decode_seconds: float = 0.0
    prefill_seconds: float = 0.0

    def as_dict(self) -> dict:
        d = dict(self.__dict__)
        d["decode_tok_per_s"] = self.generated_tokens / self.decode_seconds if self.decode_seconds > 0 else 0.0
        return d


class ContinuousBatchEngine:
    def __init__(self, model, eos_ids: Sequence[int] = (), max_slots: int = 64, num_blocks: int = 8192,
                 prefill_chunk: int = PREFILL_CHUNK, prefix_cache: bool = True, max_queue: int = 1024,
                 cache_options: Optional[dict] = None, adapters=None):
        self.model = model
        self.adapters = adapters        # lora.batched.AdapterSet: every request picks an adapter (or none) by name
        opts = dict(cache_options or {})
        self.gen = Generator(model, cache=model.new_cache(num_blocks, **opts)) if opts else Generator(model, num_blocks=num_blocks)
        if opts.get("window"):
            prefix_cache = False      # a rotating cache recycles prompt blocks: there is no stable prefix to share
        if adapters is not None:
            self.gen.cuda_graphs = False      # the adapter of every row changes from step to step
            prefix_cache = False              # cached keys/values depend on the adapter that produced them
        self.cache = self.gen.cache
        self.device = self.gen.device
        self.eos = set(eos_ids)
        self.max_slots, self.prefill_chunk, self.max_queue = max_slots, prefill_chunk, max_queue
        self.queue: Deque[Request] = deque()
        self.slots: List[_Slot] = []
        self.prefix = PrefixCache(self.cache) if prefix_cache else None
        self.stats = EngineStats()
        self._lock = threading.Lock()
        self._wake = threading.Event()
        self._stop = False
        self._thread: Optional[threading.Thread] = None
        self._next_req = 0
        self._step = 0
        self._counts: Optional[torch.Tensor] = None      # [max_slots, vocab] int32, allocated on first use
        self._free_rows = list(range(max_slots))

    # ------------------------------------------------------------------ submission
    def submit(self, req: Request) -> Request:
        if req.adapter:
            if self.adapters is None:
                raise KeyError(f"no adapters are loaded (request asked for {req.adapter!r})")
            self.adapters.index(req.adapter)         # raises KeyError for an unknown name
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
        """Blocking helper: submit one request and pump (or wait for the background thread) until it is done."""
        req = self.submit(Request(list(prompt), params or SamplingParams(), **kw))
        if self._thread is None:
            while not req.done.is_set():
                self.tick()
        else:
            req.done.wait()
        return req

    # ------------------------------------------------------------------ scheduling
    def _blocks_needed(self, req: Request) -> int:
        return (len(req.prompt) + req.params.max_tokens + BLOCK - 1) // BLOCK + 1

    def _admit(self) -> None:
        while self.queue and len(self.slots) < self.max_slots:
            req = self.queue[0]
            need = self._blocks_needed(req)
            reserved = sum(self._blocks_needed(s.req) - (self.cache.length(s.seq) // BLOCK) for s in self.slots)
            if self.cache.num_free() - reserved < need:
                if self.prefix is not None and self.prefix.entries:
                    self.prefix.evict_for_blocks(need + reserved)
                    if self.cache.num_free() - reserved >= need:
                        continue
                if not self.slots:      # nothing running and still no room: the request can never fit
                    self.queue.popleft()
                    self._finish(req, "error:too_long")
                break
            self.queue.popleft()
            seq = self.gen.new_seq()
            slot = _Slot(req, seq)
            if self.prefix is not None:
                entry, n = self.prefix.lookup(req.prompt)
                if entry is not None:
                    self.cache.free_sequence(seq)
                    self.prefix.attach(entry, n, seq)
                    slot.prefill_pos = n
                    req.cached_tokens = n
                    self.stats.prefix_hits += 1
            self.stats.prompt_tokens += len(req.prompt)
            p = req.params
            if p.repetition_penalty != 1.0 or p.frequency_penalty != 0.0 or p.presence_penalty != 0.0:
                slot.row = self._free_rows.pop()
                if self._counts is None:
                    self._counts = torch.zeros(self.max_slots, self.model.cfg.vocab_size, dtype=torch.int32,
                                               device=self.device)
                else:
                    self._counts[slot.row].zero_()
            self.slots.append(slot)

    def _finish(self, req: Request, reason: str) -> None:
        req.finish_reason = reason
        req.t_done = time.perf_counter()
        self.stats.requests_done += 1
        req.done.set()
        if req.on_done:
            req.on_done(req)

    def _emit(self, slot: _Slot, tok: int, lp: Optional[float]) -> bool:
        """Record a sampled token; returns True when the request is finished."""
        req = slot.req
        req.output.append(tok)
        if lp is not None:
            req.logprobs.append(lp)
        if not req.t_first:
            req.t_first = time.perf_counter()
        self.stats.generated_tokens += 1
        if req.on_token:
            req.on_token(tok, lp)
        if tok in self.eos or tok in req.params.stop_token_ids:
            return self._retire(slot, "stop")
        for ss in req.stop_sequences:
            if ss and len(req.output) >= len(ss) and req.output[-len(ss):] == ss:
                return self._retire(slot, "stop")
        if req.stop_strings and req.decode is not None:
            cut = detect_stop_suffix(req.decode, req.output, req.stop_strings)
            if cut:                                  # the tokens that spell the stop string are not part of the answer
                del req.output[-cut:]
                del req.logprobs[len(req.output):]
                del req.top_entries[len(req.output):]
                return self._retire(slot, "stop")
        if len(req.output) >= req.params.max_tokens:
            return self._retire(slot, "length")
        slot.last_token = tok
        return False

    def _retire(self, slot: _Slot, reason: str) -> bool:
        if slot.row >= 0:
            self._free_rows.append(slot.row)
            slot.row = -1
        self.cache.free_sequence(slot.seq)
        self.slots.remove(slot)
        self._finish(slot.req, reason)
        return True

    def _sample(self, logits: torch.Tensor, slots: List[_Slot]):
        """One fused launch for all rows on the GPU; per-request Sampler objects otherwise. Returns (token ids,
        log-probabilities or None); alternatives for requests that asked for ``top_logprobs`` are stored on the request."""
        from ..ops import functional as ops
        want_lp = any(s.req.want_logprobs for s in slots)
        pen = any(s.row >= 0 for s in slots)
        top_n = max((s.req.top_logprobs for s in slots), default=0)
        if top_n > 0:
            # alternatives come from the unfiltered distribution, as the chosen token's reported log-probability does
            lsm = torch.log_softmax(logits.float(), -1)
            tv, ti = lsm.topk(min(top_n, lsm.shape[-1]), -1)
            tv, ti = tv.tolist(), ti.tolist()
            for j, s in enumerate(slots):
                n = s.req.top_logprobs
                if n > 0:
                    s.req.top_entries.append(list(zip(ti[j][:n], tv[j][:n])))
        if ops.native_enabled(logits):
            from ..ops import native
            dev = logits.device
            ps = [s.req.params for s in slots]
            f = lambda xs: torch.tensor(xs, dtype=torch.float32, device=dev)      # noqa: E731
            temp = f([0.0 if p.is_greedy else p.temperature for p in ps])
            seeds = torch.tensor([(p.seed if p.seed is not None else 0x5DEECE66D) + 7919 * s.req.id
                                  for p, s in zip(ps, slots)], dtype=torch.int64, device=dev)
            self._step += 1
            lg = logits if logits.stride(-1) == 1 else logits.contiguous()
            if lg.dtype not in (torch.float32, torch.bfloat16):
                lg = lg.float()
            counts = rows = rep_t = freq_t = pres_t = None
            if pen:
                # rows without a penalty point at row 0 with neutral factors, which leaves their logits untouched
                counts = self._counts
                rows = torch.tensor([max(s.row, 0) for s in slots], dtype=torch.int32, device=dev)
                on = [s.row >= 0 for s in slots]
                rep_t = f([p.repetition_penalty if o else 1.0 for p, o in zip(ps, on)])
                freq_t = f([p.frequency_penalty if o else 0.0 for p, o in zip(ps, on)])
                pres_t = f([p.presence_penalty if o else 0.0 for p, o in zip(ps, on)])
            ids, lp = native.sample(lg, temp, torch.tensor([p.top_k for p in ps], dtype=torch.int32, device=dev),
                                    f([p.top_p for p in ps]), f([p.min_p for p in ps]), counts, rep_t, freq_t, pres_t,
                                    seeds, self._step, want_lp, count_rows=rows)
            if pen:
                sel = [j for j, s in enumerate(slots) if s.row >= 0]
                if len(sel) == len(slots):
                    native.count_tokens(counts, ids, rows)
                else:
                    ix = torch.tensor(sel, dtype=torch.int64, device=dev)
                    native.count_tokens(counts, ids[ix].contiguous(), rows[ix].contiguous())
            return ids.tolist(), (lp.tolist() if want_lp else None)
        ids, lps = [], []
        for j, s in enumerate(slots):
            smp = getattr(s, "_sampler", None)
            if smp is None:
                smp = s._sampler = Sampler(s.req.params, logits.device)
            cnt = self._counts[s.row:s.row + 1] if s.row >= 0 else None
            if want_lp:
                i, l = smp.sample(logits[j:j + 1], cnt, True)
                lps.append(float(l[0]))
            else:
                i = smp.sample(logits[j:j + 1], cnt)
            if s.row >= 0:
                self._counts[s.row, int(i[0])] += 1
            ids.append(int(i[0]))
        return ids, (lps if want_lp else None)

    # ------------------------------------------------------------------ one scheduler tick
    @torch.no_grad()
    def tick(self) -> bool:
        """Admit, prefill one chunk of one request, decode one token for every active slot. False when idle."""
        with self._lock:
            self._admit()
        if not self.slots:
            return False
        pre = next((s for s in self.slots if s.state == "prefill"), None)
        if pre is not None:
            t0 = time.perf_counter()
            req = pre.req
            take = min(self.prefill_chunk, len(req.prompt) - pre.prefill_pos)
            meta = self.cache.prepare([pre.seq], [take])
            ids = torch.tensor(req.prompt[pre.prefill_pos:pre.prefill_pos + take], dtype=torch.int64, device=self.device)
            if self.adapters is not None:
                self.adapters.set_rows([self.adapters.index(req.adapter)] * take)
            logits = self.model.forward_paged(ids, self.cache, meta)
            pre.prefill_pos += take
            if pre.prefill_pos == len(req.prompt):
                if self.prefix is not None:
                    self.prefix.insert(pre.seq, req.prompt)
                pre.state = "decode"
                toks, lps = self._sample(logits[-1:], [pre])
                self._emit(pre, toks[0], lps[0] if lps else None)
            self.stats.prefill_seconds += time.perf_counter() - t0
        dec = [s for s in self.slots if s.state == "decode" and s.last_token >= 0 and s is not pre]
        if dec:
            t0 = time.perf_counter()
            toks = torch.tensor([s.last_token for s in dec], dtype=torch.int64, device=self.device)
            if self.adapters is not None:
                self.adapters.set_rows([self.adapters.index(s.req.adapter) for s in dec])
            logits = self.gen.decode_step([s.seq for s in dec], toks)
            ids, lps = self._sample(logits, dec)
            for j, s in enumerate(list(dec)):
                self._emit(s, ids[j], lps[j] if lps else None)
            self.stats.decode_steps += 1
            self.stats.decode_seconds += time.perf_counter() - t0
        return True

    # ------------------------------------------------------------------ background pump
    def start(self) -> None:
        if self._thread is not None:
            return
        self._stop = False

        def loop():
            while not self._stop:
                if not self.tick():
                    self._wake.wait(0.05)
                    self._wake.clear()
        self._thread = threading.Thread(target=loop, name="pmetal-engine", daemon=True)
        self._thread.start()

    def shutdown(self) -> None:
        self._stop = True
        self._wake.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
            self._thread = None
        for s in list(self.slots):
            self._retire(s, "cancelled")
        if self.prefix is not None:
            self.prefix.clear()
