"""Text generation on the paged KV cache.

``Generator`` runs any number of sequences in lock-step: chunked prefill (2048 tokens per chunk,
crates/pmetal-models/src/generation.rs:316-355), then batched single-token decode steps with
per-row sampling, stop tokens and length limits. It is the engine under ``pmetal infer``, the
batched RL rollouts (the reference decodes the G rollouts of a group one by one,
rl_generation.rs:285-420; here they share the prompt blocks and decode as one batch) and
speculative decoding (``speculative.py``).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Iterator, List, Optional, Sequence

import torch

from .kv_cache import BLOCK, BatchMeta, PagedKVCache
from .sampling import Sampler, SamplingParams

PREFILL_CHUNK = 2048


@dataclass
class GenerationResult:
    tokens: List[List[int]]
    logprobs: Optional[List[List[float]]] = None
    finish_reasons: List[str] = field(default_factory=list)
    prompt_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0

    @property
    def generated_tokens(self) -> int:
        return sum(len(t) for t in self.tokens)

    @property
    def decode_tok_per_s(self) -> float:
        return self.generated_tokens / self.decode_seconds if self.decode_seconds > 0 else 0.0

    @property
    def prefill_tok_per_s(self) -> float:
        return self.prompt_tokens / self.prefill_seconds if self.prefill_seconds > 0 else 0.0


def _bucket(n: int, lo: int = 1) -> int:
    b = lo
    while b < n:
        b *= 2
    return b


class GraphedDecoder:
    """Single-token decode steps replayed from CUDA graphs.

    A decode step is a few hundred small launches (28 layers of norm, projections, rope, cache append, paged attention,
    MLP): eager execution is bound by launch and interpreter overhead, not by the GPU. One graph is captured per
    (batch bucket, block-table width bucket); every step copies the step's slots, positions, lengths and block tables
    into the graph's static buffers from pinned host memory (two async copies) and replays it. Batches are padded to the
    bucket with rows that point at a private scratch block, so a shrinking batch does not trigger new captures.
    The reference compiles its decode layers with ``mx::compile`` for the same reason
    (crates/pmetal-bridge/cpp/bridge_compiled.cpp:213-400; "~7x" in crates/pmetal-bridge/src/compile.rs:3-8)."""

    PAD_SEQ = -(1 << 40)

    def __init__(self, model, cache: PagedKVCache, pad_block: Optional[int] = None):
        self.model, self.cache, self.device = model, cache, cache.device
        self.graphs = {}
        self.channel = getattr(model, "step_channel", None)
        if pad_block is not None:           # a rank that follows another rank's scheduler uses that rank's scratch block
            self.pad_block = pad_block
            return
        if self.PAD_SEQ not in cache.seqs:
            cache.add_sequence(self.PAD_SEQ)
            cache.reserve(self.PAD_SEQ, 1)
        self.pad_block = cache.seqs[self.PAD_SEQ].blocks[0]

    def _state(self, nb: int, mb: int):
        key = (nb, mb)
        st = self.graphs.get(key)
        if st is not None:
            return st
        ch = self.channel
        if ch is not None:
            if ch.leader:           # the other ranks warm up and capture the same graph now: its collectives pair up
                from ..serve.replica import KIND_CAPTURE
                ch.publish(KIND_CAPTURE, [nb, mb, 0, self.pad_block])
            ch.muted += 1
        try:
            return self._capture(key, nb, mb)
        finally:
            if ch is not None:
                ch.muted -= 1

    def _capture(self, key, nb: int, mb: int):
        dev = self.device
        st = {
            "h64": torch.zeros(2 * nb, dtype=torch.int64).pin_memory(),              # slots | tokens
            "h32": torch.zeros(2 * nb + nb * mb, dtype=torch.int32).pin_memory(),    # positions | seq_lens | table
            "d64": torch.zeros(2 * nb, dtype=torch.int64, device=dev),
            "d32": torch.zeros(2 * nb + nb * mb, dtype=torch.int32, device=dev),
        }
        d64, d32 = st["d64"], st["d32"]
        st["meta"] = BatchMeta(list(range(nb)), d32[2 * nb:].view(nb, mb), d32[nb:2 * nb],
                               torch.arange(nb, dtype=torch.int32, device=dev), torch.ones(nb, dtype=torch.int32, device=dev),
                               d64[:nb], d32[:nb], nb, 1, mb * BLOCK)
        st["tokens"] = d64[nb:]
        self._fill(st, nb, mb, [], [], [], [], [])
        self._copy(st)
        # warm-up outside capture (lazy initialisations), then capture
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self.model.forward_paged(st["tokens"], self.cache, st["meta"])
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            st["logits"] = self.model.forward_paged(st["tokens"], self.cache, st["meta"])
        st["graph"] = g
        self.graphs[key] = st
        return st

    def _fill(self, st, nb, mb, slots, pos, lens, tables, tokens):
        """Write one step's metadata into the pinned host buffers (numpy views; no tensor constructions)."""
        if "n64" not in st:
            st["n64"], st["n32"] = st["h64"].numpy(), st["h32"].numpy()
            st["rows"] = [None] * nb               # (first block, block count) last written per row
            st["n32"][2 * nb:] = self.pad_block
        a64, a32 = st["n64"], st["n32"]
        n = len(slots)
        a64[:n] = slots
        a64[n:nb] = self.pad_block * BLOCK
        a64[nb:nb + n] = tokens
        a64[nb + n:] = 0
        a32[:n] = pos
        a32[n:nb] = 0
        a32[nb:nb + n] = lens
        a32[nb + n:2 * nb] = 1
        tab = a32[2 * nb:].reshape(nb, mb)
        rows = st["rows"]
        for i in range(nb):
            bl = tables[i] if i < n else None
            sig = None if bl is None else (bl[0], len(bl), bl[-1], sum(1 for b in bl if b < 0) if self.cache.window > 0 else 0)
            if rows[i] == sig:
                continue
            rows[i] = sig
            if bl is None:
                tab[i, :] = self.pad_block
            else:
                tab[i, :len(bl)] = bl
                tab[i, len(bl):] = self.pad_block
                if self.cache.window > 0:          # blocks given back by the rotating window are never visited
                    row = tab[i, :len(bl)]
                    row[row < 0] = self.pad_block

    def _copy(self, st):
        st["d64"].copy_(st["h64"], non_blocking=True)
        st["d32"].copy_(st["h32"], non_blocking=True)

    @torch.no_grad()
    def step(self, seq_ids: Sequence[int], tokens) -> torch.Tensor:
        n = len(seq_ids)
        cache = self.cache
        slots, pos, lens, tables = [], [], [], []
        for sid in seq_ids:
            start = cache.seqs[sid].length
            slots.extend(cache.reserve(sid, 1))
            if cache.window > 0:
                cache._evict_outside_window(sid, start)
            pos.append(start)
            lens.append(start + 1)
            tables.append(cache.seqs[sid].blocks)
        nb, mb = _bucket(n), _bucket(max(len(t) for t in tables), 8)
        st = self._state(nb, mb)
        toks = tokens.tolist() if isinstance(tokens, torch.Tensor) else list(tokens)
        self._fill(st, nb, mb, slots, pos, lens, tables, toks)
        if self.channel is not None and self.channel.leader:
            self.channel.publish_graph(nb, mb, n, self.pad_block, st["h64"], st["h32"])
        self._copy(st)
        st["graph"].replay()
        return st["logits"][:n].clone()      # the static buffer is overwritten by the next replay


class Generator:
    def __init__(self, model, cache: Optional[PagedKVCache] = None, num_blocks: Optional[int] = None,
                 cuda_graphs: Optional[bool] = None):
        self.model = model
        self.device = model.embed_tokens.device
        if cache is None:
            cache = model.new_cache(num_blocks or 4096)
        self.cache = cache
        self._next_id = 0
        self._graphed: Optional[GraphedDecoder] = None
        if cuda_graphs is None:
            import os
            cuda_graphs = os.environ.get("PMETAL_DECODE_GRAPHS", "1") == "1"
        # experts streamed from disk are chosen on the host every step: nothing to capture
        self.cuda_graphs = (bool(cuda_graphs) and self.device.type == "cuda"
                            and getattr(model, "expert_store", None) is None)

    def new_seq(self) -> int:
        sid = self._next_id
        self._next_id += 1
        self.cache.add_sequence(sid)
        return sid

    # ------------------------------------------------------------------ prefill / decode primitives
    @torch.no_grad()
    def prefill(self, seq_ids: Sequence[int], prompts: Sequence[Sequence[int]], chunk: int = PREFILL_CHUNK):
        """Feed whole prompts (chunked); returns logits of each prompt's last token [n, V]."""
        n = len(seq_ids)
        offs = [0] * n
        last_logits = [None] * n
        while True:
            ids, sids, counts = [], [], []
            budget = chunk
            for i in range(n):
                rem = len(prompts[i]) - offs[i]
                if rem <= 0 or budget <= 0:
                    continue
                take = min(rem, budget)
                ids.extend(prompts[i][offs[i]:offs[i] + take])
                sids.append(i)
                counts.append(take)
                budget -= take
            if not sids:
                break
            meta = self.cache.prepare([seq_ids[i] for i in sids], counts)
            t = torch.tensor(ids, dtype=torch.int64, device=self.device)
            logits = self.model.forward_paged(t, self.cache, meta)
            for j, i in enumerate(sids):
                offs[i] += counts[j]
                if offs[i] == len(prompts[i]):
                    last_logits[i] = logits[j]
        return torch.stack(last_logits)

    @torch.no_grad()
    def decode_step(self, seq_ids: Sequence[int], tokens: torch.Tensor) -> torch.Tensor:
        """One new token per sequence → next-token logits [n, V]."""
        from ..utils import nvtx
        with nvtx.range("decode_step"):
            return self._decode_step(seq_ids, tokens)

    def _decode_step(self, seq_ids: Sequence[int], tokens: torch.Tensor) -> torch.Tensor:
        if self.cuda_graphs:
            from ..ops import functional as ops
            if ops.native_enabled(self.model.embed_tokens) and self.model.cfg.head_dim == 128:
                if self._graphed is None:
                    self._graphed = GraphedDecoder(self.model, self.cache)
                return self._graphed.step(seq_ids, tokens)
        meta = self.cache.prepare(seq_ids, [1] * len(seq_ids))
        return self.model.forward_paged(tokens, self.cache, meta)

    # ------------------------------------------------------------------ full loop
    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], params: Optional[SamplingParams] = None,
                 eos_ids: Sequence[int] = (), num_return_sequences: int = 1, return_logprobs: bool = False,
                 on_token: Optional[Callable[[int, int], None]] = None, keep_sequences: bool = False,
                 track_history: bool = True) -> GenerationResult:
        """Generate for every prompt (``num_return_sequences`` samples each, sharing the prompt's KV blocks)."""
        p = params or SamplingParams()
        sampler = Sampler(p, self.device)
        stop = set(eos_ids) | set(p.stop_token_ids)
        G = num_return_sequences
        t0 = time.perf_counter()
        base_ids = [self.new_seq() for _ in prompts]
        logits = self.prefill(base_ids, prompts)
        seq_ids: List[int] = []
        for b in base_ids:
            seq_ids.append(b)
            for _ in range(G - 1):
                sid = self._next_id
                self._next_id += 1
                self.cache.fork(b, sid)
                seq_ids.append(sid)
        if G > 1:
            logits = logits.repeat_interleave(G, dim=0)
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        t1 = time.perf_counter()
        n = len(seq_ids)
        V = logits.shape[-1]
        counts = None
        if track_history and (p.repetition_penalty != 1.0 or p.frequency_penalty or p.presence_penalty):
            counts = torch.zeros(n, V, dtype=torch.int32, device=self.device)
            for i, pr in enumerate(prompts):
                c = torch.bincount(torch.tensor(pr, device=self.device), minlength=V).to(torch.int32)
                counts[i * G:(i + 1) * G] = c
        out: List[List[int]] = [[] for _ in range(n)]
        lps: List[List[float]] = [[] for _ in range(n)]
        reasons = ["length"] * n
        alive = list(range(n))
        for step in range(p.max_tokens):
            cur_counts = counts[alive] if counts is not None else None
            if return_logprobs:
                ids, lp = sampler.sample(logits, cur_counts, True)
                lp_l = lp.tolist()
            else:
                ids = sampler.sample(logits, cur_counts)
            id_l = ids.tolist()
            keep = []
            for j, i in enumerate(alive):
                tok = id_l[j]
                out[i].append(tok)
                if return_logprobs:
                    lps[i].append(lp_l[j])
                if on_token:
                    on_token(i, tok)
                if tok in stop:
                    reasons[i] = "stop"
                else:
                    keep.append(j)
            if counts is not None:
                counts[alive, ids] += 1
            if not keep or step == p.max_tokens - 1:
                break
            if len(keep) != len(alive):
                sel = torch.tensor(keep, device=self.device)
                ids = ids[sel]
                alive = [alive[j] for j in keep]
            logits = self.decode_step([seq_ids[i] for i in alive], ids)
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        t2 = time.perf_counter()
        if not keep_sequences:
            for sid in seq_ids:
                self.cache.free_sequence(sid)
        res = GenerationResult(out, lps if return_logprobs else None, reasons, sum(len(x) for x in prompts),
                               t1 - t0, t2 - t1)
        res.seq_ids = seq_ids
        return res

    def stream(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
               eos_ids: Sequence[int] = ()) -> Iterator[int]:
        """Yield tokens of a single sequence as they are sampled."""
        p = params or SamplingParams()
        sampler = Sampler(p, self.device)
        stop = set(eos_ids) | set(p.stop_token_ids)
        sid = self.new_seq()
        try:
            logits = self.prefill([sid], [prompt])
            counts = None
            if p.repetition_penalty != 1.0 or p.frequency_penalty or p.presence_penalty:
                counts = torch.bincount(torch.tensor(list(prompt), device=self.device),
                                        minlength=logits.shape[-1]).to(torch.int32)[None]
            for _ in range(p.max_tokens):
                ids = sampler.sample(logits, counts)
                tok = int(ids[0])
                yield tok
                if tok in stop:
                    break
                if counts is not None:
                    counts[0, tok] += 1
                logits = self.decode_step([sid], ids)
        finally:
            self.cache.free_sequence(sid)
