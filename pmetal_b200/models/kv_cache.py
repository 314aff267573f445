"""Block-paged KV cache with reference-counted blocks.

The reference's ``PagedKVCache`` (crates/pmetal-mlx/src/kv_cache/paged.rs:10-720) is a block
allocator plus per-sequence block table, but attention still runs on a gathered dense tensor; here
the block table is consumed directly by the decode/verify attention kernel. Blocks hold 64 tokens
(one key tile of the kernel). ``fork`` shares full blocks between sequences (prompt prefix reuse
for group rollouts and the serving prefix cache) and copies the partially filled tail block.

Variants on the same block table (the reference keeps separate cache classes, crates/pmetal-mlx/src/kv_cache/
quantized.rs and rotating.rs; ``select_cache_mode`` restates its choice rule,
crates/pmetal/src/inference_runner.rs:1187-1258,1335-1405):

* ``quant="tq4"``: keys and values are rotated by a random signed Hadamard transform, normalised and stored as 4-bit
  Lloyd-Max codes plus one scale per vector (the TurboQuant scheme, 3.6x smaller than bf16); queries are rotated once,
  attention runs in the rotated basis on the same kernel with a code-book lookup, and the output is rotated back.
* ``quant="int8"``: keys and values are stored as int8 with one fp32 scale per (token, kv head, 64 channels); the
  append kernel quantises, the attention kernel expands a block to bf16 in shared memory while it loads it.
* ``window > 0`` (with ``sink`` leading tokens kept): a rotating cache. Blocks that lie wholly before the window of
  the oldest query of a step, and after the sink, are returned to the pool; the attention kernel never visits them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

BLOCK = 64


@dataclass
class SeqState:
    blocks: List[int] = field(default_factory=list)
    length: int = 0


@dataclass
class BatchMeta:
    """Device tensors describing one forward over new tokens of several sequences."""
    seq_ids: List[int]
    block_table: torch.Tensor   # [n_seq, max_blocks] int32
    seq_lens: torch.Tensor      # [n_seq] int32, keys available after this step's append
    q_start: torch.Tensor       # [n_seq] int32
    q_lens: torch.Tensor        # [n_seq] int32
    slots: torch.Tensor         # [total_q] int64: cache slot (block*64+offset) of each new token
    positions: torch.Tensor     # [total_q] int32
    total_q: int = 0
    max_q: int = 1
    max_kv: int = 0
    host: Optional[tuple] = None    # host copies (slots, positions, seq_lens, q_start, q_lens, block table) when known


GROUP = 64      # channels per quantisation scale of the int8 cache


@dataclass
class CacheMode:
    """Outcome of ``select_cache_mode``: ``kind`` is "standard", "quantized" (``bits``) or "turboquant"; ``source`` says
    whether flags forced it or the memory estimate chose it."""
    kind: str = "standard"
    bits: int = 16
    group_size: int = GROUP
    source: str = "auto_fp16"
    k_bits: Optional[int] = None
    v_bits: Optional[int] = None


def select_cache_mode(weight_bytes: int, fp16_kv_bytes: int, device_bytes: Optional[int], kv_quant: Optional[int] = None,
                      no_kv_quant: bool = False, k_bits: Optional[int] = None, v_bits: Optional[int] = None,
                      turboquant: bool = False, group_size: int = GROUP) -> CacheMode:
    """Which KV cache to build. Flags win: ``no_kv_quant`` / ``kv_quant == 0`` force 16-bit; any of ``kv_quant``,
    ``k_bits``, ``v_bits``, ``turboquant`` selects the named quantised cache (missing sides default to ``kv_quant`` or
    8 bits). Without flags an 8-bit cache is chosen when weights plus a 16-bit cache would take more than 70 % of the
    device's memory, else the 16-bit cache."""
    if no_kv_quant or kv_quant == 0:
        return CacheMode("standard", 16, group_size, "forced_fp16")
    if kv_quant is not None or k_bits is not None or v_bits is not None or turboquant:
        base = kv_quant if kv_quant is not None else 8
        kb, vb = (k_bits if k_bits is not None else base), (v_bits if v_bits is not None else base)
        if turboquant:
            return CacheMode("turboquant", max(kb, vb), group_size, "explicit", kb, vb)
        if kb == vb:
            return CacheMode("quantized", kb, group_size, "explicit", kb, vb)
        return CacheMode("asymmetric", max(kb, vb), group_size, "explicit", kb, vb)
    if device_bytes and weight_bytes + fp16_kv_bytes > int(device_bytes * 0.70):
        return CacheMode("quantized", 8, group_size, "auto_q8", 8, 8)
    return CacheMode("standard", 16, group_size, "auto_fp16")


class PagedKVCache:
    def __init__(self, num_layers: int, num_kv_heads: int, head_dim: int, num_blocks: int, dtype=torch.bfloat16,
                 device="cuda", quant: Optional[str] = None, window: int = 0, sink: int = 0):
        self.num_layers, self.hkv, self.d, self.num_blocks = num_layers, num_kv_heads, head_dim, num_blocks
        self.device = torch.device(device)
        if quant not in (None, "int8", "tq4"):
            raise ValueError("the paged cache stores bf16, int8 or rotated 4-bit codes; other widths use the portable "
                             "QuantKVCache")
        if quant == "int8" and head_dim % GROUP:
            raise ValueError(f"int8 cache needs head_dim to be a multiple of {GROUP}")
        if quant == "tq4" and head_dim != 128:
            raise ValueError("the rotated 4-bit cache is built for head_dim 128")
        self.quant, self.window, self.sink = quant, int(window), int(sink)
        shape = (num_blocks, BLOCK, num_kv_heads, head_dim // 2 if quant == "tq4" else head_dim)
        store = torch.int8 if quant == "int8" else (torch.uint8 if quant == "tq4" else dtype)
        self.tq = None
        if quant == "tq4":
            # random signed Hadamard rotation + 16-level Lloyd-Max code book of the unit normal (models/turboquant.py)
            from .turboquant import TurboQuant
            self.tq = TurboQuant(head_dim, 4, qjl=False, seed=0, device=device)
            self.tq_lut = [float(x) for x in self.tq.centroids.tolist()]
        self.compute_dtype = dtype
        self.k = [torch.zeros(shape, dtype=store, device=device) for _ in range(num_layers)]
        self.v = [torch.zeros(shape, dtype=store, device=device) for _ in range(num_layers)]
        self.k_scale = self.v_scale = None
        if quant in ("int8", "tq4"):
            sshape = (num_blocks, BLOCK, num_kv_heads, head_dim // GROUP)
            self.k_scale = [torch.ones(sshape, dtype=torch.float32, device=device) for _ in range(num_layers)]
            self.v_scale = [torch.ones(sshape, dtype=torch.float32, device=device) for _ in range(num_layers)]
        self.free: List[int] = list(range(num_blocks - 1, -1, -1))
        self.ref = [0] * num_blocks
        self.seqs: Dict[int, SeqState] = {}

    # ------------------------------------------------------------------ allocation
    @classmethod
    def blocks_for_budget(cls, bytes_budget: int, num_layers: int, num_kv_heads: int, head_dim: int,
                          elem_size: int = 2) -> int:
        per_block = 2 * num_layers * BLOCK * num_kv_heads * head_dim * elem_size
        return max(int(bytes_budget // per_block), 1)

    def num_free(self) -> int:
        return len(self.free)

    def _take(self) -> int:
        if not self.free:
            raise MemoryError("paged KV cache is out of blocks")
        b = self.free.pop()
        self.ref[b] = 1
        return b

    def _release(self, b: int) -> None:
        if b < 0:                 # a block that the rotating window already gave back
            return
        self.ref[b] -= 1
        if self.ref[b] == 0:
            self.free.append(b)

    def add_sequence(self, seq_id: int) -> None:
        if seq_id in self.seqs:
            raise KeyError(f"sequence {seq_id} exists")
        self.seqs[seq_id] = SeqState()

    def free_sequence(self, seq_id: int) -> None:
        st = self.seqs.pop(seq_id)
        for b in st.blocks:
            self._release(b)

    def length(self, seq_id: int) -> int:
        return self.seqs[seq_id].length

    def can_append(self, seq_id: int, n: int) -> bool:
        st = self.seqs[seq_id]
        need = -(-(st.length + n) // BLOCK) - len(st.blocks)
        return need <= len(self.free)

    def reserve(self, seq_id: int, n: int) -> List[int]:
        """Make room for ``n`` more tokens; returns their slots (block*64+offset) and advances the length. Work is per
        block, not per token: only the block that holds the current tail can be shared (copy-on-write), every later
        block is new."""
        st = self.seqs[seq_id]
        slots: List[int] = []
        pos, end = st.length, st.length + n
        while pos < end:
            bi = pos // BLOCK
            if bi == len(st.blocks):
                st.blocks.append(self._take())
            b = st.blocks[bi]
            if self.ref[b] > 1:          # copy-on-write of a shared, partially filled block
                nb = self._take()
                for l in range(self.num_layers):
                    self.k[l][nb].copy_(self.k[l][b])
                    self.v[l][nb].copy_(self.v[l][b])
                    if self.k_scale is not None:
                        self.k_scale[l][nb].copy_(self.k_scale[l][b])
                        self.v_scale[l][nb].copy_(self.v_scale[l][b])
                self._release(b)
                st.blocks[bi] = b = nb
            stop = min(end, (bi + 1) * BLOCK)
            base = b * BLOCK - bi * BLOCK
            slots.extend(range(base + pos, base + stop))
            pos = stop
        st.length = end
        return slots

    def truncate(self, seq_id: int, new_len: int) -> None:
        """Drop tokens beyond ``new_len`` (rejected speculative tokens)."""
        st = self.seqs[seq_id]
        keep = -(-new_len // BLOCK) if new_len > 0 else 0
        for b in st.blocks[keep:]:
            self._release(b)
        st.blocks = st.blocks[:keep]
        st.length = new_len

    def fork(self, src_id: int, dst_id: int) -> None:
        """``dst`` starts as a copy of ``src`` sharing its blocks (the tail block is copied on first write)."""
        src = self.seqs[src_id]
        self.seqs[dst_id] = SeqState(list(src.blocks), src.length)
        for b in src.blocks:
            if b >= 0:
                self.ref[b] += 1

    # ------------------------------------------------------------------ batch metadata
    def prepare(self, seq_ids: Sequence[int], new_tokens: Sequence[int]) -> BatchMeta:
        """Reserve ``new_tokens[i]`` positions for each sequence and build the device-side metadata."""
        slots: List[int] = []
        pos: List[int] = []
        q_start, q_lens, seq_lens = [], [], []
        for sid, n in zip(seq_ids, new_tokens):
            start = self.seqs[sid].length
            q_start.append(len(slots))
            slots.extend(self.reserve(sid, n))
            if self.window > 0:
                self._evict_outside_window(sid, start)
            pos.extend(range(start, start + n))
            q_lens.append(n)
            seq_lens.append(start + n)
        mb = max(len(self.seqs[s].blocks) for s in seq_ids)
        bt = torch.zeros(len(seq_ids), mb, dtype=torch.int32)
        for i, sid in enumerate(seq_ids):
            bl = self.seqs[sid].blocks
            bt[i, :len(bl)] = torch.tensor(bl, dtype=torch.int32).clamp_(min=0)   # recycled blocks are never visited
        dev = self.device

        def t(x, dt):
            return torch.tensor(x, dtype=dt).to(dev, non_blocking=True)
        return BatchMeta(list(seq_ids), bt.to(dev, non_blocking=True), t(seq_lens, torch.int32), t(q_start, torch.int32),
                         t(q_lens, torch.int32), t(slots, torch.int64), t(pos, torch.int32), len(slots),
                         max(q_lens), max(seq_lens), host=(slots, pos, seq_lens, q_start, q_lens, bt))

    def _evict_outside_window(self, seq_id: int, first_query_pos: int) -> None:
        """Give back the blocks that no query at or after ``first_query_pos`` can see: blocks that end before
        ``first_query_pos - window + 1`` and start at or after ``sink`` (the same rule as the attention kernel's)."""
        st = self.seqs[seq_id]
        for bi, b in enumerate(st.blocks):
            if b >= 0 and bi * BLOCK + BLOCK - 1 < first_query_pos - self.window + 1 and bi * BLOCK >= self.sink:
                self._release(b)
                st.blocks[bi] = -1

    def live_blocks(self, seq_id: int) -> int:
        return sum(1 for b in self.seqs[seq_id].blocks if b >= 0)

    # ------------------------------------------------------------------ device-side append / attention
    def append(self, layer: int, k: torch.Tensor, v: torch.Tensor, slots: torch.Tensor) -> None:
        """k, v [n, hkv, d] of the new tokens -> cache slots (quantised on the way in for the int8 cache)."""
        from ..ops import native as nat
        if self.quant == "int8":
            nat.kv_append_q8(k, v, self.k[layer], self.v[layer], self.k_scale[layer], self.v_scale[layer], slots)
        elif self.quant == "tq4":
            nat.kv_append_tq4(k, v, self.k[layer], self.v[layer], self.k_scale[layer], self.v_scale[layer], slots,
                              self.tq.sign, self.tq.thresholds)
        else:
            nat.kv_append(k, v, self.k[layer], self.v[layer], slots)

    def attention(self, layer: int, q: torch.Tensor, meta: "BatchMeta", scale: float, window: int = 0) -> torch.Tensor:
        """Block-table attention of the new queries over this layer's cache. A model-level sliding window and the
        cache's own rotating window combine to the smaller of the two; the sink applies to the cache's window."""
        from ..ops import native as nat
        win = min(w for w in (window, self.window) if w > 0) if (window > 0 or self.window > 0) else 0
        if self.quant == "tq4":
            # keys and values are stored in the rotated basis: rotate the queries once, attend there, rotate the result back
            o = nat.paged_attn(nat.tq_rotate(q.contiguous(), self.tq.sign), self.k[layer], self.v[layer], meta, scale, win,
                               sink=self.sink if self.window > 0 else 0, k_scale=self.k_scale[layer],
                               v_scale=self.v_scale[layer], lut=self.tq_lut)
            return nat.tq_rotate(o, self.tq.sign, inverse=True)
        return nat.paged_attn(q, self.k[layer], self.v[layer], meta, scale, win, sink=self.sink if self.window > 0 else 0,
                              k_scale=self.k_scale[layer] if self.quant else None,
                              v_scale=self.v_scale[layer] if self.quant else None)

    # ------------------------------------------------------------------ reference gather (CPU path / tests)
    def quantize_rows(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Reference of the append kernel's quantiser: x [n, hkv, d] -> (int8 codes, fp32 scales [n, hkv, d/64])."""
        g = x.float().reshape(x.shape[0], x.shape[1], -1, GROUP)
        mx = g.abs().amax(-1)
        sc = torch.where(mx > 0, mx / 127.0, torch.ones_like(mx))
        q = torch.clamp(torch.round(g / sc[..., None]), -127, 127).to(torch.int8)
        return q.reshape(x.shape), sc

    def write_reference(self, layer: int, k: torch.Tensor, v: torch.Tensor, slots: torch.Tensor) -> None:
        """PyTorch statement of ``append`` (CPU path and the oracle of the GPU test)."""
        for cache, scales, x in ((self.k[layer], self.k_scale, k), (self.v[layer], self.v_scale, v)):
            flat = cache.view(-1, self.hkv, self.d)
            if self.quant == "int8":
                q, sc = self.quantize_rows(x)
                flat[slots] = q
                scales[layer].view(-1, self.hkv, self.d // GROUP)[slots] = sc
            elif self.quant == "tq4":
                c = self.tq.encode(x.float())
                cache.view(-1, self.hkv, self.d // 2)[slots] = c.codes
                sc = (x.float().norm(dim=-1) / self.d ** 0.5)[..., None].expand(-1, -1, self.d // GROUP)
                scales[layer].view(-1, self.hkv, self.d // GROUP)[slots] = sc
            else:
                flat[slots] = x.to(flat.dtype)

    def gather(self, layer: int, seq_id: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Dense [length, hkv, d] keys and values of a sequence (recycled blocks read as zeros; they are masked)."""
        st = self.seqs[seq_id]
        idx = torch.tensor([max(b, 0) for b in st.blocks], dtype=torch.int64, device=self.device)
        return self.gather_blocks(layer, idx, st.length)

    def gather_blocks(self, layer: int, idx: torch.Tensor, length: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Dense [length, hkv, d] keys and values behind a row of a block table (``idx`` int64, one entry per block)."""
        idx = idx[:(length + BLOCK - 1) // BLOCK].long()
        out = []
        for cache, scales in ((self.k[layer], self.k_scale), (self.v[layer], self.v_scale)):
            x = cache[idx]
            if self.quant == "int8":
                sc = scales[layer][idx]
                x = (x.float().reshape(*x.shape[:-1], -1, GROUP) * sc[..., None]).reshape(x.shape).to(self.compute_dtype)
            elif self.quant == "tq4":
                from .turboquant import unpack_bits
                sc = scales[layer][idx][..., 0]                                     # |x| / sqrt(d) per (token, head)
                y = self.tq.centroids[unpack_bits(x, 4, self.d).long()] * sc[..., None]
                x = self.tq.unrotate(y).to(self.compute_dtype)                      # back in the original basis
            out.append(x.reshape(-1, self.hkv, self.d)[:length])
        return out[0], out[1]
