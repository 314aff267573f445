"""Block-paged KV cache with reference-counted blocks.

The reference's ``PagedKVCache`` (crates/pmetal-mlx/src/kv_cache/paged.rs:10-720) is a block
allocator plus per-sequence block table, but attention still runs on a gathered dense tensor; here
the block table is consumed directly by the decode/verify attention kernel. Blocks hold 64 tokens
(one key tile of the kernel). ``fork`` shares full blocks between sequences (prompt prefix reuse
for group rollouts and the serving prefix cache) and copies the partially filled tail block.
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


class PagedKVCache:
    def __init__(self, num_layers: int, num_kv_heads: int, head_dim: int, num_blocks: int, dtype=torch.bfloat16,
                 device="cuda"):
        self.num_layers, self.hkv, self.d, self.num_blocks = num_layers, num_kv_heads, head_dim, num_blocks
        self.device = torch.device(device)
        shape = (num_blocks, BLOCK, num_kv_heads, head_dim)
        self.k = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(num_layers)]
        self.v = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(num_layers)]
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
        """Make room for ``n`` more tokens; returns their slots (block*64+offset) and advances the length."""
        st = self.seqs[seq_id]
        slots = []
        for i in range(n):
            pos = st.length + i
            bi = pos // BLOCK
            if bi == len(st.blocks):
                st.blocks.append(self._take())
            elif pos % BLOCK == 0 and False:
                pass
            b = st.blocks[bi]
            if self.ref[b] > 1:          # copy-on-write of a shared, partially filled block
                nb = self._take()
                for l in range(self.num_layers):
                    self.k[l][nb].copy_(self.k[l][b])
                    self.v[l][nb].copy_(self.v[l][b])
                self._release(b)
                st.blocks[bi] = b = nb
            slots.append(b * BLOCK + pos % BLOCK)
        st.length += n
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
            pos.extend(range(start, start + n))
            q_lens.append(n)
            seq_lens.append(start + n)
        mb = max(len(self.seqs[s].blocks) for s in seq_ids)
        bt = torch.zeros(len(seq_ids), mb, dtype=torch.int32)
        for i, sid in enumerate(seq_ids):
            bl = self.seqs[sid].blocks
            bt[i, :len(bl)] = torch.tensor(bl, dtype=torch.int32)
        dev = self.device

        def t(x, dt):
            return torch.tensor(x, dtype=dt).to(dev, non_blocking=True)
        return BatchMeta(list(seq_ids), bt.to(dev, non_blocking=True), t(seq_lens, torch.int32), t(q_start, torch.int32),
                         t(q_lens, torch.int32), t(slots, torch.int64), t(pos, torch.int32), len(slots),
                         max(q_lens), max(seq_lens))

    # ------------------------------------------------------------------ reference gather (CPU path / tests)
    def gather(self, layer: int, seq_id: int) -> Tuple[torch.Tensor, torch.Tensor]:
        st = self.seqs[seq_id]
        idx = torch.tensor(st.blocks, dtype=torch.int64, device=self.device)
        k = self.k[layer][idx].reshape(-1, self.hkv, self.d)[:st.length]
        v = self.v[layer][idx].reshape(-1, self.hkv, self.d)[:st.length]
        return k, v
