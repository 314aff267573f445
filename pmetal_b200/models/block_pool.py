"""Reference-counted KV block pool (``csrc/host/runtime.cpp: pm_pool_*``).

The bookkeeping half of a paged KV cache, in native code: per-sequence block lists, a LIFO free list, reference counts so
that forked sequences (prefix sharing, beam or tree search, GRPO rollouts of one prompt) share blocks, copy-on-write of a
shared tail block, and the ``[n_seqs, max_blocks]`` block table / length arrays a decode launch reads. It owns no device
memory: the caller performs the block copies it reports and indexes its own K/V tensors with the returned slots.
The reference keeps one contiguous cache per sequence (crates/pmetal-mlx/src/kv_cache.rs:1-120); paging is what lets many
sequences of unknown final length share 180 GB without reserving the maximum for each."""
from __future__ import annotations

import ctypes
from typing import List, Sequence, Tuple

import numpy as np

from ..utils import hostlib

_READY = False


def _lib():
    global _READY
    L = hostlib.load()
    if not _READY:
        c = ctypes
        L.pm_pool_create.restype = c.c_void_p
        L.pm_pool_create.argtypes = [c.c_int32, c.c_int32]
        L.pm_pool_destroy.argtypes = [c.c_void_p]
        L.pm_pool_num_free.argtypes = [c.c_void_p]
        L.pm_pool_ref.argtypes = [c.c_void_p, c.c_int32]
        for name in ("pm_pool_add", "pm_pool_free", "pm_pool_num_blocks"):
            getattr(L, name).argtypes = [c.c_void_p, c.c_int64]
        L.pm_pool_length.restype = c.c_int64
        L.pm_pool_length.argtypes = [c.c_void_p, c.c_int64]
        L.pm_pool_blocks_needed.argtypes = [c.c_void_p, c.c_int64, c.c_int64]
        L.pm_pool_reserve.argtypes = [c.c_void_p, c.c_int64, c.c_int64, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p]
        L.pm_pool_truncate.argtypes = [c.c_void_p, c.c_int64, c.c_int64]
        L.pm_pool_fork.argtypes = [c.c_void_p, c.c_int64, c.c_int64]
        L.pm_pool_tables.argtypes = [c.c_void_p, c.c_void_p, c.c_int64, c.c_int32, c.c_void_p, c.c_void_p]
        _READY = True
    return L


class BlockPool:
    def __init__(self, num_blocks: int, block_size: int):
        self.num_blocks, self.block_size = int(num_blocks), int(block_size)
        self._L = _lib()
        self._h = self._L.pm_pool_create(self.num_blocks, self.block_size)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._L.pm_pool_destroy(h)

    @property
    def num_free(self) -> int:
        return self._L.pm_pool_num_free(self._h)

    def ref(self, block: int) -> int:
        return self._L.pm_pool_ref(self._h, int(block))

    def add(self, seq: int) -> None:
        if self._L.pm_pool_add(self._h, int(seq)) != 0:
            raise KeyError(f"sequence {seq} already exists")

    def free(self, seq: int) -> None:
        if self._L.pm_pool_free(self._h, int(seq)) != 0:
            raise KeyError(seq)

    def length(self, seq: int) -> int:
        n = self._L.pm_pool_length(self._h, int(seq))
        if n < 0:
            raise KeyError(seq)
        return n

    def blocks_needed(self, seq: int, n: int) -> int:
        r = self._L.pm_pool_blocks_needed(self._h, int(seq), int(n))
        if r < 0:
            raise KeyError(seq)
        return r

    def reserve(self, seq: int, n: int) -> Tuple[List[int], List[Tuple[int, int]]]:
        """Slots of the ``n`` new tokens and the (source, destination) block copies to perform before writing them."""
        slots = np.empty(max(int(n), 1), dtype=np.int64)
        src, dst, nc = ctypes.c_int32(0), ctypes.c_int32(0), ctypes.c_int32(0)
        rc = self._L.pm_pool_reserve(self._h, int(seq), int(n), slots.ctypes.data, ctypes.byref(src), ctypes.byref(dst),
                                     ctypes.byref(nc))
        if rc == -1:
            raise KeyError(seq)
        if rc == -2:
            raise MemoryError("KV block pool exhausted")
        return slots[:int(n)].tolist(), ([(src.value, dst.value)] if nc.value else [])

    def truncate(self, seq: int, new_len: int) -> None:
        if self._L.pm_pool_truncate(self._h, int(seq), int(new_len)) != 0:
            raise KeyError(seq)

    def fork(self, src: int, dst: int) -> None:
        if self._L.pm_pool_fork(self._h, int(src), int(dst)) != 0:
            raise KeyError((src, dst))

    def tables(self, seqs: Sequence[int], max_blocks: int) -> Tuple[np.ndarray, np.ndarray]:
        ids = np.ascontiguousarray(seqs, dtype=np.int64)
        table = np.empty((len(ids), int(max_blocks)), dtype=np.int32)
        lens = np.empty(len(ids), dtype=np.int32)
        rc = self._L.pm_pool_tables(self._h, ids.ctypes.data, len(ids), int(max_blocks), table.ctypes.data, lens.ctypes.data)
        if rc == -1:
            raise KeyError("unknown sequence")
        if rc == -2:
            raise ValueError("a sequence holds more than max_blocks blocks")
        return table, lens
