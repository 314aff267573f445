"""Ring all-reduce and barrier over a message transport (CPU reference of the collective).

The arithmetic is the reference's (crates/pmetal-distributed/src/ring.rs:48-254): the buffer is cut into N
chunks (chunk i has len/N elements plus one for the first len%N chunks); N-1 scatter-reduce steps, after
which rank r owns the fully reduced chunk (r+1)%N; N-1 all-gather steps; Mean divides by N at the end.
Each step sends and receives concurrently under a 30 s timeout; a missing peer surfaces as
``PeerTimeout`` ("peer may have crashed"). The barrier is two passes of a sequence-numbered token.
The GPU product path is ``parallel.fused_dp``; this module is the oracle for it and the engine of the
``cluster`` CPU diagnostics.
"""
from __future__ import annotations

import struct
import threading
from typing import List, Tuple

import numpy as np

from .errors import PeerTimeout, ProtocolError

STEP_TIMEOUT = 30.0


def chunk_bounds(length: int, world: int) -> List[Tuple[int, int]]:
    base, rem = divmod(length, world)
    out, off = [], 0
    for i in range(world):
        n = base + (1 if i < rem else 0)
        out.append((off, off + n))
        off += n
    return out


class RingBackend:
    def __init__(self, transport, rank: int, world: int, step_timeout: float = STEP_TIMEOUT):
        self.t, self.rank, self.world, self.timeout = transport, rank, world, step_timeout
        self._seq = 0

    def _exchange(self, payload: bytes) -> bytes:
        err: List[BaseException] = []

        def tx():
            try:
                self.t.send(payload)
            except BaseException as e:
                err.append(e)
        th = threading.Thread(target=tx, daemon=True)
        th.start()
        try:
            got = self.t.recv(self.timeout)
        except PeerTimeout as e:
            raise PeerTimeout(f"ring step timed out after {self.timeout} s: peer may have crashed") from e
        th.join(self.timeout)
        if err:
            raise err[0]
        return got

    def all_reduce(self, buf: np.ndarray, op: str = "sum") -> np.ndarray:
        """In-place on a float32 array. ``op``: "sum" | "mean"."""
        if buf.dtype != np.float32 or not buf.flags["C_CONTIGUOUS"]:
            raise ValueError("all_reduce expects a contiguous float32 buffer")
        n = self.world
        if n == 1:
            return buf
        flat = buf.reshape(-1)
        bounds = chunk_bounds(flat.size, n)
        for step in range(n - 1):                              # scatter-reduce
            s_lo, s_hi = bounds[(self.rank - step) % n]
            r_lo, r_hi = bounds[(self.rank - step - 1) % n]
            got = np.frombuffer(self._exchange(flat[s_lo:s_hi].tobytes()), dtype=np.float32)
            if got.size != r_hi - r_lo:
                raise ProtocolError(f"chunk length mismatch: got {got.size}, expected {r_hi - r_lo}")
            flat[r_lo:r_hi] += got
        for step in range(n - 1):                              # all-gather
            s_lo, s_hi = bounds[(self.rank + 1 - step) % n]
            r_lo, r_hi = bounds[(self.rank - step) % n]
            got = np.frombuffer(self._exchange(flat[s_lo:s_hi].tobytes()), dtype=np.float32)
            if got.size != r_hi - r_lo:
                raise ProtocolError(f"chunk length mismatch: got {got.size}, expected {r_hi - r_lo}")
            flat[r_lo:r_hi] = got
        if op == "mean":
            flat /= n
        return buf

    def barrier(self) -> None:
        if self.world == 1:
            return
        self._seq += 1
        for phase in (0, 1):
            token = struct.pack("<QI", self._seq, phase)
            if self.rank == 0:
                self.t.send(token)
                got = self.t.recv(self.timeout)
            else:
                got = self.t.recv(self.timeout)
                self.t.send(token)
            seq, ph = struct.unpack("<QI", got)
            if seq != self._seq or ph != phase:
                raise ProtocolError(f"stale barrier token (seq {seq} phase {ph}, expected {self._seq}/{phase})")
