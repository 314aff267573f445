"""Dequantisers for the GGUF i-quant formats with grid code books: IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S, IQ1_S, IQ1_M.

Each 256-element super-block stores, per group of eight (IQ2, IQ1) or four (IQ3) values, an index into a grid of
magnitudes (``iq_grids.py``), a sign mask, and a small integer scale per 32 (or 16) values on top of one f16 scale.
All decoders here work on whole tensors at once with numpy indexing: ``[blocks, ...]`` arrays of indices, signs and
scales are built from the raw bytes and the grid is gathered in one step. Behaviour parity:
crates/pmetal-gguf/src/iq_quants.rs:1155-1660 (``dequantize_iq*_bytes``); IQ4_NL / IQ4_XS live in the native host library.
"""
from __future__ import annotations

from typing import Callable, Dict

import numpy as np

from .iq_grids import KSIGNS, grid
from .types import BLOCK_GEOMETRY, GgmlType

IQ1_DELTA = 0.125
_BITS = (1 << np.arange(8, dtype=np.uint8))


def _blocks(raw: np.ndarray, t: GgmlType) -> np.ndarray:
    elems, nbytes = BLOCK_GEOMETRY[t]
    assert elems == 256
    if raw.size % nbytes:
        raise ValueError(f"{t.name}: {raw.size} bytes is not a whole number of {nbytes}-byte blocks")
    return raw.reshape(-1, nbytes)


def _f16(b: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(b).view("<f2").astype(np.float32)[:, 0]


def _signs(mask: np.ndarray) -> np.ndarray:
    """uint8 sign masks [...] -> float32 [..., 8] of +1 / -1 (bit j set = value j negative)."""
    return 1.0 - 2.0 * ((mask[..., None] & _BITS) != 0).astype(np.float32)


def _u16(b: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(b).view("<u2")


def _u32(b: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(b).view("<u4")


def dequant_iq2_xxs(raw: np.ndarray) -> np.ndarray:
    """Block {d f16, qs u16[32]}: per 32 values two u32 words: four grid bytes; four 7-bit sign indices + a 4-bit scale."""
    b = _blocks(raw, GgmlType.IQ2_XXS)
    d = _f16(b[:, 0:2])
    w = _u32(b[:, 2:66]).reshape(-1, 8, 2)                       # [nb, ib32, (indices, signs+scale)]
    idx = np.ascontiguousarray(w[:, :, 0]).view(np.uint8).reshape(-1, 8, 4)
    aux = w[:, :, 1]
    db = d[:, None] * (0.5 + (aux >> 28).astype(np.float32)) * 0.25
    sidx = (aux[:, :, None] >> (7 * np.arange(4, dtype=np.uint32))) & 127
    vals = grid("IQ2XXS")[idx].astype(np.float32) * _signs(KSIGNS[sidx])          # [nb, 8, 4, 8]
    return (vals * db[:, :, None, None]).reshape(-1)


def dequant_iq2_xs(raw: np.ndarray) -> np.ndarray:
    """Block {d, qs u16[32], scales u8[8]}: each u16 = 9-bit grid index + 7-bit sign index; a 4-bit scale per 16 values."""
    b = _blocks(raw, GgmlType.IQ2_XS)
    d = _f16(b[:, 0:2])
    q = _u16(b[:, 2:66]).reshape(-1, 8, 4)
    sc = b[:, 66:74]
    ls = np.stack((sc & 15, sc >> 4), axis=-1).astype(np.float32)                # [nb, 8, 2]: first / second 16 values
    db = d[:, None, None] * (0.5 + ls) * 0.25
    vals = grid("IQ2XS")[q & 511].astype(np.float32) * _signs(KSIGNS[q >> 9])     # [nb, 8, 4, 8]
    return (vals * np.repeat(db, 2, axis=2)[:, :, :, None]).reshape(-1)


def dequant_iq2_s(raw: np.ndarray) -> np.ndarray:
    """Block {d, qs[32] low index bytes, signs[32], qh[8] (2 high index bits per group), scales[8]}."""
    b = _blocks(raw, GgmlType.IQ2_S)
    d = _f16(b[:, 0:2])
    lo = b[:, 2:34].reshape(-1, 8, 4).astype(np.uint16)
    sg = b[:, 34:66].reshape(-1, 8, 4)
    qh = b[:, 66:74].astype(np.uint16)
    sc = b[:, 74:82]
    hi = (qh[:, :, None] >> (2 * np.arange(4, dtype=np.uint16))) & 3
    ls = np.stack((sc & 15, sc >> 4), axis=-1).astype(np.float32)
    db = d[:, None, None] * (0.5 + ls) * 0.25
    vals = grid("IQ2S")[lo | (hi << 8)].astype(np.float32) * _signs(sg)
    return (vals * np.repeat(db, 2, axis=2)[:, :, :, None]).reshape(-1)


def dequant_iq3_xxs(raw: np.ndarray) -> np.ndarray:
    """Block {d, qs[64] grid bytes (one per 4 values), 8 u32 words: four 7-bit sign indices + a 4-bit scale per 32 values}."""
    b = _blocks(raw, GgmlType.IQ3_XXS)
    d = _f16(b[:, 0:2])
    idx = b[:, 2:66].reshape(-1, 8, 4, 2)                                         # two grid entries per group of 8
    aux = _u32(b[:, 66:98])                                                       # [nb, 8]
    db = d[:, None] * (0.5 + (aux >> 28).astype(np.float32)) * 0.5
    sidx = (aux[:, :, None] >> (7 * np.arange(4, dtype=np.uint32))) & 127
    vals = grid("IQ3XXS")[idx].astype(np.float32).reshape(-1, 8, 4, 8) * _signs(KSIGNS[sidx])
    return (vals * db[:, :, None, None]).reshape(-1)


def dequant_iq3_s(raw: np.ndarray) -> np.ndarray:
    """Block {d, qs[64], qh[8] (ninth index bit per group of 4), signs[32], scales[4] (a nibble per 32 values)}."""
    b = _blocks(raw, GgmlType.IQ3_S)
    d = _f16(b[:, 0:2])
    lo = b[:, 2:66].reshape(-1, 8, 8).astype(np.uint16)                           # [nb, ib32, 8 groups of 4]
    qh = b[:, 66:74].astype(np.uint16)
    sg = b[:, 74:106].reshape(-1, 8, 4)
    sc = b[:, 106:110]
    hi = (qh[:, :, None] >> np.arange(8, dtype=np.uint16)) & 1
    ls = np.stack((sc & 15, sc >> 4), axis=-1).reshape(-1, 8).astype(np.float32)
    db = d[:, None] * (1.0 + 2.0 * ls)
    vals = grid("IQ3S")[lo | (hi << 8)].astype(np.float32).reshape(-1, 8, 4, 8) * _signs(sg)
    return (vals * db[:, :, None, None]).reshape(-1)


def dequant_iq1_s(raw: np.ndarray) -> np.ndarray:
    """Block {d, qs[32], qh u16[8]}: per 32 values a u16 holds four 3-bit high index parts, a 3-bit scale and the sign of
    the shared offset; values are scale * (grid + offset) with grid in {-1, 0, 1}."""
    b = _blocks(raw, GgmlType.IQ1_S)
    d = _f16(b[:, 0:2])
    lo = b[:, 2:34].reshape(-1, 8, 4).astype(np.uint16)
    qh = _u16(b[:, 34:50])                                                        # [nb, 8]
    hi = (qh[:, :, None] >> (3 * np.arange(4, dtype=np.uint16))) & 7
    dl = d[:, None] * (2.0 * ((qh >> 12) & 7).astype(np.float32) + 1.0)
    delta = np.where(qh & 0x8000, -IQ1_DELTA, IQ1_DELTA).astype(np.float32)
    vals = grid("IQ1S")[lo | (hi << 8)].astype(np.float32) + delta[:, :, None, None]
    return (vals * dl[:, :, None, None]).reshape(-1)


def dequant_iq1_m(raw: np.ndarray) -> np.ndarray:
    """Block {qs[32], qh[16], scales u16[4]} without a separate f16: the top nibbles of the four scale words spell it.
    Per 16 values a 3-bit scale; per 8 values a 3-bit high index part and the sign of the offset (nibbles of qh)."""
    b = _blocks(raw, GgmlType.IQ1_M)
    lo = b[:, 0:32].reshape(-1, 8, 4).astype(np.uint16)
    qh = b[:, 32:48].reshape(-1, 8, 2)
    sc = _u16(b[:, 48:56])                                                        # [nb, 4]
    dbits = ((sc[:, 0] >> 12) | ((sc[:, 1] >> 8) & 0x00f0) | ((sc[:, 2] >> 4) & 0x0f00) | (sc[:, 3] & 0xf000)).astype("<u2")
    d = dbits.view("<f2").astype(np.float32)
    nib = np.stack((qh[:, :, 0] & 15, qh[:, :, 0] >> 4, qh[:, :, 1] & 15, qh[:, :, 1] >> 4), axis=-1)   # [nb, 8, 4]
    idx = lo | ((nib.astype(np.uint16) & 7) << 8)
    delta = np.where(nib & 8, -IQ1_DELTA, IQ1_DELTA).astype(np.float32)
    # 3-bit scales: word ib/2, bits 6*(ib%2) .. +2 for the first 16 values and +3 .. +5 for the second
    word = np.repeat(sc, 2, axis=1)                                               # [nb, 8]
    base = 6 * (np.arange(8, dtype=np.uint16) % 2)
    s = np.stack(((word >> base) & 7, (word >> (base + 3)) & 7), axis=-1).astype(np.float32)           # [nb, 8, 2]
    dl = d[:, None, None] * (2.0 * s + 1.0)
    vals = grid("IQ1S")[idx].astype(np.float32) + delta[:, :, :, None]
    return (vals * np.repeat(dl, 2, axis=2)[:, :, :, None]).reshape(-1)


DEQUANTIZERS: Dict[GgmlType, Callable[[np.ndarray], np.ndarray]] = {
    GgmlType.IQ2_XXS: dequant_iq2_xxs, GgmlType.IQ2_XS: dequant_iq2_xs, GgmlType.IQ2_S: dequant_iq2_s,
    GgmlType.IQ3_XXS: dequant_iq3_xxs, GgmlType.IQ3_S: dequant_iq3_s, GgmlType.IQ1_S: dequant_iq1_s,
    GgmlType.IQ1_M: dequant_iq1_m,
}


def dequantize(raw: np.ndarray, t: GgmlType, n_elements: int) -> np.ndarray:
    """uint8 block bytes -> float32 [n_elements] for the grid-coded i-quant types."""
    t = GgmlType(t)
    if t not in DEQUANTIZERS:
        raise NotImplementedError(f"{t.name} is not a grid-coded i-quant type")
    elems, nbytes = BLOCK_GEOMETRY[t]
    nb = (n_elements + elems - 1) // elems
    raw = np.ascontiguousarray(raw).reshape(-1).view(np.uint8)
    if raw.size < nb * nbytes:
        raise ValueError(f"{t.name}: need {nb * nbytes} bytes for {n_elements} elements, got {raw.size}")
    return np.ascontiguousarray(DEQUANTIZERS[t](raw[:nb * nbytes])[:n_elements])
