"""ctypes binding of the host C++ block codecs (``csrc/host/gguf_quant.cpp``)."""
from __future__ import annotations

import ctypes
import threading

import numpy as np

from .types import BLOCK_GEOMETRY, GgmlType, tensor_nbytes

from ..utils import hostlib

_LOCK = threading.Lock()
_LIB = None
CXX_FLAGS = hostlib.CXX_FLAGS


def build(force: bool = False) -> str:
    return hostlib.build(force)


def lib():
    global _LIB
    with _LOCK:
        if _LIB is None:
            L = hostlib.load()
            L.pm_gguf_quantize.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int]
            L.pm_gguf_dequantize.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int]
            L.pm_gguf_row_bytes.restype = ctypes.c_int64
            L.pm_gguf_row_bytes.argtypes = [ctypes.c_int, ctypes.c_int64]
            L.pm_gguf_vec_dot_q8k.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                              ctypes.POINTER(ctypes.c_float)]
            L.pm_gguf_matvec_q8k.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p,
                                             ctypes.c_void_p, ctypes.c_int]
            _LIB = L
    return _LIB


def can_quantize(t: GgmlType) -> bool:
    return t in (GgmlType.F32, GgmlType.F16, GgmlType.BF16, GgmlType.Q4_0, GgmlType.Q4_1, GgmlType.Q5_0, GgmlType.Q5_1,
                 GgmlType.Q8_0, GgmlType.Q8_1, GgmlType.Q2K, GgmlType.Q3K, GgmlType.Q4K, GgmlType.Q5K, GgmlType.Q6K,
                 GgmlType.Q8K, GgmlType.MXFP4, GgmlType.NVFP4, GgmlType.TQ1_0, GgmlType.TQ2_0, GgmlType.Q1_0)


GRID_IQ_TYPES = (GgmlType.IQ2_XXS, GgmlType.IQ2_XS, GgmlType.IQ2_S, GgmlType.IQ3_XXS, GgmlType.IQ3_S, GgmlType.IQ1_S,
                 GgmlType.IQ1_M)


def can_dequantize(t: GgmlType) -> bool:
    return can_quantize(t) or t in (GgmlType.IQ4_NL, GgmlType.IQ4_XS) or t in GRID_IQ_TYPES


def quantize(x: np.ndarray, t: GgmlType, threads: int = 0) -> np.ndarray:
    """float32 array (any shape, row-major) -> uint8 array of block bytes."""
    t = GgmlType(t)
    if not can_quantize(t):
        raise NotImplementedError(f"quantisation to {t.name} is not implemented (dequantise-only or unsupported type)")
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    out = np.zeros(tensor_nbytes(t, x.size), dtype=np.uint8)
    rc = lib().pm_gguf_quantize(int(t), x.ctypes.data, out.ctypes.data, x.size, threads)
    if rc == -2:
        raise NotImplementedError(f"quantisation to {t.name} is not implemented (dequantise-only type)")
    if rc != 0:
        raise ValueError(f"unknown ggml type {int(t)}")
    return out


def dequantize(buf, t: GgmlType, n_elements: int, threads: int = 0) -> np.ndarray:
    t = GgmlType(t)
    if not can_dequantize(t):
        raise NotImplementedError(f"dequantisation of {t.name} is not implemented")
    raw = np.frombuffer(buf, dtype=np.uint8) if not isinstance(buf, np.ndarray) else buf.reshape(-1).view(np.uint8)
    if t in GRID_IQ_TYPES:                      # grid-coded i-quants: vectorised numpy decoders (gguf/iq_quants.py)
        from . import iq_quants
        return iq_quants.dequantize(raw, t, n_elements)
    need = tensor_nbytes(t, n_elements)
    if raw.size < need:
        raise ValueError(f"{t.name}: need {need} bytes for {n_elements} elements, got {raw.size}")
    raw = np.ascontiguousarray(raw[:need])
    out = np.empty(n_elements, dtype=np.float32)
    rc = lib().pm_gguf_dequantize(int(t), raw.ctypes.data, out.ctypes.data, n_elements, threads)
    if rc == -2:
        raise NotImplementedError(f"dequantisation of {t.name} is not implemented")
    if rc != 0:
        raise ValueError(f"unknown ggml type {int(t)}")
    return out


VEC_DOT_TYPES = (GgmlType.Q2K, GgmlType.Q3K, GgmlType.Q4K, GgmlType.Q5K, GgmlType.Q6K, GgmlType.Q8K)


def vec_dot_q8k(x_blocks: np.ndarray, t: GgmlType, y_q8k: np.ndarray, n: int) -> float:
    """Integer dot product of ``n`` elements stored as K-quant blocks of type ``t`` with the same ``n`` elements of an
    activation row stored as Q8_K blocks (crates/pmetal-gguf/src/vec_dot.rs)."""
    t = GgmlType(t)
    if t not in VEC_DOT_TYPES:
        raise NotImplementedError(f"no integer dot product for {t.name}")
    if n <= 0 or n % 256:
        raise ValueError("n must be a positive multiple of 256")
    x = np.ascontiguousarray(x_blocks).reshape(-1).view(np.uint8)
    y = np.ascontiguousarray(y_q8k).reshape(-1).view(np.uint8)
    if x.size < tensor_nbytes(t, n) or y.size < tensor_nbytes(GgmlType.Q8K, n):
        raise ValueError("block buffers are shorter than n elements")
    out = ctypes.c_float(0.0)
    rc = lib().pm_gguf_vec_dot_q8k(int(t), x.ctypes.data, y.ctypes.data, n, ctypes.byref(out))
    if rc != 0:
        raise ValueError(f"pm_gguf_vec_dot_q8k failed with {rc}")
    return float(out.value)


def matvec_q8k(w_blocks: np.ndarray, t: GgmlType, rows: int, n: int, y: np.ndarray, threads: int = 0) -> np.ndarray:
    """``W @ y`` for a quantised row-major matrix ``W`` [rows, n] and a float32 vector ``y`` [n]: ``y`` is quantised to
    Q8_K once and every row is an integer dot product (the CPU inference path for quantised weights)."""
    t = GgmlType(t)
    if t not in VEC_DOT_TYPES:
        raise NotImplementedError(f"no integer dot product for {t.name}")
    if n <= 0 or n % 256:
        raise ValueError("n must be a positive multiple of 256")
    w = np.ascontiguousarray(w_blocks).reshape(-1).view(np.uint8)
    if w.size < rows * tensor_nbytes(t, n):
        raise ValueError("weight buffer is shorter than rows x n elements")
    yq = quantize(np.asarray(y, dtype=np.float32).reshape(-1)[:n], GgmlType.Q8K)
    out = np.empty(rows, dtype=np.float32)
    rc = lib().pm_gguf_matvec_q8k(int(t), w.ctypes.data, rows, n, yq.ctypes.data, out.ctypes.data, threads)
    if rc != 0:
        raise ValueError(f"pm_gguf_matvec_q8k failed with {rc}")
    return out


__all__ = ["vec_dot_q8k", "matvec_q8k", "VEC_DOT_TYPES", "build", "lib", "quantize", "dequantize", "can_quantize", "can_dequantize", "BLOCK_GEOMETRY"]
