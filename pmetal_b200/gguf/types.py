"""GGUF / ggml constants: type ids, block geometry, metadata value types.

Type ids and block sizes follow crates/pmetal-gguf/src/types.rs:14-171 of the reference (which follows ggml)."""
from __future__ import annotations

import enum

GGUF_MAGIC = 0x46554747          # "GGUF" little-endian
GGUF_VERSION = 3
GGUF_DEFAULT_ALIGNMENT = 32


class GgmlType(enum.IntEnum):
    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q4_1 = 3
    Q5_0 = 6
    Q5_1 = 7
    Q8_0 = 8
    Q8_1 = 9
    Q2K = 10
    Q3K = 11
    Q4K = 12
    Q5K = 13
    Q6K = 14
    Q8K = 15
    IQ2_XXS = 16
    IQ2_XS = 17
    IQ3_XXS = 18
    IQ1_S = 19
    IQ4_NL = 20
    IQ3_S = 21
    IQ2_S = 22
    IQ4_XS = 23
    I8 = 24
    I16 = 25
    I32 = 26
    I64 = 27
    F64 = 28
    IQ1_M = 29
    BF16 = 30
    TQ1_0 = 34
    TQ2_0 = 35
    MXFP4 = 39
    NVFP4 = 40
    Q1_0 = 41


# type -> (elements per block, bytes per block)
BLOCK_GEOMETRY = {
    GgmlType.F32: (1, 4), GgmlType.F16: (1, 2), GgmlType.BF16: (1, 2), GgmlType.F64: (1, 8),
    GgmlType.I8: (1, 1), GgmlType.I16: (1, 2), GgmlType.I32: (1, 4), GgmlType.I64: (1, 8),
    GgmlType.Q4_0: (32, 18), GgmlType.Q4_1: (32, 20), GgmlType.Q5_0: (32, 22), GgmlType.Q5_1: (32, 24),
    GgmlType.Q8_0: (32, 34), GgmlType.Q8_1: (32, 36),
    GgmlType.Q2K: (256, 84), GgmlType.Q3K: (256, 110), GgmlType.Q4K: (256, 144), GgmlType.Q5K: (256, 176),
    GgmlType.Q6K: (256, 210), GgmlType.Q8K: (256, 292),
    GgmlType.IQ4_NL: (32, 18), GgmlType.IQ4_XS: (256, 136),
    GgmlType.IQ2_XXS: (256, 66), GgmlType.IQ2_XS: (256, 74), GgmlType.IQ2_S: (256, 82), GgmlType.IQ3_XXS: (256, 98),
    GgmlType.IQ3_S: (256, 110), GgmlType.IQ1_S: (256, 50), GgmlType.IQ1_M: (256, 56),
    GgmlType.TQ1_0: (256, 54), GgmlType.TQ2_0: (256, 66), GgmlType.MXFP4: (32, 17), GgmlType.NVFP4: (64, 36),
    GgmlType.Q1_0: (128, 18),
}


def tensor_nbytes(t: GgmlType, n_elements: int) -> int:
    el, by = BLOCK_GEOMETRY[t]
    return -(-n_elements // el) * by


def bits_per_weight(t: GgmlType) -> float:
    el, by = BLOCK_GEOMETRY[t]
    return 8.0 * by / el


class ValueType(enum.IntEnum):
    UINT8 = 0
    INT8 = 1
    UINT16 = 2
    INT16 = 3
    UINT32 = 4
    INT32 = 5
    FLOAT32 = 6
    BOOL = 7
    STRING = 8
    ARRAY = 9
    UINT64 = 10
    INT64 = 11
    FLOAT64 = 12


# CLI method name -> (default ggml type, llama.cpp file-type id). Names as accepted by the reference CLI
# (crates/pmetal/src/main.rs:44-187).
QUANT_METHODS = {
    "dynamic": (GgmlType.Q4K, 15), "q8_0": (GgmlType.Q8_0, 7), "q8_1": (GgmlType.Q8_1, 7), "q6_k": (GgmlType.Q6K, 18),
    "q5_k_m": (GgmlType.Q5K, 17), "q5_k_s": (GgmlType.Q5K, 16), "q5_0": (GgmlType.Q5_0, 8), "q5_1": (GgmlType.Q5_1, 9),
    "q4_k_m": (GgmlType.Q4K, 15), "q4_k_s": (GgmlType.Q4K, 14), "q4_0": (GgmlType.Q4_0, 2), "q4_1": (GgmlType.Q4_1, 3),
    "q3_k_m": (GgmlType.Q3K, 12), "q3_k_s": (GgmlType.Q3K, 11), "q3_k_l": (GgmlType.Q3K, 13), "q2_k": (GgmlType.Q2K, 10),
    "q1_0": (GgmlType.Q1_0, 40), "tq1_0": (GgmlType.TQ1_0, 36), "tq2_0": (GgmlType.TQ2_0, 37),
    "mxfp4": (GgmlType.MXFP4, 38), "nvfp4": (GgmlType.NVFP4, 39), "bf16": (GgmlType.BF16, 32), "f16": (GgmlType.F16, 1),
    "f32": (GgmlType.F32, 0),
}
