"""QLoRA: frozen base weights stored 4-bit (NF4/FP4) or int8, LoRA factors trained in full precision.

Counterpart of the reference's ``QLoraLinear`` (crates/pmetal-lora/src/qlora.rs:33-480), which dequantises
the weight on the CPU at every forward unless a dequantised cache is kept. Here the packed weight stays in
HBM; each forward/backward dequantises one projection group into a transient bf16 buffer with a CUDA
kernel and feeds the tcgen05 GEMM (input gradient reads the same buffer as an MN-major operand, so no
transposed copy exists).
"""
from __future__ import annotations

import torch

from .nf4 import QuantizedTensor, dequantize, quantize


def dequantize_weight(q: QuantizedTensor, dtype=torch.bfloat16) -> torch.Tensor:
    if q.data.is_cuda and q.scheme in ("nf4", "fp4") and dtype == torch.bfloat16:
        from ..ops import native
        if native.available():
            return native.dequant_4bit(q)
    if q.data.is_cuda and q.scheme == "fp8" and dtype == torch.bfloat16:
        from ..ops import native
        if native.available():
            return native.fp8_dequant(q.data, q.absmax).view(q.shape)
    return dequantize(q, dtype)


@torch.no_grad()
def quantize_base(model, scheme: str = "nf4", block_size: int = 64, double_quant: bool = False) -> int:
    """Quantise every projection group of ``model`` in place. Returns the bytes saved."""
    saved = 0
    for _, _, fl in model.fused_linears():
        w = fl.weight
        # quantise where the weight lives (GPU when available: the codebook search is plain tensor ops)
        q = quantize(w.detach(), scheme, block_size, double_quant)
        if q.data.device != w.device:
            q = q.to(w.device)
        saved += w.numel() * w.element_size() - q.nbytes()
        fl.qweight = q
        fl.weight = torch.nn.Parameter(torch.empty(0, dtype=w.dtype, device=w.device), requires_grad=False)
        fl.weight_t = None
    return saved
