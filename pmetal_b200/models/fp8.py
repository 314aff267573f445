"""Block-scaled FP8 (E4M3) weights for inference, FP8 checkpoint export / import.

The reference quantises weights to E4M3 at load time for ``--fp8`` inference
(crates/pmetal-mlx/src/fp8_quantization.rs, ``DynamicModel::quantize_fp8`` crates/pmetal-models/src/dispatcher.rs:813),
reads fp8 checkpoints (crates/pmetal-models/src/fp8_utils.rs) and has an fp8 merge path
(crates/pmetal-merge/src/fp8_merge.rs). Here every projection group stores E4M3 codes with one fp32 scale per 128
consecutive elements (scale = amax / 448); the forward dequantises a group into a transient bf16 buffer with a CUDA
kernel and feeds the tcgen05 GEMM, halving resident weight memory."""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

from ..lora.nf4 import QuantizedTensor

FP8_BLOCK = 128
FP8_MAX = 448.0


def fp8_quantize_tensor(w: torch.Tensor) -> QuantizedTensor:
    """Any float tensor whose numel is a multiple of 128 -> QuantizedTensor(scheme='fp8')."""
    shape = tuple(w.shape)
    if w.numel() % FP8_BLOCK:
        raise ValueError(f"numel {w.numel()} is not a multiple of {FP8_BLOCK}")
    if w.is_cuda and w.dtype == torch.bfloat16:
        from ..ops import native
        if native.available():
            q, sc = native.fp8_quant(w)
            return QuantizedTensor(q.reshape(-1), sc, None, 0.0, 1.0, shape, FP8_BLOCK, "fp8")
    x = w.detach().float().reshape(-1, FP8_BLOCK)
    amax = x.abs().amax(-1)
    sc = torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))
    q = (x / sc[:, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(torch.uint8).reshape(-1)
    return QuantizedTensor(q, sc, None, 0.0, 1.0, shape, FP8_BLOCK, "fp8")


@torch.no_grad()
def quantize_model_fp8(model) -> int:
    """Replace every projection group's weight by FP8 codes in place. Returns the bytes saved."""
    saved = 0
    for _, _, fl in model.fused_linears():
        w = fl.weight
        if w.numel() == 0 or w.numel() % FP8_BLOCK:
            continue
        q = fp8_quantize_tensor(w.detach())
        saved += w.numel() * w.element_size() - q.nbytes()
        fl.qweight = q
        fl.weight = torch.nn.Parameter(torch.empty(0, dtype=w.dtype, device=w.device), requires_grad=False)
        fl.weight_t = None
    return saved


def export_fp8_checkpoint(model_dir: str, out_dir: str) -> dict:
    """Writes ``model.safetensors`` with ``<name>`` (uint8 E4M3 codes) + ``<name>_scale_inv`` (fp32 per-128 scales) for
    every 2-D weight and the other tensors unchanged, plus ``config.json`` with a ``quantization_config`` entry."""
    from ..utils import safetensors_io as st
    from .loader import read_state_dict
    sd = read_state_dict(model_dir)
    out: Dict[str, torch.Tensor] = {}
    n_q = 0
    for k, v in sd.items():
        if v.dim() == 2 and v.numel() % FP8_BLOCK == 0 and k.endswith(".weight") and "norm" not in k and "embed" not in k:
            q = fp8_quantize_tensor(v.to(torch.bfloat16))
            out[k] = q.data.view(v.shape).cpu()
            out[k + "_scale_inv"] = q.absmax.cpu()
            n_q += 1
        else:
            out[k] = v.contiguous()
    os.makedirs(out_dir, exist_ok=True)
    st.save_file(out, os.path.join(out_dir, "model.safetensors"), metadata={"format": "pt"})
    cfg_path = os.path.join(model_dir, "config.json")
    cfg = {}
    if os.path.exists(cfg_path):
        with open(cfg_path, "r", encoding="utf-8") as fh:
            cfg = json.load(fh)
    cfg["quantization_config"] = {"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": [1, FP8_BLOCK]}
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(cfg, fh, indent=2)
    return {"output": out_dir, "quantized_tensors": n_q, "bytes": sum(t.numel() * t.element_size() for t in out.values())}


def dequantize_fp8_state_dict(sd: Dict[str, torch.Tensor], dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Inverse of ``export_fp8_checkpoint`` for loading: merges ``name`` + ``name_scale_inv`` pairs."""
    out = {}
    for k, v in sd.items():
        if k.endswith("_scale_inv"):
            continue
        s = sd.get(k + "_scale_inv")
        if s is not None and v.dtype in (torch.uint8, torch.float8_e4m3fn):
            vals = v.view(torch.float8_e4m3fn).float().reshape(-1, FP8_BLOCK) * s.float()[:, None]
            out[k] = vals.reshape(v.shape).to(dtype)
        else:
            out[k] = v
    return out
