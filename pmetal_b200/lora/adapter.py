"""Attach LoRA factors to a model and read/write adapter files.

Adapter file contract (crates/pmetal-lora/src/lora_helpers.rs:71-117,207-236 and
crates/pmetal-lora/src/lora.rs:268-289):

* keys ``layers.{i}.self_attn.{q,k,v,o}_proj.lora_{a,b}`` and
  ``layers.{i}.mlp.{gate,up,down}_proj.lora_{a,b}`` — no ``model.`` prefix;
* ``lora_a`` is [r, in], ``lora_b`` is [out, r], both F32;
* all seven projections of every layer are written; a projection that is not a
  target is written as the rank-0 placeholders ``lora_a = zeros[1, in]`` and
  ``lora_b = zeros[out, 1]``;
* ``adapter_config.json`` is pretty-printed
  ``{"r", "alpha", "target_modules", "use_rslora"[, "base_model"]}``
  (crates/pmetal-trainer/src/orchestrator.rs:1880-1904).
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

import torch

from ..core.config import LoraConfig
from ..models.decoder import ALL_PROJ, DecoderLM
from ..utils import safetensors_io as st

WEIGHTS_NAME = "lora_weights.safetensors"
CONFIG_NAME = "adapter_config.json"


def apply_lora(model: DecoderLM, cfg: LoraConfig, seed: int = 42) -> DecoderLM:
    """Add trainable LoRA factors to the targeted projections and freeze everything else."""
    g = torch.Generator().manual_seed(seed)
    targets = set(cfg.target_modules)
    for _, _, fl in model.fused_linears():
        active = [n in targets for n in fl.seg_names]
        fl.add_lora(cfg.r, cfg.scaling(), active, cfg.use_rslora, g)
    model.freeze_base()
    if cfg.use_dora:
        from .dora import attach_dora
        attach_dora(model)
    return model


def lora_state_dict(model: DecoderLM) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for i, scope, fl in model.fused_linears():
        o = 0
        for j, (nm, sz) in enumerate(zip(fl.seg_names, fl.seg_sizes)):
            key = f"layers.{i}.{scope}.{nm}"
            if fl.lora_a is not None and fl.active[j]:
                out[key + ".lora_a"] = fl.lora_a.detach()[j * fl.r:(j + 1) * fl.r].float().cpu().contiguous()
                out[key + ".lora_b"] = fl.lora_b.detach()[o:o + sz].float().cpu().contiguous()
            else:
                out[key + ".lora_a"] = torch.zeros(1, fl.in_features, dtype=torch.float32)
                out[key + ".lora_b"] = torch.zeros(sz, 1, dtype=torch.float32)
            mag = getattr(fl, "dora_magnitude", None)
            if mag is not None and fl.active[j]:
                out[key + ".magnitude"] = mag.detach()[o:o + sz].float().cpu().reshape(sz, 1).contiguous()
            o += sz
    return out


def save_adapter(model: DecoderLM, out_dir: str, cfg: LoraConfig, base_model: Optional[str] = None) -> str:
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, WEIGHTS_NAME)
    st.save_file(lora_state_dict(model), path, metadata={"format": "mlx"})
    save_adapter_config(out_dir, cfg, base_model)
    return path


def save_adapter_config(out_dir: str, cfg: LoraConfig, base_model: Optional[str] = None) -> str:
    d = {"r": cfg.r, "alpha": cfg.alpha, "target_modules": list(cfg.target_modules), "use_rslora": cfg.use_rslora}
    if base_model:
        d["base_model"] = base_model
    p = os.path.join(out_dir, CONFIG_NAME)
    with open(p, "w", encoding="utf-8") as fh:
        json.dump(d, fh, indent=2)
    return p


def load_adapter_config(path: str) -> LoraConfig:
    if os.path.isdir(path):
        path = os.path.join(path, CONFIG_NAME)
    with open(path, "r", encoding="utf-8") as fh:
        d = json.load(fh)
    return LoraConfig(r=int(d.get("r", 16)), alpha=float(d.get("alpha", 32.0)),
                      target_modules=list(d.get("target_modules", ["q_proj", "k_proj", "v_proj", "o_proj"])),
                      use_rslora=bool(d.get("use_rslora", False)))


def resolve_adapter_file(path: str) -> str:
    """A directory means ``<dir>/lora_weights.safetensors`` (lora_helpers.rs:218-236)."""
    return os.path.join(path, WEIGHTS_NAME) if os.path.isdir(path) else path


@torch.no_grad()
def load_adapter(model: DecoderLM, path: str, strict: bool = False) -> int:
    """Copy adapter tensors into an already LoRA-wrapped model. Unknown keys are ignored and rank-0
    placeholders are skipped. Returns the number of tensors loaded."""
    tensors = st.load_file(resolve_adapter_file(path))
    n = 0
    for i, scope, fl in model.fused_linears():
        if fl.lora_a is None:
            continue
        o = 0
        for j, (nm, sz) in enumerate(zip(fl.seg_names, fl.seg_sizes)):
            key = f"layers.{i}.{scope}.{nm}"
            a, b = tensors.get(key + ".lora_a"), tensors.get(key + ".lora_b")
            if a is not None and b is not None and a.shape[0] == fl.r and b.shape[1] == fl.r:
                fl.lora_a[j * fl.r:(j + 1) * fl.r].copy_(a.to(fl.lora_a.dtype))
                fl.lora_b[o:o + sz].copy_(b.to(fl.lora_b.dtype))
                n += 2
            elif strict and fl.active[j]:
                raise KeyError(f"adapter file lacks rank-{fl.r} factors for {key}")
            mag = getattr(fl, "dora_magnitude", None)
            if mag is not None and key + ".magnitude" in tensors:
                mag[o:o + sz].copy_(tensors[key + ".magnitude"].reshape(-1).to(mag.dtype))
            o += sz
    return n


def infer_rank_from_file(path: str) -> int:
    """Rank from the first attention ``lora_a`` with more than one row (commands/fuse.rs:67-81)."""
    with st.LazyFile(resolve_adapter_file(path)) as f:
        for k in sorted(f.keys()):
            if "self_attn" in k and k.endswith("lora_a"):
                _, shape = f.info(k)
                if shape[0] > 1:
                    return shape[0]
    return 0


@torch.no_grad()
def merge_adapter_into_base(model: DecoderLM) -> None:
    """Fold s·B·A into the base weights and drop the factors."""
    for _, _, fl in model.fused_linears():
        if fl.lora_a is not None:
            fl.weight.copy_(fl.merged_weight().to(fl.weight.dtype))
            fl.lora_a = fl.lora_b = None
            fl.r = 0
