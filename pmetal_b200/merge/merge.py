"""Merge driver: mergekit-style YAML, lazy safetensors loading, tensor-at-a-time streaming, layer slices.

Follows crates/pmetal-merge/src/{config.rs:145-600, merge.rs:73-1120, lora_merge.rs:60-1204}: a config
names ``merge_method``, ``models`` (each with optional per-model ``parameters``: weight, density),
``base_model``, global ``parameters`` (weight, density, lambda, t, rescale, ...), ``dtype``, optional
``slices`` (passthrough-style layer stacking) and ``tokenizer`` source. Tensors are read one name at a time
from memory-mapped checkpoints, merged on the compute device (CUDA when present) and written to
``model.safetensors`` + index, so peak memory is one tensor per input model. ``merge_lora_into_base``
folds an adapter into base weights in float64.
"""
from __future__ import annotations

import json
import os
import shutil
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..utils import safetensors_io as st
from .methods import METHODS, REQUIRES_BASE, MergeParameters, merge_tensor


@dataclass
class ModelEntry:
    model: str
    parameters: MergeParameters = field(default_factory=MergeParameters)


@dataclass
class OutputSlice:
    sources: List[dict]          # [{"model": path, "layer_range": [a, b]}]


@dataclass
class MergeConfig:
    merge_method: str = "linear"
    models: List[ModelEntry] = field(default_factory=list)
    base_model: Optional[str] = None
    output_path: Optional[str] = None
    dtype: str = "bfloat16"
    parameters: MergeParameters = field(default_factory=MergeParameters)
    tokenizer_source: Optional[str] = None
    slices: Optional[List[OutputSlice]] = None
    allow_mixed_dtype: bool = False
    dry_run: bool = False
    aux_paths: List[str] = field(default_factory=list)     # fisher / gram files for fisher and regmean
    align_moe_experts: bool = False                        # permute each model's experts onto the first model's before merging
    sanity: str = "quick"                                  # off | quick | full (merge/sanity.py)

    @staticmethod
    def _params(d: Optional[dict], base: Optional[MergeParameters] = None) -> MergeParameters:
        p = MergeParameters(**vars(base)) if base else MergeParameters()
        for k, v in (d or {}).items():
            k2 = "lambda_" if k == "lambda" else k
            if hasattr(p, k2):
                setattr(p, k2, v)
            else:
                p.extra[k] = v
        return p

    @classmethod
    def from_dict(cls, d: dict) -> "MergeConfig":
        mm = d.get("merge_method", "linear")
        aux: List[str] = []
        if isinstance(mm, dict):                       # {"fisher": {"fisher_paths": [...]}}
            (name, body), = mm.items()
            aux = list((body or {}).get("fisher_paths") or (body or {}).get("gram_paths") or [])
            mm = name
        mm = {"reg_mean": "regmean", "multi_slerp": "multislerp", "ram_plus": "ram"}.get(mm, mm)
        if mm not in METHODS:
            raise ValueError(f"unknown merge_method {mm!r}")
        g = cls._params(d.get("parameters"))
        models = [ModelEntry(m["model"], cls._params(m.get("parameters"), g)) for m in d.get("models", [])]
        slices = None
        if d.get("slices"):
            slices = [OutputSlice(list(s.get("sources", []))) for s in d["slices"]]
        tok = d.get("tokenizer") or {}
        return cls(mm, models, d.get("base_model"), d.get("output_path"), d.get("dtype", "bfloat16"), g,
                   tok.get("source") if isinstance(tok, dict) else tok, slices, bool(d.get("allow_mixed_dtype")),
                   bool(d.get("dry_run")), aux, bool(d.get("align_moe_experts") or d.get("align_experts")),
                   str(d.get("sanity", "quick")))

    @classmethod
    def from_yaml(cls, path: str) -> "MergeConfig":
        import yaml
        with open(path, "r", encoding="utf-8") as fh:
            return cls.from_dict(yaml.safe_load(fh))


class LazyCheckpoint:
    """All safetensors shards of a model directory, opened lazily."""

    def __init__(self, path: str):
        self.path = path
        files = [path] if path.endswith(".safetensors") else sorted(
            os.path.join(path, f) for f in os.listdir(path) if f.endswith(".safetensors") and "lora" not in f)
        if not files:
            raise FileNotFoundError(f"no safetensors in {path}")
        self.files = [st.LazyFile(f) for f in files]
        self.index: Dict[str, st.LazyFile] = {}
        for f in self.files:
            for k in f.keys():
                self.index[k] = f

    def keys(self):
        return list(self.index.keys())

    def get(self, name: str) -> torch.Tensor:
        return self.index[name].get(name)

    def close(self):
        for f in self.files:
            f.close()


def _dtype(name: str) -> torch.dtype:
    return {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[name]


def run_merge(cfg: MergeConfig, device: Optional[str] = None) -> dict:
    """Execute a merge; returns a summary. With ``dry_run`` only validates and reports the plan."""
    dev = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    if cfg.slices:
        return _run_slices(cfg)
    if cfg.merge_method in REQUIRES_BASE and not cfg.base_model:
        raise ValueError(f"merge method {cfg.merge_method} needs base_model")
    if len(cfg.models) < 1:
        raise ValueError("no models to merge")
    cks = [LazyCheckpoint(m.model) for m in cfg.models]
    base = LazyCheckpoint(cfg.base_model) if cfg.base_model else None
    aux = [st.load_file(p) for p in cfg.aux_paths]
    names = cks[0].keys()
    missing = [n for n in names for c in cks[1:] if n not in c.index]
    if missing:
        raise ValueError(f"tensor {missing[0]} is missing from one of the models")
    plan = {"method": cfg.merge_method, "tensors": len(names), "models": [m.model for m in cfg.models],
            "base": cfg.base_model, "dtype": cfg.dtype}
    alignment = None
    if cfg.align_moe_experts and len(cks) > 1:
        from .moe_align import align_experts
        alignment = align_experts(cks)
        if alignment is not None:
            plan["expert_alignment"] = {"layers": len(alignment.layers), "identity": alignment.is_identity()}
    if cfg.dry_run:
        return plan
    out: Dict[str, torch.Tensor] = {}
    odt = _dtype(cfg.dtype)
    params = [m.parameters for m in cfg.models]
    for n in names:
        ts = [(alignment.fetch(c, i, n) if alignment is not None else c.get(n)).to(dev) for i, c in enumerate(cks)]
        if not cfg.allow_mixed_dtype and len({t.dtype for t in ts}) > 1:
            raise ValueError(f"mixed dtypes for {n}; set allow_mixed_dtype")
        if any(t.shape != ts[0].shape for t in ts):
            raise ValueError(f"shape mismatch for {n}")
        b = base.get(n).to(dev) if (base is not None and n in base.index) else None
        if not ts[0].is_floating_point():
            out[n] = ts[0].cpu()
            continue
        a = None
        if aux:
            key = "fishers" if cfg.merge_method == "fisher" else "grams"
            a = {key: [x[n].to(dev) for x in aux]} if all(n in x for x in aux) else None
        if cfg.merge_method in ("fisher", "regmean") and a is None:
            merged = merge_tensor("linear", ts, b, params, cfg.parameters)      # fallback_to_mean
        else:
            merged = merge_tensor(cfg.merge_method, ts, b, params, cfg.parameters, a)
        from .sanity import check_tensor
        if cfg.sanity == "off":
            if not torch.isfinite(merged).all():
                raise ValueError(f"merge produced non-finite values in {n}")
        else:
            rep = check_tensor(n, merged, cfg.sanity)
            if rep.is_outlier():
                plan.setdefault("outliers", []).append({"name": n, "mean": rep.mean, "std": rep.std, "abs_max": rep.abs_max})
            if cfg.sanity == "full":
                plan.setdefault("tensor_reports", []).append(rep.to_dict())
        out[n] = merged.to(odt).cpu()
    _write(cfg, out, cfg.tokenizer_source or cfg.base_model or cfg.models[0].model)
    for c in cks:
        c.close()
    if base:
        base.close()
    plan["output"] = cfg.output_path
    return plan


def _layer_of(name: str) -> Optional[int]:
    parts = name.split(".")
    if "layers" in parts:
        i = parts.index("layers")
        if i + 1 < len(parts) and parts[i + 1].isdigit():
            return int(parts[i + 1])
    return None


def _run_slices(cfg: MergeConfig) -> dict:
    """Passthrough layer stacking: output layers are the concatenation of the listed layer ranges."""
    out: Dict[str, torch.Tensor] = {}
    nxt, first = 0, None
    for sl in cfg.slices:
        src = sl.sources[0]
        ck = LazyCheckpoint(src["model"])
        first = first or src["model"]
        a, b = src["layer_range"]
        for n in ck.keys():
            li = _layer_of(n)
            if li is None:
                if nxt == 0 or "norm" in n or "lm_head" in n:
                    out[n] = ck.get(n)
                continue
            if a <= li < b:
                out[n.replace(f"layers.{li}.", f"layers.{nxt + li - a}.")] = ck.get(n)
        nxt += b - a
        ck.close()
    if not cfg.dry_run:
        _write(cfg, out, cfg.tokenizer_source or first, num_layers=nxt)
    return {"method": "passthrough_slices", "num_layers": nxt, "tensors": len(out), "output": cfg.output_path}


def _write(cfg: MergeConfig, tensors: Dict[str, torch.Tensor], copy_from: Optional[str], num_layers: Optional[int] = None):
    if not cfg.output_path:
        raise ValueError("output_path is required")
    os.makedirs(cfg.output_path, exist_ok=True)
    st.save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(cfg.output_path, "model.safetensors"),
                 metadata={"format": "pt"})
    total = sum(v.numel() * v.element_size() for v in tensors.values())
    with open(os.path.join(cfg.output_path, "model.safetensors.index.json"), "w", encoding="utf-8") as fh:
        json.dump({"metadata": {"total_size": total}, "weight_map": {k: "model.safetensors" for k in sorted(tensors)}},
                  fh, indent=2)
    if copy_from and os.path.isdir(copy_from):
        for f in os.listdir(copy_from):
            if f.endswith(".json") and "index" not in f or f.startswith("tokenizer") or f in ("merges.txt", "vocab.json"):
                src = os.path.join(copy_from, f)
                if f == "config.json" and num_layers is not None:
                    with open(src) as fh:
                        c = json.load(fh)
                    c["num_hidden_layers"] = num_layers
                    with open(os.path.join(cfg.output_path, f), "w") as fh:
                        json.dump(c, fh, indent=2)
                else:
                    shutil.copy2(src, os.path.join(cfg.output_path, f))


def merge_lora_into_base(base_dir: str, adapter_path: str, out_dir: str, dtype: str = "bfloat16",
                         alpha: Optional[float] = None, rank: Optional[int] = None, accurate: bool = True,
                         low_memory: bool = False) -> dict:
    """W <- W + (alpha/r or alpha/sqrt(r)) * B A, tensor by tensor (commands/fuse.rs:67-204). ``accurate`` accumulates in
    float64 (float32 otherwise); ``low_memory`` forms the product 1024 output rows at a time so the wide intermediate
    never exists for the whole matrix. ``alpha`` / ``rank`` override the adapter's own values.
    Adapter key ``layers.N.<scope>.<proj>.lora_a`` maps to ``model.layers.N.<scope>.<proj>.weight``."""
    import dataclasses

    from ..lora.adapter import load_adapter_config, resolve_adapter_file
    lcfg = load_adapter_config(adapter_path if os.path.isdir(adapter_path) else os.path.dirname(adapter_path))
    if alpha is not None or rank is not None:
        lcfg = dataclasses.replace(lcfg, alpha=lcfg.alpha if alpha is None else float(alpha),
                                   r=lcfg.r if rank is None else int(rank))
    ad = st.load_file(resolve_adapter_file(adapter_path))
    scale = lcfg.scaling()
    acc = torch.float64 if accurate else torch.float32
    ck = LazyCheckpoint(base_dir)
    out: Dict[str, torch.Tensor] = {}
    fused = 0
    for n in ck.keys():
        w = ck.get(n)
        if n.startswith("model.") and n.endswith(".weight"):
            key = n[len("model."):-len(".weight")]
            a, b = ad.get(key + ".lora_a"), ad.get(key + ".lora_b")
            if a is not None and b is not None and a.shape[0] == lcfg.r and a.shape[0] > 0 and b.shape[1] == a.shape[0] \
                    and not (a.shape[0] == 1 and lcfg.r != 1):
                if low_memory:
                    new = torch.empty_like(w)
                    for r0 in range(0, w.shape[0], 1024):
                        r1 = min(r0 + 1024, w.shape[0])
                        new[r0:r1] = (w[r0:r1].to(acc) + scale * (b[r0:r1].to(acc) @ a.to(acc))).to(w.dtype)
                    w = new
                else:
                    w = (w.to(acc) + scale * (b.to(acc) @ a.to(acc))).to(w.dtype)
                fused += 1
        out[n] = w.to(_dtype(dtype)) if w.is_floating_point() else w
    cfg = MergeConfig(output_path=out_dir, dtype=dtype)
    _write(cfg, out, base_dir)
    ck.close()
    return {"fused_projections": fused, "output": out_dir, "scale": scale}
