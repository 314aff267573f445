"""Model resolution and weight loading.

* ``resolve_model_path`` — a string is a hub id only if it does not start with ``/`` or ``.``,
  contains ``/`` and no such local path exists (crates/pmetal-hub/src/resolve.rs:12-33). The box is
  offline, so hub ids resolve through the local Hugging Face cache only.
* ``load_pretrained`` — ``config.json`` + ``model.safetensors`` or the shards named by
  ``model.safetensors.index.json`` (crates/pmetal-models/src/weight_format.rs:186-256), or a GGUF file
  dequantised on load (weight_format.rs:258-388). ``random:<preset>`` builds a random-init model.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional, Tuple

import torch

from ..utils import safetensors_io as st
from .config import PRESETS, ModelArgs, preset
from .decoder import DecoderLM


def is_hf_id(s: str) -> bool:
    return not s.startswith("/") and not s.startswith(".") and "/" in s


def resolve_model_path(model: str) -> str:
    if model.startswith("random:") or os.path.exists(model):
        return model
    if is_hf_id(model):
        cache = os.environ.get("HF_HOME", os.path.expanduser("~/.cache/huggingface"))
        d = os.path.join(cache, "hub", "models--" + model.replace("/", "--"), "snapshots")
        if os.path.isdir(d):
            snaps = sorted(os.listdir(d))
            if snaps:
                return os.path.join(d, snaps[-1])
        raise FileNotFoundError(f"model {model!r} is not in the local cache ({d}) and this machine has no network; "
                                "pass a local directory or random:<preset>")
    raise FileNotFoundError(model)


def read_state_dict(model_dir: str) -> Dict[str, torch.Tensor]:
    idx = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx, "r", encoding="utf-8") as fh:
            files = sorted(set(json.load(fh)["weight_map"].values()))
    else:
        files = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors") and "lora" not in f)
    if not files:
        raise FileNotFoundError(f"no safetensors weights in {model_dir}")
    sd: Dict[str, torch.Tensor] = {}
    for f in files:        # shards above 64 MiB go through the threaded positional reader
        path = os.path.join(model_dir, f)
        big = os.path.getsize(path) >= (64 << 20) and os.environ.get("PMETAL_PY_LOADER") != "1"
        sd.update(st.load_file_parallel(path) if big else st.load_file(path))
    return sd


def load_pretrained(model: str, dtype: torch.dtype = torch.bfloat16, device="cpu", seed: int = 0,
                    strict: bool = False, experts_dir: Optional[str] = None) -> Tuple[DecoderLM, ModelArgs, Optional[str]]:
    """Returns (model, args, model_dir or None). With ``experts_dir`` (written by ``pack-experts``) the routed experts are
    not read from the checkpoint: they are served from that directory on demand (models/expert_store.py)."""
    path = resolve_model_path(model)
    if path.startswith("random:"):
        name = path.split(":", 1)[1]
        args = preset(name)
        m = DecoderLM(args).init_weights(0.02, seed)
        return _cast(m, dtype, device), args, None
    if path.endswith(".gguf"):
        from ..gguf.loader import load_gguf_model
        m, args = load_gguf_model(path)
        return _cast(m, dtype, device), args, os.path.dirname(path)
    args = ModelArgs.from_pretrained(path)
    m = DecoderLM(args)
    sd = read_state_dict(path)
    sd = {k: v for k, v in sd.items() if not k.endswith("rotary_emb.inv_freq")}
    if any(k.endswith(".scales") for k in sd):          # affine group-quantised checkpoint (MLX layout): expand on load
        from ..quant.mlx_affine import load_quantized_state_dict
        with open(os.path.join(path, "config.json"), "r", encoding="utf-8") as fh:
            qcfg = json.load(fh).get("quantization") or {"bits": 4, "group_size": 64}
        sd = load_quantized_state_dict(sd, qcfg, torch.float32)
    if experts_dir:
        from .expert_store import enable_expert_offloading
        sd = {k: v for k, v in sd.items() if ".experts." not in k and ".switch_mlp." not in k}
        m.load_hf_state_dict(sd, strict=False)
        enable_expert_offloading(m, experts_dir)
        return _cast(m, dtype, device), args, path
    m.load_hf_state_dict(sd, strict=strict)
    return _cast(m, dtype, device), args, path


def _cast(m: DecoderLM, dtype, device) -> DecoderLM:
    m = m.to(device)
    for n, p in m.named_parameters():
        if "lora_" not in n:
            p.data = p.data.to(dtype)
    return m


def save_pretrained(m: DecoderLM, out_dir: str, merged: bool = True, max_shard_bytes: int = 5 << 30,
                    copy_from: Optional[str] = None) -> None:
    """Write ``model.safetensors`` (+ index) and ``config.json``; copy tokenizer files from ``copy_from``
    (layout of the reference's fuse command, crates/pmetal/src/commands/fuse.rs:150-204)."""
    import shutil
    os.makedirs(out_dir, exist_ok=True)
    sd = {k: v.detach().cpu().contiguous() for k, v in m.hf_state_dict(merged=merged).items()}
    total = sum(v.numel() * v.element_size() for v in sd.values())
    st.save_file(sd, os.path.join(out_dir, "model.safetensors"), metadata={"format": "pt"})
    with open(os.path.join(out_dir, "model.safetensors.index.json"), "w", encoding="utf-8") as fh:
        json.dump({"metadata": {"total_size": total}, "weight_map": {k: "model.safetensors" for k in sorted(sd)}},
                  fh, indent=2)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(m.cfg.to_hf_dict(), fh, indent=2)
    if copy_from and os.path.isdir(copy_from):
        for f in os.listdir(copy_from):
            if f.startswith("tokenizer") or f in ("special_tokens_map.json", "generation_config.json", "vocab.json",
                                                  "merges.txt", "chat_template.jinja", "added_tokens.json"):
                shutil.copy2(os.path.join(copy_from, f), os.path.join(out_dir, f))
