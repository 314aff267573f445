"""Architecture registry: model_type / architectures of a Hugging Face ``config.json`` -> implementation.

Mirrors the reference's dispatcher (crates/pmetal-models/src/dispatcher.rs:90-160: ``from_model_type`` then
``from_architectures``). The families with hand-written kernels (Qwen3, Qwen3-MoE, Llama, Qwen2, Mistral) resolve to
``models.decoder.DecoderLM``; every other decoder resolves to the portable ``GenericDecoderLM``; hybrids, encoders and
encoder-decoders have their own classes."""
from __future__ import annotations

import json
import os
from typing import Optional

FAST_DECODER = {"llama", "llama3", "qwen2", "qwen2_5", "qwen3", "qwen3_moe", "mistral"}
GENERIC_DECODER = {"mixtral", "gemma", "gemma2", "gemma3", "gemma3_text", "phi", "phi3", "phi4", "cohere", "cohere2",
                   "command_r", "command-r", "granite", "granitemoe", "granite_moe", "olmo2", "gpt_oss", "gptoss", "gpt-oss",
                   "llama4", "llama4_text", "deepseek", "deepseek2", "deepseek_v2", "deepseek_v3", "qwen3_next", "qwen3_5",
                   "qwen3.5", "qwen3_5_text", "qwen3_5_moe", "qwen3_5_moe_text"}
OTHER = {"nemotron_h": "nemotron_h", "nemotronh": "nemotron_h", "nemotron-h": "nemotron_h", "bert": "bert", "roberta": "bert",
         "distilbert": "bert", "xlm-roberta": "bert", "xlm_roberta": "bert", "t5": "t5", "clip": "clip", "whisper": "whisper",
         "flux": "flux", "flux-1": "flux", "flux.1": "flux", "pixtral": "pixtral", "qwen2_vl": "qwen2_vl", "mllama": "mllama",
         "gemma4": "gemma4", "gemma4_text": "gemma4"}


def family_of(config: dict) -> Optional[str]:
    """``fast`` | ``generic`` | one of the names in ``OTHER`` | None for an unknown architecture."""
    mt = str(config.get("model_type", "")).lower()
    if mt in ("gemma4", "gemma4_text"):
        return "gemma4"
    if "text_config" in config and mt not in OTHER:
        mt = str(config["text_config"].get("model_type", mt)).lower()
    if mt in FAST_DECODER:
        return "fast"
    if mt in GENERIC_DECODER:
        return "generic"
    if mt in OTHER:
        return OTHER[mt]
    for arch in config.get("architectures") or []:          # fall back to the class names
        a = arch.lower()
        for key, fam in (("llama4", "generic"), ("llama", "fast"), ("qwen3moe", "fast"), ("qwen3next", "generic"),
                         ("qwen3", "fast"), ("qwen2", "fast"), ("mistral", "fast"), ("mixtral", "generic"),
                         ("gemma4", "gemma4"), ("gemma", "generic"), ("phi", "generic"), ("cohere", "generic"), ("granite", "generic"),
                         ("deepseek", "generic"), ("gptoss", "generic"), ("nemotronh", "nemotron_h"), ("bert", "bert"),
                         ("t5", "t5"), ("clip", "clip"), ("whisper", "whisper")):
            if key in a:
                return fam
    return None


def build_model(config: dict, dtype=None, device=None):
    """Instantiate (uninitialised weights) the implementation for a Hugging Face config dict."""
    import torch
    fam = family_of(config)
    if fam is None:
        raise ValueError(f"unsupported architecture: model_type={config.get('model_type')!r}")
    if fam == "fast":
        from ..config import ModelArgs
        from ..decoder import DecoderLM
        return DecoderLM(ModelArgs.from_dict(config), dtype=dtype or torch.float32, device=device)
    if fam == "generic":
        from .generic import GenericDecoderLM
        m = GenericDecoderLM.from_hf_config(config)
    elif fam == "gemma4":
        from .gemma4 import Gemma4LM
        m = Gemma4LM.from_hf_config(config)
    elif fam == "nemotron_h":
        from .hybrid import NemotronHLM
        m = NemotronHLM(config)
    elif fam in ("bert", "t5", "clip", "whisper"):
        from . import encoders
        m = {"bert": encoders.BertModel, "t5": encoders.T5Model, "clip": encoders.ClipModel,
             "whisper": encoders.WhisperModel}[fam](config)
    elif fam in ("pixtral", "qwen2_vl", "mllama"):
        from . import vision
        m = vision.build_vision_language(config)
    elif fam == "flux":
        from .diffusion import FluxTransformer
        m = FluxTransformer(config)
    else:
        raise ValueError(fam)
    if dtype is not None or device is not None:
        m = m.to(device=device, dtype=dtype)
    return m


def load_pretrained(model_dir: str, dtype=None, device=None):
    """Build the model for ``model_dir/config.json`` and load its safetensors shards."""
    from ..loader import read_state_dict
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as fh:
        config = json.load(fh)
    model = build_model(config, dtype, device)
    sd = read_state_dict(model_dir)
    if family_of(config) == "generic":
        from .generic import convert_legacy_expert_keys
        sd = convert_legacy_expert_keys(sd, model.c)
    if hasattr(model, "load_hf_state_dict"):
        model.load_hf_state_dict(sd, strict=False)
    else:
        model.load_state_dict(sd, strict=False)
    return model


def save_pretrained(model, out_dir: str, copy_from: str) -> None:
    """Write the weights of a config-driven model next to the configuration and tokenizer files of ``copy_from`` (the
    directory it was loaded from): parameter names are the checkpoint's own, so the result loads with ``load_pretrained``
    here and with the Hugging Face classes. Tied read-outs are stored once."""
    import shutil

    from safetensors.torch import save_file
    os.makedirs(out_dir, exist_ok=True)
    sd, seen = {}, {}
    for k, v in model.state_dict().items():
        t = v.detach()
        key = (t.data_ptr(), tuple(t.shape))
        if key in seen:                                    # shared storage (tied embeddings): keep the first name
            continue
        seen[key] = k
        sd[k] = t.cpu().contiguous()
    save_file(sd, os.path.join(out_dir, "model.safetensors"), metadata={"format": "pt"})
    for f in os.listdir(copy_from):
        if f.endswith(".safetensors") or f.endswith(".safetensors.index.json") or f.endswith(".bin"):
            continue
        src = os.path.join(copy_from, f)
        if os.path.isfile(src):
            shutil.copy2(src, os.path.join(out_dir, f))
