"""GGUF -> HF-named state dict and model config (the inference-side load path).

Every tensor is dequantised on the host to float32 and renamed ``blk.N.attn_q.weight`` ->
``model.layers.N.self_attn.q_proj.weight``; stacked expert tensors are split back into per-expert weights; tensors of
types without a dequantiser are skipped with a warning (crates/pmetal-models/src/weight_format.rs:258-312,332-388)."""
from __future__ import annotations

import logging
import re
from typing import Dict, Tuple

import numpy as np

from . import native
from .convert import gguf_to_hf_name
from .reader import GgufFile

log = logging.getLogger(__name__)
_EXPS = re.compile(r"^blk\.(\d+)\.ffn_(gate|up|down)_exps\.weight$")


def config_from_metadata(meta: Dict[str, object]) -> dict:
    """HF-style config dict from ``{arch}.*`` keys."""
    arch = str(meta.get("general.architecture", "llama"))

    def g(suffix, default=None):
        return meta.get(f"{arch}.{suffix}", default)
    cfg = {"model_type": {"qwen3moe": "qwen3_moe", "qwen2moe": "qwen2_moe"}.get(arch, arch),
           "hidden_size": g("embedding_length"), "num_hidden_layers": g("block_count"),
           "num_attention_heads": g("attention.head_count"),
           "num_key_value_heads": g("attention.head_count_kv", g("attention.head_count")),
           "intermediate_size": g("feed_forward_length"), "max_position_embeddings": g("context_length"),
           "vocab_size": g("vocab_size"), "head_dim": g("attention.key_length", g("attention.head_dim")),
           "rope_theta": g("rope.freq_base", 10000.0), "rms_norm_eps": g("attention.layer_norm_rms_epsilon", 1e-6)}
    kind = g("rope.scaling.type")
    if kind and kind != "none":
        rs = {"rope_type": kind, "factor": float(g("rope.scaling.factor", 1.0))}
        if g("rope.scaling.original_context_length"):
            rs["original_max_position_embeddings"] = int(g("rope.scaling.original_context_length"))
        cfg["rope_scaling"] = rs
    if g("expert_count"):
        cfg["num_experts"] = g("expert_count")
        cfg["num_experts_per_tok"] = g("expert_used_count")
    if cfg["vocab_size"] is None and isinstance(meta.get("tokenizer.ggml.tokens"), list):
        cfg["vocab_size"] = len(meta["tokenizer.ggml.tokens"])
    return {k: v for k, v in cfg.items() if v is not None}


def load_gguf_state_dict(path: str, threads: int = 0) -> Tuple[Dict[str, np.ndarray], dict]:
    """Returns (HF-named float32 arrays, config dict)."""
    out: Dict[str, np.ndarray] = {}
    with GgufFile(path) as f:
        cfg = config_from_metadata(f.metadata)
        for name in f.tensor_order:
            info = f.tensors[name]
            if not native.can_dequantize(info.dtype) and info.dtype.name not in ("I8", "I16", "I32", "I64", "F64"):
                log.warning("skipping %s: no dequantiser for %s", name, info.dtype.name)
                continue
            arr = f.tensor_f32(name, threads)
            m = _EXPS.match(name)
            if m and arr.ndim == 3:
                for e in range(arr.shape[0]):
                    out[f"model.layers.{m.group(1)}.mlp.experts.{e}.{m.group(2)}_proj.weight"] = arr[e]
            else:
                out[gguf_to_hf_name(name)] = arr
        if "lm_head.weight" not in out and "model.embed_tokens.weight" in out:
            cfg.setdefault("tie_word_embeddings", True)
    return out, cfg


def load_gguf_model(path: str, threads: int = 0):
    """Builds a ``DecoderLM`` from a GGUF file. Returns (model, ModelArgs)."""
    import torch

    from ..models.config import ModelArgs
    from ..models.decoder import DecoderLM
    sd, cfg = load_gguf_state_dict(path, threads)
    args = ModelArgs.from_dict(cfg)
    m = DecoderLM(args)
    m.load_hf_state_dict({k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in sd.items()}, strict=False)
    return m, args
