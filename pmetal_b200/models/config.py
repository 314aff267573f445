"""Architecture description read from a Hugging Face ``config.json``.

One dataclass covers the decoder-only families the reference dispatches on
(crates/pmetal-models/src/dispatcher.rs:42-118): llama, mistral, qwen2, qwen3,
qwen3_moe, gemma, phi, granite, cohere share the same pre-norm GQA block and differ
in the flags below. Defaults are Qwen3-0.6B (architectures/qwen3.rs:198-222).
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class ModelArgs:
    model_type: str = "qwen3"
    vocab_size: int = 151936
    hidden_size: int = 1024
    intermediate_size: int = 3072
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: Optional[int] = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    rope_scale: float = 1.0
    rope_scaling: Optional[dict] = None  # llama3 / yarn / dynamic / longrope schedule (linear folds into rope_scale)
    max_position_embeddings: int = 40960
    tie_word_embeddings: bool = True
    qk_norm: bool = True
    attention_bias: bool = False
    mlp_bias: bool = False
    sliding_window: int = 0
    max_window_layers: int = 0
    layer_types: Optional[List[str]] = None
    attn_logit_softcap: float = 0.0
    final_logit_softcap: float = 0.0
    hidden_act: str = "silu"
    # mixture of experts (qwen3_moe)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    decoder_sparse_step: int = 1
    mlp_only_layers: List[int] = field(default_factory=list)
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    pad_token_id: Optional[int] = None

    def __post_init__(self):
        if not self.head_dim:
            self.head_dim = self.hidden_size // self.num_attention_heads
        if not self.num_key_value_heads:
            self.num_key_value_heads = self.num_attention_heads

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def is_moe_layer(self, idx: int) -> bool:
        """qwen3_moe.rs:127-136: sparse unless listed in mlp_only_layers, every ``decoder_sparse_step`` layers."""
        return (self.num_experts > 0 and idx not in self.mlp_only_layers
                and (idx + 1) % max(self.decoder_sparse_step, 1) == 0)

    def uses_sliding_window(self, idx: int) -> bool:
        if self.sliding_window <= 0:
            return False
        if self.layer_types:
            return self.layer_types[idx] == "sliding_attention"
        return idx >= self.max_window_layers if self.max_window_layers else True

    @classmethod
    def from_dict(cls, d: dict) -> "ModelArgs":
        d = dict(d)
        mt = d.get("model_type", "qwen3")
        names = {f.name for f in dataclasses.fields(cls)}
        out = {k: v for k, v in d.items() if k in names and v is not None}
        out["model_type"] = mt
        if "qk_norm" not in d:
            out["qk_norm"] = mt in ("qwen3", "qwen3_moe", "gemma3", "olmo2")
        if "attention_bias" not in d:
            out["attention_bias"] = mt == "qwen2"
        if "tie_word_embeddings" not in d:
            out["tie_word_embeddings"] = mt in ("gemma", "gemma2")
        if "rope_theta" not in d:
            out["rope_theta"] = 10000.0
        rs = d.get("rope_scaling") or {}
        kind = rs.get("rope_type", rs.get("type"))
        if kind == "linear":
            out["rope_scale"] = float(rs.get("factor", 1.0))
            out["rope_scaling"] = None
        elif kind in (None, "default"):
            out["rope_scaling"] = None
        else:
            out["rope_scaling"] = dict(rs, rope_type=kind)
        if not d.get("use_sliding_window", True):
            out["sliding_window"] = 0
        if isinstance(out.get("eos_token_id"), list):
            out["eos_token_id"] = out["eos_token_id"][0]
        return cls(**out)

    @classmethod
    def from_pretrained(cls, model_dir: str) -> "ModelArgs":
        with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as fh:
            return cls.from_dict(json.load(fh))

    def to_hf_dict(self) -> dict:
        d = dataclasses.asdict(self)
        if d.get("rope_scaling") is None and self.rope_scale != 1.0:
            d["rope_scaling"] = {"rope_type": "linear", "factor": self.rope_scale}
        d["architectures"] = [{"qwen3": "Qwen3ForCausalLM", "qwen3_moe": "Qwen3MoeForCausalLM",
                               "qwen2": "Qwen2ForCausalLM", "llama": "LlamaForCausalLM",
                               "mistral": "MistralForCausalLM"}.get(self.model_type, "LlamaForCausalLM")]
        return d


PRESETS = {
    "qwen3-0.6b": dict(),
    "qwen3-4b": dict(hidden_size=2560, intermediate_size=9728, num_hidden_layers=36, num_attention_heads=32,
                     num_key_value_heads=8, head_dim=128),
    "qwen3-30b-a3b": dict(model_type="qwen3_moe", hidden_size=2048, intermediate_size=6144, num_hidden_layers=48,
                          num_attention_heads=32, num_key_value_heads=4, head_dim=128, num_experts=128,
                          num_experts_per_tok=8, moe_intermediate_size=768, tie_word_embeddings=False),
    "tiny-qwen3": dict(vocab_size=1024, hidden_size=256, intermediate_size=768, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=64),
    "tiny-qwen3-moe": dict(model_type="qwen3_moe", vocab_size=1024, hidden_size=256, intermediate_size=768,
                           num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                           num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128,
                           tie_word_embeddings=False),
    "tiny-llama": dict(model_type="llama", vocab_size=256, hidden_size=64, intermediate_size=128,
                       num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4, head_dim=16,
                       qk_norm=False, rope_theta=10000.0, tie_word_embeddings=False),
}


def preset(name: str, **over) -> ModelArgs:
    d = dict(PRESETS[name.lower()])
    d.update(over)
    return ModelArgs(**d)
