"""HF checkpoint directory -> GGUF file (the ``quantize`` command), and tensor-name / config mapping both ways.

Reference behaviour (crates/pmetal/src/commands/quantize.rs:105-283,1236-1263,1340-1428 and
crates/pmetal-models/src/weight_format.rs:332-435): architecture string from ``config.json``, ``{arch}.*`` keys from
the HF config, ``general.name = "quantized-model"``, tokenizer metadata when ``tokenizer.json`` is present, tensors
renamed ``model.layers.N.self_attn.q_proj.weight`` -> ``blk.N.attn_q.weight``, stacked MoE expert tensors first, all
others sorted by HF name, per-tensor type from the recipe."""
from __future__ import annotations

import json
import os
import re
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import numpy as np

from . import native
from .imatrix import IMatrix
from .recipe import DynamicConfig, DynamicQuantizer, fit_to_shape, tensor_type
from .types import QUANT_METHODS, GgmlType, ValueType
from .writer import GgufWriter

ARCH_MAP = {
    "LlamaForCausalLM": "llama", "LlamaModel": "llama", "MistralForCausalLM": "mistral", "MixtralForCausalLM": "mistral",
    "Qwen2ForCausalLM": "qwen2", "Qwen2Model": "qwen2", "Qwen2MoeForCausalLM": "qwen2moe", "Qwen3ForCausalLM": "qwen3",
    "Qwen3Model": "qwen3", "Qwen3MoeForCausalLM": "qwen3moe", "Qwen3NextForCausalLM": "qwen3next",
    "Qwen3_5ForCausalLM": "qwen35", "Qwen3_5ForConditionalGeneration": "qwen35", "Qwen3_5MoeForCausalLM": "qwen35moe",
    "Qwen3_5MoeForConditionalGeneration": "qwen35moe", "GemmaForCausalLM": "gemma", "Gemma2ForCausalLM": "gemma",
    "PhiForCausalLM": "phi", "Phi3ForCausalLM": "phi", "DeepseekV2ForCausalLM": "deepseek2",
    "DeepseekV3ForCausalLM": "deepseek2", "GptOssForCausalLM": "gpt-oss",
}

_LAYER_SUFFIX = {
    "input_layernorm.weight": "attn_norm.weight", "self_attn.q_proj.weight": "attn_q.weight",
    "self_attn.k_proj.weight": "attn_k.weight", "self_attn.v_proj.weight": "attn_v.weight",
    "self_attn.o_proj.weight": "attn_output.weight", "post_attention_layernorm.weight": "ffn_norm.weight",
    "mlp.gate.weight": "ffn_gate_inp.weight", "mlp.router.weight": "ffn_gate_inp.weight",
    "mlp.gate_proj.weight": "ffn_gate.weight", "mlp.up_proj.weight": "ffn_up.weight",
    "mlp.down_proj.weight": "ffn_down.weight", "mlp.experts.gate_proj.weight": "ffn_gate_exps.weight",
    "mlp.experts.up_proj.weight": "ffn_up_exps.weight", "mlp.experts.down_proj.weight": "ffn_down_exps.weight",
    "mlp.shared_expert.gate_proj.weight": "ffn_gate_shexp.weight", "mlp.shared_expert.up_proj.weight": "ffn_up_shexp.weight",
    "mlp.shared_expert.down_proj.weight": "ffn_down_shexp.weight",
    "mlp.shared_experts.gate_proj.weight": "ffn_gate_shexp.weight", "mlp.shared_experts.up_proj.weight": "ffn_up_shexp.weight",
    "mlp.shared_experts.down_proj.weight": "ffn_down_shexp.weight", "mlp.shared_expert_gate.weight": "ffn_gate_inp_shexp.weight",
    "self_attn.q_norm.weight": "attn_q_norm.weight", "self_attn.k_norm.weight": "attn_k_norm.weight",
    "self_attn.q_proj.bias": "attn_q.bias", "self_attn.k_proj.bias": "attn_k.bias", "self_attn.v_proj.bias": "attn_v.bias",
}
_TOP = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
        "lm_head.weight": "output.weight"}
_TOP_INV = {v: k for k, v in _TOP.items()}
_LAYER_INV = {}
for _k, _v in _LAYER_SUFFIX.items():
    _LAYER_INV.setdefault(_v, _k)
_EXPERT_RE = re.compile(r"^model\.layers\.(\d+)\.mlp\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight$")


def hf_to_gguf_name(name: str) -> str:
    if name in _TOP:
        return _TOP[name]
    if not name.startswith("model.layers."):
        return name
    rest = name[len("model.layers."):]
    idx, _, suffix = rest.partition(".")
    if not idx.isdigit() or not suffix:
        return name
    return f"blk.{idx}.{_LAYER_SUFFIX.get(suffix, suffix)}"


def gguf_to_hf_name(name: str) -> str:
    if name in _TOP_INV:
        return _TOP_INV[name]
    if not name.startswith("blk."):
        return name
    idx, _, suffix = name[4:].partition(".")
    if not idx.isdigit() or not suffix:
        return name
    return f"model.layers.{idx}.{_LAYER_INV.get(suffix, suffix)}"


def architecture_of(config: Optional[dict]) -> str:
    for a in (config or {}).get("architectures", []) or []:
        if a in ARCH_MAP:
            return ARCH_MAP[a]
    return "llama"


def add_config_metadata(w: GgufWriter, arch: str, config: Optional[dict], method: str) -> None:
    w.add_string("general.type", "model")
    w.add_u32("general.file_type", QUANT_METHODS[method][1])
    if not config:
        return

    def first(keys):
        for k in keys:
            v = config.get(k)
            if isinstance(v, int) and not isinstance(v, bool) and v >= 0:
                return v
        return None
    for keys, suffix in (
            (("hidden_size", "n_embd", "dim"), "embedding_length"),
            (("num_hidden_layers", "n_layer", "n_layers"), "block_count"),
            (("num_attention_heads", "n_head", "n_heads"), "attention.head_count"),
            (("num_key_value_heads", "n_kv_heads"), "attention.head_count_kv"),
            (("intermediate_size", "n_inner", "hidden_dim"), "feed_forward_length"),
            (("max_position_embeddings", "n_ctx", "n_positions", "max_length", "max_sequence_length", "model_max_length"),
             "context_length"),
            (("vocab_size",), "vocab_size"), (("num_local_experts", "num_experts"), "expert_count"),
            (("num_experts_per_tok", "num_experts_per_token", "top_k_experts"), "expert_used_count"),
            (("n_group",), "expert_group_count"), (("topk_group",), "expert_group_used_count")):
        v = first(keys)
        if v is not None:
            w.add_u32(f"{arch}.{suffix}", v)
    if config.get("is_causal") is False:
        w.add_bool(f"{arch}.attention.causal", False)
    if isinstance(config.get("sliding_window"), int):
        w.add_u32(f"{arch}.attention.sliding_window", config["sliding_window"])
    head_dim = config.get("head_dim")
    if not isinstance(head_dim, int):
        h, n = config.get("hidden_size"), config.get("num_attention_heads")
        head_dim = h // n if isinstance(h, int) and isinstance(n, int) and n else None
    if head_dim is not None:
        for s in ("attention.head_dim", "attention.key_length", "attention.value_length", "rope.dimension_count"):
            w.add_u32(f"{arch}.{s}", head_dim)
    if isinstance(config.get("rope_theta"), (int, float)):
        w.add_f32(f"{arch}.rope.freq_base", config["rope_theta"])
    if isinstance(config.get("rms_norm_eps"), (int, float)):
        w.add_f32(f"{arch}.attention.layer_norm_rms_epsilon", config["rms_norm_eps"])
    for k in ("layer_norm_eps", "layer_norm_epsilon", "norm_epsilon"):
        if isinstance(config.get(k), (int, float)):
            w.add_f32(f"{arch}.attention.layer_norm_epsilon", config[k])
            break
    rs = config.get("rope_scaling")
    if isinstance(rs, dict):
        rt = str(rs.get("rope_type", rs.get("type", ""))).lower()
        mapped = {"linear": "linear", "yarn": "yarn", "su": "longrope", "longrope": "longrope", "none": "none"}.get(rt)
        if mapped:
            w.add_string(f"{arch}.rope.scaling.type", mapped)
        if isinstance(rs.get("factor"), (int, float)):
            w.add_f32(f"{arch}.rope.scaling.factor", rs["factor"])
        for k in ("original_max_position_embeddings", "original_context_length"):
            if isinstance(rs.get(k), int):
                w.add_u32(f"{arch}.rope.scaling.original_context_length", rs[k])
                break


def add_tokenizer_metadata(w: GgufWriter, model_dir: str) -> None:
    path = os.path.join(model_dir, "tokenizer.json")
    if not os.path.exists(path):
        return
    with open(path, "r", encoding="utf-8") as fh:
        tk = json.load(fh)
    model = tk.get("model", {})
    vocab = model.get("vocab")
    if not isinstance(vocab, dict):
        return
    size = max(vocab.values()) + 1
    added = {t["id"]: t for t in tk.get("added_tokens", []) if isinstance(t.get("id"), int)}
    size = max(size, max(added, default=-1) + 1)
    tokens = [f"[PAD{i}]" for i in range(size)]
    types = [1] * size                      # 1 normal, 3 control, 4 user-defined
    for t, i in vocab.items():
        tokens[i] = t
    for i, t in added.items():
        tokens[i] = t["content"]
        types[i] = 3 if t.get("special") else 4
    w.add_string("tokenizer.ggml.model", "gpt2" if model.get("type", "BPE") == "BPE" else "llama")
    w.add_array("tokenizer.ggml.tokens", ValueType.STRING, tokens)
    w.add_array("tokenizer.ggml.token_type", ValueType.INT32, types)
    merges = model.get("merges")
    if isinstance(merges, list) and merges:
        w.add_array("tokenizer.ggml.merges", ValueType.STRING,
                    [m if isinstance(m, str) else " ".join(m) for m in merges])
    cfg_path = os.path.join(model_dir, "tokenizer_config.json")
    if os.path.exists(cfg_path):
        with open(cfg_path, "r", encoding="utf-8") as fh:
            tc = json.load(fh)
        inv = {t: i for i, t in enumerate(tokens)}
        for key, gk in (("bos_token", "bos_token_id"), ("eos_token", "eos_token_id"), ("pad_token", "padding_token_id"),
                        ("unk_token", "unknown_token_id")):
            v = tc.get(key)
            v = v.get("content") if isinstance(v, dict) else v
            if isinstance(v, str) and v in inv:
                w.add_u32(f"tokenizer.ggml.{gk}", inv[v])
        if isinstance(tc.get("chat_template"), str):
            w.add_string("tokenizer.chat_template", tc["chat_template"])


def plan_tensors(names_shapes: Iterable[Tuple[str, Tuple[int, ...]]], method: str, config: Optional[dict],
                 dyn: Optional[DynamicQuantizer] = None) -> Dict[str, GgmlType]:
    """GGUF tensor name -> type for every tensor (1-D tensors stay F32)."""
    plan = {}
    for name, shape in names_shapes:
        if len(shape) < 2:
            plan[name] = GgmlType.F32
            continue
        proposed = dyn.propose(name) if dyn is not None else None
        plan[name] = fit_to_shape(tensor_type(method, name, shape, config, proposed), shape)
    return plan


def quantize_model(model_dir: str, output: str, method: str = "q4_k_m", imatrix_path: Optional[str] = None,
                   dynamic: Optional[DynamicConfig] = None, threads: int = 0,
                   progress: Optional[Callable[[str, GgmlType], None]] = None) -> dict:
    """Reads ``model_dir`` (safetensors, single file or sharded) and writes a GGUF file. Returns a summary."""
    from ..models.loader import read_state_dict
    method = method.lower()
    if method not in QUANT_METHODS:
        raise ValueError(f"unknown quantisation method {method!r}; choose from {sorted(QUANT_METHODS)}")
    config = None
    cp = os.path.join(model_dir, "config.json")
    if os.path.exists(cp):
        with open(cp, "r", encoding="utf-8") as fh:
            config = json.load(fh)
    arch = architecture_of(config)
    state = read_state_dict(model_dir)
    w = GgufWriter()
    w.add_string("general.architecture", arch)
    w.add_string("general.name", "quantized-model")
    add_config_metadata(w, arch, config, method)
    add_tokenizer_metadata(w, model_dir)
    dyn = None
    if method == "dynamic":
        dyn = DynamicQuantizer(dynamic or DynamicConfig(), IMatrix.load(imatrix_path) if imatrix_path else None)

    # stacked experts first: model.layers.N.mlp.experts.E.{gate,up,down}_proj.weight -> blk.N.ffn_*_exps.weight [E, out, in]
    groups: Dict[Tuple[int, str], List[Tuple[int, str]]] = {}
    plain: List[str] = []
    for name in state:
        m = _EXPERT_RE.match(name)
        if m:
            groups.setdefault((int(m.group(1)), m.group(3)), []).append((int(m.group(2)), name))
        else:
            plain.append(name)
    total_in = total_out = 0
    counts: Dict[str, int] = {}

    def emit(gname: str, arr: np.ndarray):
        nonlocal total_in, total_out
        shape = arr.shape
        if arr.ndim < 2:
            t = GgmlType.F32
        else:
            proposed = None
            if dyn is not None:
                proposed = dyn.calibrate(gname, arr) if dyn.config.kl_calibrate else dyn.propose(gname)
            t = fit_to_shape(tensor_type(method, gname, shape, config, proposed), shape)
        if not native.can_quantize(t):
            raise NotImplementedError(f"{gname}: host quantiser for {t.name} is not available")
        data = native.quantize(arr, t, threads)
        w.add_tensor_bytes(gname, shape, t, data.tobytes())
        total_in += arr.size * 4
        total_out += data.size
        counts[t.name] = counts.get(t.name, 0) + 1
        if progress:
            progress(gname, t)

    for (layer, proj), members in sorted(groups.items()):
        members.sort()
        stacked = np.stack([_as_f32(state[n]) for _, n in members])
        emit(f"blk.{layer}.ffn_{proj.split('_')[0]}_exps.weight", stacked)
    for name in sorted(plain):
        emit(hf_to_gguf_name(name), _as_f32(state[name]))
    nbytes = w.write_to(output)
    return {"output": output, "architecture": arch, "method": method, "tensors": len(w.tensors), "types": counts,
            "bytes": nbytes, "compression": round(total_in / max(total_out, 1), 3)}


def _as_f32(t) -> np.ndarray:
    try:
        import torch
        if isinstance(t, torch.Tensor):
            return t.detach().to(torch.float32).cpu().numpy()
    except ImportError:
        pass
    return np.asarray(t, dtype=np.float32)
