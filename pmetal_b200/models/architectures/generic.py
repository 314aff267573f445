"""Config-driven decoder-only transformer covering the dense and mixture-of-experts families the reference dispatches on.

The reference keeps one Rust module per family (crates/pmetal-models/src/architectures/{llama,mistral,qwen2,gemma,phi,
cohere,granite,gpt_oss,llama4,deepseek}.rs, selected in crates/pmetal-models/src/dispatcher.rs:90-118). Here the families
are one module whose behaviour is described by ``ArchConfig``: normalisation flavour, block wiring (sequential, parallel,
sandwich, post-norm), rotary variant, per-layer attention pattern (full / sliding / chunked / no position encoding),
query-key normalisation, soft-capping, attention sinks, multipliers, and the feed-forward kind per layer (gated MLP,
plain MLP, or one of the routed-expert variants). Parameter names follow the Hugging Face checkpoints of every family, so
``load_state_dict`` takes such a checkpoint as it is.

The Qwen3 / Llama fast path with hand-written kernels is ``models.decoder.DecoderLM``; this module is the portable
implementation of everything else (plain PyTorch ops; runs on CPU and GPU) with a contiguous KV cache for generation."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..rope import rope_inv_freq  # noqa: F401  (re-exported for the architecture files)
from .fast import Linear, glu as _glu


# ------------------------------------------------------------------------------------------------ configuration
@dataclass
class ArchConfig:
    model_type: str = "llama"
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 32
    head_dim: int = 128
    # normalisation
    norm: str = "rms"                 # rms | rms_plus1 (weight stored as w-1) | layernorm | layernorm_bias
    norm_eps: float = 1e-5
    # block wiring
    block: str = "sequential"         # sequential | parallel (shared input norm) | sandwich (pre+post norms) | post
    act: str = "silu"
    gated_mlp: bool = True
    fused_qkv: bool = False           # phi3: qkv_proj / gate_up_proj stored fused
    attn_out_name: str = "o_proj"     # phi: "dense"
    attn_bias: bool = False
    o_bias: bool = False
    mlp_bias: bool = False
    final_norm_name: str = "norm"     # phi: "final_layernorm"
    lm_head_bias: bool = False
    tie_embeddings: bool = False
    # rotary
    rope_theta: float = 10000.0
    rope_local_theta: float = 0.0     # gemma3: base of sliding-window layers
    rope_dim: int = 0                 # rotated dims per head (0 = head_dim)
    rope_interleaved: bool = False    # pairs (2i, 2i+1) instead of (i, i + d/2)
    rope_scaling: Optional[dict] = None
    max_position: int = 8192
    # attention pattern
    layer_types: List[str] = field(default_factory=list)     # full | sliding | chunked per layer
    nope_layers: List[int] = field(default_factory=list)     # layers without rotary
    sliding_window: int = 0
    chunk_size: int = 0
    qk_norm: str = ""                 # "" | head (rms over head_dim, weight [d]) | per_head (layernorm, weight [h, d])
    #                                   | flat (rms over all heads, weight [h*d]) | l2 (no weight)
    qk_norm_rope_only: bool = False   # llama4: only on layers with rotary
    attn_scale: float = 0.0           # 0 = head_dim ** -0.5
    attn_softcap: float = 0.0
    final_softcap: float = 0.0
    sinks: bool = False
    temperature_tuning: Tuple[float, float] = (0.0, 0.0)    # llama4 (floor_scale, attn_scale) on NoPE layers
    # multipliers
    embed_scale: float = 1.0
    residual_multiplier: float = 1.0
    logits_divisor: float = 1.0
    logit_scale: float = 1.0
    # feed-forward kind per layer: dense | moe
    mlp_types: List[str] = field(default_factory=list)
    dense_intermediate: int = 0       # llama4 dense layers (0 = intermediate_size)
    num_experts: int = 0
    top_k: int = 0
    moe_intermediate: int = 0
    router: str = "softmax_topk"      # softmax_topk | topk_softmax | sigmoid_group | softmax_group | sigmoid_input
    norm_topk_prob: bool = True
    routed_scale: float = 1.0
    n_group: int = 1
    topk_group: int = 1
    group_score: str = "top2sum"      # top2sum (deepseek v3) | max (deepseek v2)
    router_bias: bool = False
    expert_bias: bool = False
    expert_layout: str = "out_in"     # out_in: gate_up [E, 2I, H] | in_out: gate_up [E, H, 2I]
    expert_act: str = "silu"          # silu | oss (clamped, interleaved gate/up)
    moe_name: str = "mlp"             # llama4: feed_forward; granitemoe: block_sparse_moe
    router_name: str = "gate"
    n_shared_experts: int = 0
    shared_name: str = "shared_experts"
    shared_gate: bool = False         # qwen: sigmoid gate on the shared expert
    shared_intermediate: int = 0      # size of the shared expert when it is not n_shared_experts * moe_intermediate
    # gated attention output and gated-delta-net layers (qwen3-next)
    attn_output_gate: bool = False
    lin_v_heads: int = 0
    lin_k_heads: int = 0
    lin_k_dim: int = 0
    lin_v_dim: int = 0
    lin_conv: int = 4
    # multi-head latent attention (deepseek)
    mla: bool = False
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_dim: int = 0
    qk_rope_dim: int = 0
    v_head_dim: int = 0
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None

    def layer_type(self, i: int) -> str:
        return self.layer_types[i] if self.layer_types else ("sliding" if self.sliding_window else "full")

    def mlp_type(self, i: int) -> str:
        return self.mlp_types[i] if self.mlp_types else ("moe" if self.num_experts else "dense")


def _rope_params(d: dict) -> Tuple[float, Optional[dict], float]:
    """(theta, scaling dict or None, local theta) from either the flat keys or the nested ``rope_parameters`` form."""
    rp = d.get("rope_parameters") or {}
    local = 0.0
    if "full_attention" in rp or "sliding_attention" in rp:          # per-layer-type form (gemma3)
        local = float((rp.get("sliding_attention") or {}).get("rope_theta", 0.0))
        rp = rp.get("full_attention") or {}
    theta = float(rp.get("rope_theta", d.get("rope_theta", 10000.0)))
    sc = d.get("rope_scaling") or ({k: v for k, v in rp.items() if k != "rope_theta"} if rp else None)
    if sc:
        kind = sc.get("rope_type", sc.get("type", "default"))
        sc = None if kind == "default" else dict(sc, rope_type=kind)
    if d.get("rope_local_base_freq"):
        local = float(d["rope_local_base_freq"])
    return theta, sc, local


def arch_config_from_hf(d: dict) -> ArchConfig:
    """Translate a Hugging Face ``config.json`` (multimodal wrappers: its ``text_config``) into an ``ArchConfig``."""
    if "text_config" in d and "hidden_size" not in d:
        d = dict(d["text_config"], model_type=d["text_config"].get("model_type", d.get("model_type")))
    mt = str(d.get("model_type", "llama")).lower()
    H = d["hidden_size"]
    nh = d["num_attention_heads"]
    nkv = d.get("num_key_value_heads") or nh
    L = d["num_hidden_layers"]
    theta, scaling, local = _rope_params(d)
    c = ArchConfig(model_type=mt, vocab_size=d["vocab_size"], hidden_size=H,
                   intermediate_size=d.get("intermediate_size", 4 * H), num_layers=L, n_heads=nh, n_kv_heads=nkv,
                   head_dim=d.get("head_dim") or H // nh, norm_eps=d.get("rms_norm_eps", d.get("layer_norm_eps", 1e-5)),
                   rope_theta=theta, rope_scaling=scaling, rope_local_theta=local,
                   max_position=d.get("max_position_embeddings", 8192), act=d.get("hidden_act", d.get("hidden_activation", "silu")),
                   attn_bias=bool(d.get("attention_bias", False)), mlp_bias=bool(d.get("mlp_bias", False)),
                   tie_embeddings=bool(d.get("tie_word_embeddings", False)), bos_token_id=d.get("bos_token_id"),
                   eos_token_id=d.get("eos_token_id") if not isinstance(d.get("eos_token_id"), list) else d["eos_token_id"][0])
    c.o_bias = c.attn_bias
    lt = d.get("layer_types")
    if lt:
        c.layer_types = [{"full_attention": "full", "sliding_attention": "sliding", "chunked_attention": "chunked",
                          "linear_attention": "linear"}.get(t, t) for t in lt]
    sw = d.get("sliding_window") or 0
    if mt in ("llama", "llama3"):
        pass
    elif mt in ("mistral", "mixtral"):
        c.sliding_window = sw
        if mt == "mixtral":
            c.num_experts, c.top_k = d["num_local_experts"], d["num_experts_per_tok"]
            c.moe_intermediate = c.intermediate_size
            c.router, c.norm_topk_prob = "softmax_topk", True
    elif mt in ("qwen2", "qwen2_5", "qwen3", "qwen3_moe"):
        c.attn_bias, c.o_bias = mt.startswith("qwen2"), False
        if "attention_bias" in d:
            c.attn_bias = bool(d["attention_bias"])
        c.qk_norm = "head" if mt.startswith("qwen3") else ""
        if d.get("use_sliding_window"):
            c.sliding_window = sw
            if not lt:
                c.layer_types = ["sliding" if i >= d.get("max_window_layers", L) else "full" for i in range(L)]
        if mt == "qwen3_moe":
            c.num_experts, c.top_k = d["num_experts"], d["num_experts_per_tok"]
            c.moe_intermediate = d["moe_intermediate_size"]
            c.norm_topk_prob = bool(d.get("norm_topk_prob", False))
            step, only = d.get("decoder_sparse_step", 1), set(d.get("mlp_only_layers") or [])
            c.mlp_types = ["moe" if (i not in only and (i + 1) % step == 0) else "dense" for i in range(L)]
    elif mt in ("qwen3_next", "qwen3_5", "qwen3.5", "qwen3_5_text", "qwen3_5_moe", "qwen3_5_moe_text"):
        c.norm, c.qk_norm, c.attn_output_gate = "rms_plus1", "head", True
        c.norm_eps = d.get("rms_norm_eps", 1e-6)
        prf = (d.get("rope_parameters") or {}).get("partial_rotary_factor", d.get("partial_rotary_factor", 0.25))
        c.rope_dim = int(c.head_dim * prf)
        if c.rope_scaling:
            c.rope_scaling = {k: v for k, v in c.rope_scaling.items() if k != "partial_rotary_factor"}
            if c.rope_scaling.get("rope_type", "default") == "default":
                c.rope_scaling = None
        if not lt:
            step = d.get("full_attention_interval", 4)
            c.layer_types = ["full" if (i + 1) % step == 0 else "linear" for i in range(L)]
        c.lin_v_heads, c.lin_k_heads = d.get("linear_num_value_heads", 32), d.get("linear_num_key_heads", 16)
        c.lin_k_dim, c.lin_v_dim = d.get("linear_key_head_dim", 128), d.get("linear_value_head_dim", 128)
        c.lin_conv = d.get("linear_conv_kernel_dim", 4)
        c.num_experts, c.top_k = d.get("num_experts", 0), d.get("num_experts_per_tok", 0)
        c.moe_intermediate = d.get("moe_intermediate_size", 0)
        c.norm_topk_prob = bool(d.get("norm_topk_prob", True))
        if c.num_experts:
            c.n_shared_experts, c.shared_name, c.shared_gate = 1, "shared_expert", True
            c.shared_intermediate = d.get("shared_expert_intermediate_size", c.moe_intermediate)
            step, only = d.get("decoder_sparse_step", 1), set(d.get("mlp_only_layers") or [])
            c.mlp_types = ["moe" if (i not in only and (i + 1) % step == 0) else "dense" for i in range(L)]
    elif mt in ("gemma", "gemma2", "gemma3", "gemma3_text"):
        c.norm, c.embed_scale, c.act = "rms_plus1", float(H) ** 0.5, "gelu_tanh"
        c.norm_eps = d.get("rms_norm_eps", 1e-6)
        c.tie_embeddings = bool(d.get("tie_word_embeddings", True))
        if mt != "gemma":
            c.block = "sandwich"
            c.attn_scale = float(d.get("query_pre_attn_scalar", c.head_dim)) ** -0.5
            c.sliding_window = sw
            c.attn_softcap = float(d.get("attn_logit_softcapping") or 0.0)
            c.final_softcap = float(d.get("final_logit_softcapping") or 0.0)
            if not lt:
                pat = d.get("sliding_window_pattern", 6) if mt != "gemma2" else 2
                c.layer_types = ["full" if (i + 1) % pat == 0 else "sliding" for i in range(L)]
        if mt.startswith("gemma3"):
            c.qk_norm = "head"
    elif mt in ("phi3", "phi4"):
        c.fused_qkv = True
        c.sliding_window = sw
        c.rope_dim = int(c.head_dim * d.get("partial_rotary_factor", 1.0))
    elif mt == "phi":
        c.norm, c.block, c.gated_mlp, c.act = "layernorm_bias", "parallel", False, d.get("hidden_act", "gelu_new")
        c.attn_bias = c.o_bias = c.mlp_bias = c.lm_head_bias = True
        c.attn_out_name, c.final_norm_name = "dense", "final_layernorm"
        c.rope_dim = int(c.head_dim * d.get("partial_rotary_factor", 0.5))
        c.norm_eps = d.get("layer_norm_eps", 1e-5)
    elif mt in ("cohere", "cohere2", "command_r", "command-r"):
        c.norm, c.block, c.rope_interleaved = "layernorm", "parallel", True
        c.norm_eps = d.get("layer_norm_eps", 1e-5)
        c.logit_scale = float(d.get("logit_scale", 0.0625))
        c.tie_embeddings = bool(d.get("tie_word_embeddings", True))
        c.qk_norm = "per_head" if d.get("use_qk_norm") else ""
        if mt == "cohere2":
            c.sliding_window = sw
            if not lt:
                pat = d.get("sliding_window_pattern", 4)
                c.layer_types = ["full" if (i + 1) % pat == 0 else "sliding" for i in range(L)]
            c.nope_layers = [i for i in range(L) if c.layer_types[i] == "full"]
    elif mt in ("granite", "granitemoe", "granite_moe"):
        c.embed_scale = float(d.get("embedding_multiplier", 1.0))
        c.residual_multiplier = float(d.get("residual_multiplier", 1.0))
        c.attn_scale = float(d.get("attention_multiplier", c.head_dim ** -0.5))
        c.logits_divisor = float(d.get("logits_scaling", 1.0))
        if mt != "granite":
            c.num_experts, c.top_k = d["num_local_experts"], d["num_experts_per_tok"]
            c.moe_intermediate = c.intermediate_size
            c.router, c.moe_name, c.router_name = "topk_softmax", "block_sparse_moe", "router.layer"
    elif mt == "olmo2":
        c.block, c.qk_norm = "post", "flat"
    elif mt in ("gpt_oss", "gptoss", "gpt-oss"):
        c.attn_bias = c.o_bias = True
        c.sinks, c.sliding_window = True, sw
        c.num_experts, c.top_k = d["num_local_experts"], d["num_experts_per_tok"]
        c.moe_intermediate = c.intermediate_size
        c.router, c.router_name, c.router_bias, c.expert_bias = "topk_softmax", "router", True, True
        c.expert_layout, c.expert_act = "in_out", "oss"
        if not lt:
            c.layer_types = ["sliding" if i % 2 == 0 else "full" for i in range(L)]
    elif mt in ("llama4", "llama4_text"):
        c.rope_interleaved = True
        c.qk_norm, c.qk_norm_rope_only = ("l2" if d.get("use_qk_norm", True) else ""), True
        nope = d.get("no_rope_layers")
        if nope:                          # list of 1 (rotary) / 0 (none) per layer
            c.nope_layers = [i for i, v in enumerate(nope) if not v]
        else:
            c.nope_layers = [i for i in range(L) if (i + 1) % d.get("nope_layer_interval", 4) == 0]
        c.chunk_size = d.get("attention_chunk_size") or 0
        if not lt:
            c.layer_types = ["full" if i in c.nope_layers or not c.chunk_size else "chunked" for i in range(L)]
        if d.get("attn_temperature_tuning", True):
            c.temperature_tuning = (float(d.get("floor_scale", 8192)), float(d.get("attn_scale", 0.1)))
        c.num_experts, c.top_k = d["num_local_experts"], d.get("num_experts_per_tok", 1)
        c.moe_intermediate, c.dense_intermediate = c.intermediate_size, d.get("intermediate_size_mlp", c.intermediate_size)
        c.router, c.router_name, c.moe_name = "sigmoid_input", "router", "feed_forward"
        c.expert_layout, c.n_shared_experts, c.shared_name = "in_out", 1, "shared_expert"
        moe_layers = d.get("moe_layers")
        if moe_layers is None:
            step = d.get("interleave_moe_layer_step", 1)
            moe_layers = list(range(step - 1, L, step))
        c.mlp_types = ["moe" if i in set(moe_layers) else "dense" for i in range(L)]
    elif mt in ("deepseek", "deepseek2", "deepseek_v2", "deepseek_v3"):
        c.mla, c.rope_interleaved = True, True
        c.q_lora_rank, c.kv_lora_rank = d.get("q_lora_rank") or 0, d["kv_lora_rank"]
        c.qk_nope_dim, c.qk_rope_dim, c.v_head_dim = d["qk_nope_head_dim"], d["qk_rope_head_dim"], d["v_head_dim"]
        c.head_dim = c.qk_nope_dim + c.qk_rope_dim
        c.rope_dim = c.qk_rope_dim
        c.num_experts, c.top_k = d.get("n_routed_experts") or 0, d.get("num_experts_per_tok") or 0
        c.moe_intermediate = d.get("moe_intermediate_size", 0)
        c.n_shared_experts = d.get("n_shared_experts") or 0
        c.routed_scale = float(d.get("routed_scaling_factor", 1.0))
        c.norm_topk_prob = bool(d.get("norm_topk_prob", mt == "deepseek_v3"))
        c.n_group, c.topk_group = d.get("n_group") or 1, d.get("topk_group") or 1
        v3 = mt == "deepseek_v3"
        c.router = "sigmoid_group" if v3 else "softmax_group"
        c.group_score = "top2sum" if v3 else "max"
        if not v3 and d.get("topk_method", "greedy") == "greedy":
            c.n_group = c.topk_group = 1
        first = d.get("first_k_dense_replace", 0)
        step = d.get("moe_layer_freq", 1)
        c.mlp_types = ["moe" if (c.num_experts and i >= first and i % step == 0) else "dense" for i in range(L)]
    else:
        raise ValueError(f"unsupported model_type {mt!r}")
    return c


# ------------------------------------------------------------------------------------------------ building blocks
class Norm(nn.Module):
    def __init__(self, dim, kind: str, eps: float):
        super().__init__()
        self.kind, self.eps = kind, eps
        self.weight = nn.Parameter(torch.zeros(dim) if kind == "rms_plus1" else torch.ones(dim))
        if kind == "layernorm_bias":
            self.bias = nn.Parameter(torch.zeros(dim))

    def forward(self, x):
        if self.kind == "rms":
            from .fast import rms_norm
            y = rms_norm(x, self.weight, self.eps)
            if y is not None:
                return y
        xf = x.float()
        if self.kind.startswith("rms"):
            y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
            if self.kind == "rms_plus1":
                return (y * (1.0 + self.weight.float())).to(x.dtype)
            return self.weight * y.to(x.dtype)
        mu = xf.mean(-1, keepdim=True)
        var = (xf - mu).pow(2).mean(-1, keepdim=True)
        y = (xf - mu) * torch.rsqrt(var + self.eps) * self.weight.float()
        if self.kind == "layernorm_bias":
            y = y + self.bias.float()
        return y.to(x.dtype)


def _act(name: str):
    return {"silu": F.silu, "swish": F.silu, "gelu": F.gelu, "relu": F.relu,
            "gelu_tanh": lambda x: F.gelu(x, approximate="tanh"), "gelu_pytorch_tanh": lambda x: F.gelu(x, approximate="tanh"),
            "gelu_new": lambda x: F.gelu(x, approximate="tanh"), "relu2": lambda x: F.relu(x).square()}[name]


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleaved: bool) -> torch.Tensor:
    """x [B, h, T, d]; cos/sin [B, T, r/2] rotate the first r dims of every head."""
    r = cos.shape[-1] * 2
    xr, rest = x[..., :r].float(), x[..., r:]
    c, s = cos[:, None].float(), sin[:, None].float()
    if interleaved:
        a, b = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack((a * c - b * s, a * s + b * c), -1).flatten(-2)
    else:
        a, b = xr[..., : r // 2], xr[..., r // 2:]
        out = torch.cat((a * c - b * s, b * c + a * s), -1)
    return torch.cat((out.to(x.dtype), rest), -1)


def build_mask(kind: str, q_pos: torch.Tensor, k_pos: torch.Tensor, window: int, chunk: int) -> torch.Tensor:
    """Boolean [B, 1, Tq, Tk] mask (True = attend) from absolute positions."""
    qp, kp = q_pos[:, :, None], k_pos[:, None, :]
    m = kp <= qp
    if kind == "sliding" and window > 0:
        m = m & (kp > qp - window)
    elif kind == "chunked" and chunk > 0:
        m = m & (torch.div(kp, chunk, rounding_mode="floor") == torch.div(qp, chunk, rounding_mode="floor"))
    return m[:, None]


def with_documents(mask: torch.Tensor, doc_ids: Optional[torch.Tensor]) -> torch.Tensor:
    """Restrict a [B, 1, T, T] mask to pairs of the same document (packed rows); ``doc_ids`` [B, T] or None."""
    if doc_ids is None:
        return mask
    return mask & (doc_ids[:, None, :, None] == doc_ids[:, None, None, :])


def attend(q, k, v, mask, scale: float, softcap: float = 0.0, sinks: Optional[torch.Tensor] = None):
    """q [B, h, Tq, d], k/v [B, hkv, Tk, d*]. Softmax in fp32; optional tanh soft-cap and per-head sink logits."""
    B, h, Tq, _ = q.shape
    g = h // k.shape[1]
    if g > 1:
        k = k.repeat_interleave(g, 1)
        v = v.repeat_interleave(g, 1)
    if softcap <= 0 and sinks is None:
        return F.scaled_dot_product_attention(q, k, v, attn_mask=mask, scale=scale)
    s = torch.matmul(q, k.transpose(-1, -2)).float() * scale
    if softcap > 0:
        s = torch.tanh(s / softcap) * softcap
    s = s.masked_fill(~mask, float("-inf"))
    if sinks is not None:
        s = torch.cat((s, sinks.float().view(1, h, 1, 1).expand(B, h, Tq, 1)), -1)
        p = torch.softmax(s, -1)[..., :-1]
    else:
        p = torch.softmax(s, -1)
    return torch.matmul(p.to(v.dtype), v)


class KVCache:
    """Contiguous per-layer key/value store for generation with the portable models."""

    def __init__(self, num_layers: int):
        self.k: List[Optional[torch.Tensor]] = [None] * num_layers
        self.v: List[Optional[torch.Tensor]] = [None] * num_layers
        self.state: Dict[int, object] = {}          # recurrent layers keep their state here

    def append(self, layer: int, k: torch.Tensor, v: torch.Tensor):
        if self.k[layer] is not None:
            k = torch.cat((self.k[layer], k), 2)
            v = torch.cat((self.v[layer], v), 2)
        self.k[layer], self.v[layer] = k, v
        return k, v

    def length(self) -> int:
        for k in self.k:
            if k is not None:
                return k.shape[2]
        return int(self.state.get("length", 0))


class QuantKVCache(KVCache):
    """KV cache that stores keys and values quantised and expands them on read: ``bits`` 8 or 4 with one fp16 scale per
    ``group`` channels (symmetric, absmax), or ``turbo=True`` for the rotation + Lloyd-Max codebook scheme (2, 4 or 8 bits) of
    ``models/turboquant.py`` (optionally with the QJL residual sign sketch). The reference selects between fp16, q8 and
    TurboQuant caches to fit unified memory (crates/pmetal-mlx/src/kv_cache/quantized.rs, crates/pmetal-serve/src/engine.rs
    KV-mode selection); here the portable models can trade accuracy for cache size the same way."""

    def __init__(self, num_layers: int, bits: int = 8, group: int = 64, turbo: bool = False, qjl: bool = False):
        super().__init__(num_layers)
        if bits not in (2, 4, 8):
            raise ValueError("bits must be 2, 4 or 8")
        if not turbo and bits not in (4, 8):
            raise ValueError("group quantisation supports 4 or 8 bits")
        self.bits, self.group, self.turbo, self.qjl = bits, group, turbo, qjl
        self._store: List[List] = [[] for _ in range(num_layers)]        # per layer: list of (k blob, v blob, shape, dtype)
        self._tq: Dict[int, object] = {}
        self._len = [0] * num_layers

    # ---- codecs
    def _enc(self, x: torch.Tensor):
        d = x.shape[-1]
        if self.turbo:
            from ..turboquant import TurboQuant
            tq = self._tq.get(d)
            if tq is None:
                tq = self._tq[d] = TurboQuant(d, self.bits, self.qjl, device=x.device)
            return tq.encode(x.reshape(-1, d).float())
        g = self.group if d % self.group == 0 else d
        xf = x.float().reshape(*x.shape[:-1], d // g, g)
        qmax = 127.0 if self.bits == 8 else 7.0
        scale = xf.abs().amax(-1, keepdim=True).clamp(min=1e-8) / qmax
        q = torch.round(xf / scale).clamp(-qmax, qmax).to(torch.int8)
        if self.bits == 4:                                              # two codes per byte
            u = (q + 8).to(torch.uint8).reshape(*q.shape[:-1], g // 2, 2)
            q = u[..., 0] | (u[..., 1] << 4)
        return q, scale.to(torch.float16)

    def _dec(self, blob, shape, dtype):
        if self.turbo:
            return self._tq[shape[-1]].decode(blob).reshape(shape).to(dtype)
        q, scale = blob
        if self.bits == 4:
            q = torch.stack(((q & 15).to(torch.int8) - 8, (q >> 4).to(torch.int8) - 8), -1).flatten(-2)
        return (q.float() * scale.float()).reshape(shape).to(dtype)

    def append(self, layer: int, k: torch.Tensor, v: torch.Tensor):
        self._store[layer].append((self._enc(k), self._enc(v), k.shape, v.shape, k.dtype))
        self._len[layer] += k.shape[2]
        ks = [self._dec(kb, ksh, dt) for kb, _, ksh, _, dt in self._store[layer]]
        vs = [self._dec(vb, vsh, dt) for _, vb, _, vsh, dt in self._store[layer]]
        return torch.cat(ks, 2), torch.cat(vs, 2)

    def length(self) -> int:
        return max(self._len) if any(self._len) else int(self.state.get("length", 0))

    def nbytes(self) -> int:
        """Bytes held by the compressed keys and values."""
        def size(blob):
            if self.turbo:
                return blob.nbytes()
            return sum(t.numel() * t.element_size() for t in blob)
        return sum(size(kb) + size(vb) for layer in self._store for kb, vb, *_ in layer)


class Attention(nn.Module):
    def __init__(self, c: ArchConfig, idx: int):
        super().__init__()
        self.c, self.idx = c, idx
        H, d = c.hidden_size, c.head_dim
        self.kind = c.layer_type(idx)
        self.rotary = idx not in c.nope_layers
        if c.fused_qkv:
            self.qkv_proj = Linear(H, (c.n_heads + 2 * c.n_kv_heads) * d, bias=c.attn_bias)
        else:
            self.q_proj = Linear(H, c.n_heads * d * (2 if c.attn_output_gate else 1), bias=c.attn_bias)
            self.k_proj = Linear(H, c.n_kv_heads * d, bias=c.attn_bias)
            self.v_proj = Linear(H, c.n_kv_heads * d, bias=c.attn_bias)
        setattr(self, c.attn_out_name, Linear(c.n_heads * d, H, bias=c.o_bias))
        qn = c.qk_norm if (self.rotary or not c.qk_norm_rope_only) else ""
        self.qn_kind = qn
        if qn == "head":
            self.q_norm, self.k_norm = Norm(d, c.norm if c.norm.startswith("rms") else "rms", c.norm_eps), \
                Norm(d, c.norm if c.norm.startswith("rms") else "rms", c.norm_eps)
        elif qn == "per_head":
            self.q_norm, self.k_norm = Norm((c.n_heads, d), "layernorm", c.norm_eps), Norm((c.n_kv_heads, d), "layernorm", c.norm_eps)
        elif qn == "flat":
            self.q_norm, self.k_norm = Norm(c.n_heads * d, "rms", c.norm_eps), Norm(c.n_kv_heads * d, "rms", c.norm_eps)
        if c.sinks:
            self.sinks = nn.Parameter(torch.zeros(c.n_heads))

    def forward(self, x, rope, positions, cache: Optional[KVCache], k_positions):
        c = self.c
        B, T, _ = x.shape
        d = c.head_dim
        if c.fused_qkv:
            q, k, v = self.qkv_proj(x).split((c.n_heads * d, c.n_kv_heads * d, c.n_kv_heads * d), -1)
        else:
            q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
        gate = None
        if c.attn_output_gate:          # per head: [query (d) | gate (d)]
            q, gate = q.view(B, T, c.n_heads, 2 * d).chunk(2, -1)
            q, gate = q.reshape(B, T, c.n_heads * d), gate.reshape(B, T, c.n_heads * d)
        if self.qn_kind == "flat":
            q, k = self.q_norm(q), self.k_norm(k)
        q, k, v = q.view(B, T, c.n_heads, d), k.view(B, T, c.n_kv_heads, d), v.view(B, T, c.n_kv_heads, d)
        if self.qn_kind in ("head", "per_head"):
            q, k = self.q_norm(q), self.k_norm(k)
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        if self.rotary:
            cos, sin = rope["local" if (self.kind == "sliding" and "local" in rope) else "global"]
            q, k = apply_rope(q, cos, sin, c.rope_interleaved), apply_rope(k, cos, sin, c.rope_interleaved)
        if self.qn_kind == "l2":
            q = (q.float() * torch.rsqrt(q.float().pow(2).mean(-1, keepdim=True) + c.norm_eps)).to(q.dtype)
            k = (k.float() * torch.rsqrt(k.float().pow(2).mean(-1, keepdim=True) + c.norm_eps)).to(k.dtype)
        if not self.rotary and c.temperature_tuning[0] > 0:
            fs, sc = c.temperature_tuning
            t = torch.log1p(torch.floor((positions.float() + 1.0) / fs)) * sc + 1.0
            q = (q * t[:, None, :, None]).to(q.dtype)
        if cache is not None:
            k, v = cache.append(self.idx, k, v)
        scale = (c.attn_scale or d ** -0.5) * rope.get("attention_factor", 1.0) ** 2
        o = None
        docs = rope.get("doc_ids")
        if (cache is None and rope.get("mask") is None and c.attn_softcap <= 0 and not c.sinks
                and self.kind in ("full", "sliding") and q.is_cuda and (rope.get("contiguous", False) or docs is not None)):
            # whole sequences from position 0 (or packed documents whose positions restart) with a causal or
            # sliding-window mask: the varlen flash-attention kernels
            from .fast import causal_attention
            o = causal_attention(q, k, v, scale, c.sliding_window if self.kind == "sliding" else 0, docs)
        if o is None:
            mask = rope["mask"] if rope.get("mask") is not None else \
                with_documents(build_mask(self.kind, positions, k_positions, c.sliding_window, c.chunk_size), docs)
            o = attend(q, k, v, mask, scale, c.attn_softcap, self.sinks if c.sinks else None)
        o = o.transpose(1, 2).reshape(B, T, c.n_heads * d)
        if gate is not None:
            o = o * torch.sigmoid(gate)
        return getattr(self, c.attn_out_name)(o)


class GatedDeltaNet(nn.Module):
    """Linear-attention layer of the Qwen3-Next hybrids: short causal depthwise convolution over (q, k, v), gated delta
    rule recurrence per value head, gated RMSNorm of the read-out (crates/pmetal-models/src/architectures/qwen3_next.rs;
    the recurrence itself is models/gdn.py)."""

    def __init__(self, c: ArchConfig, idx: int):
        super().__init__()
        self.c, self.idx = c, idx
        self.key_dim, self.value_dim = c.lin_k_dim * c.lin_k_heads, c.lin_v_dim * c.lin_v_heads
        conv_dim = 2 * self.key_dim + self.value_dim
        self.conv1d = nn.Conv1d(conv_dim, conv_dim, c.lin_conv, groups=conv_dim, padding=c.lin_conv - 1, bias=False)
        self.in_proj_qkvz = Linear(c.hidden_size, 2 * self.key_dim + 2 * self.value_dim, bias=False)
        self.in_proj_ba = Linear(c.hidden_size, 2 * c.lin_v_heads, bias=False)
        self.dt_bias = nn.Parameter(torch.ones(c.lin_v_heads))
        self.A_log = nn.Parameter(torch.log(torch.empty(c.lin_v_heads).uniform_(0, 16)))
        self.norm = Norm(c.lin_v_dim, "rms", c.norm_eps)
        self.out_proj = Linear(self.value_dim, c.hidden_size, bias=False)

    def forward(self, x, rope, positions, cache: Optional[KVCache], k_positions):
        from ..gdn import gdn_chunked, gdn_recurrent
        c = self.c
        B, T, _ = x.shape
        hk, hv, dk, dv = c.lin_k_heads, c.lin_v_heads, c.lin_k_dim, c.lin_v_dim
        r = hv // hk
        qkvz = self.in_proj_qkvz(x).view(B, T, hk, 2 * dk + 2 * r * dv)
        ba = self.in_proj_ba(x).view(B, T, hk, 2 * r)
        q, k, v, z = qkvz.split((dk, dk, r * dv, r * dv), -1)
        b, a = ba.split((r, r), -1)
        v, z = v.reshape(B, T, hv, dv), z.reshape(B, T, hv, dv)
        b, a = b.reshape(B, T, hv), a.reshape(B, T, hv)
        mixed = torch.cat((q.reshape(B, T, -1), k.reshape(B, T, -1), v.reshape(B, T, -1)), -1).transpose(1, 2)
        st = cache.state.get(self.idx) if cache is not None else None
        kw = c.lin_conv
        prev = st[0] if st is not None else mixed.new_zeros(B, mixed.shape[1], kw - 1)
        full = torch.cat((prev, mixed), -1)
        conv = F.silu(F.conv1d(full, self.conv1d.weight, None, groups=full.shape[1]))[:, :, -T:].transpose(1, 2)
        q, k, v = conv.split((self.key_dim, self.key_dim, self.value_dim), -1)
        q, k, v = q.reshape(B, T, hk, dk), k.reshape(B, T, hk, dk), v.reshape(B, T, hv, dv)
        beta = torch.sigmoid(b)
        g = torch.exp(-self.A_log.float().exp() * F.softplus(a.float() + self.dt_bias))
        if r > 1:
            q, k = q.repeat_interleave(r, 2), k.repeat_interleave(r, 2)
        qf, kf = q.float(), k.float()
        qf = qf * torch.rsqrt((qf * qf).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
        kf = kf * torch.rsqrt((kf * kf).sum(-1, keepdim=True) + 1e-6)
        use_kernel = False
        if x.is_cuda and not torch.is_grad_enabled():
            from ...ops import native
            use_kernel = native.available() and native.gdn_scan_supported(dk, dv)
        if use_kernel:            # recurrence kernel with the state in registers (csrc/gdn.cu)
            y_all, S_all = native.gdn_scan(qf, kf, v, g, beta, st[1] if st is not None else None)
            outs, states = list(y_all), list(S_all)
        else:
            outs, states = [], []
            for i in range(B):
                S0 = st[1][i] if st is not None else None
                fn = gdn_recurrent if T <= 4 else gdn_chunked
                y, S = fn(qf[i], kf[i], v[i].float(), g[i], beta[i].float(), S0)
                outs.append(y)
                states.append(S)
        if cache is not None:
            cache.state[self.idx] = (full[:, :, -(kw - 1):].detach(), torch.stack(states))
            cache.state["length"] = int(cache.state.get("length", 0)) if self.idx != self._first_linear() else \
                int(cache.state.get("length", 0)) + T
        y = torch.stack(outs).to(x.dtype)                                          # [B, T, hv, dv]
        y = (self.norm(y).float() * F.silu(z.float())).to(x.dtype)
        return self.out_proj(y.reshape(B, T, hv * dv))

    def _first_linear(self) -> int:
        return next(i for i in range(self.c.num_layers) if self.c.layer_type(i) == "linear")


class LatentAttention(nn.Module):
    """Multi-head latent attention: low-rank query and joint key/value compression with a shared rotary key part
    (crates/pmetal-models/src/architectures/deepseek.rs)."""

    def __init__(self, c: ArchConfig, idx: int):
        super().__init__()
        self.c, self.idx = c, idx
        H, h = c.hidden_size, c.n_heads
        qd = c.qk_nope_dim + c.qk_rope_dim
        if c.q_lora_rank:
            self.q_a_proj = Linear(H, c.q_lora_rank, bias=c.attn_bias)
            self.q_a_layernorm = Norm(c.q_lora_rank, "rms", c.norm_eps)
            self.q_b_proj = Linear(c.q_lora_rank, h * qd, bias=False)
        else:
            self.q_proj = Linear(H, h * qd, bias=False)
        self.kv_a_proj_with_mqa = Linear(H, c.kv_lora_rank + c.qk_rope_dim, bias=c.attn_bias)
        self.kv_a_layernorm = Norm(c.kv_lora_rank, "rms", c.norm_eps)
        self.kv_b_proj = Linear(c.kv_lora_rank, h * (c.qk_nope_dim + c.v_head_dim), bias=False)
        self.o_proj = Linear(h * c.v_head_dim, H, bias=c.attn_bias)

    def forward(self, x, rope, positions, cache, k_positions):
        c = self.c
        B, T, _ = x.shape
        h, nd, rd, vd = c.n_heads, c.qk_nope_dim, c.qk_rope_dim, c.v_head_dim
        q = self.q_b_proj(self.q_a_layernorm(self.q_a_proj(x))) if c.q_lora_rank else self.q_proj(x)
        q = q.view(B, T, h, nd + rd).transpose(1, 2)
        ckv = self.kv_a_proj_with_mqa(x)
        k_rope = ckv[..., c.kv_lora_rank:].view(B, T, 1, rd).transpose(1, 2)
        kv = self.kv_b_proj(self.kv_a_layernorm(ckv[..., : c.kv_lora_rank])).view(B, T, h, nd + vd).transpose(1, 2)
        cos, sin = rope["global"]
        q_rope = apply_rope(q[..., nd:], cos, sin, True)
        k_rope = apply_rope(k_rope, cos, sin, True)
        q = torch.cat((q[..., :nd], q_rope), -1)
        k = torch.cat((kv[..., :nd], k_rope.expand(B, h, T, rd)), -1)
        v = kv[..., nd:]
        if cache is not None:
            k, v = cache.append(self.idx, k, v)
        mask = rope["mask"] if rope.get("mask") is not None else \
            with_documents(build_mask("full", positions, k_positions, 0, 0), rope.get("doc_ids"))
        scale = (nd + rd) ** -0.5 * rope.get("attention_factor", 1.0) ** 2
        o = attend(q, k, v, mask, scale)
        return self.o_proj(o.transpose(1, 2).reshape(B, T, h * vd))


class MLP(nn.Module):
    def __init__(self, c: ArchConfig, inter: int):
        super().__init__()
        self.c = c
        H = c.hidden_size
        if not c.gated_mlp:
            self.fc1, self.fc2 = Linear(H, inter, bias=c.mlp_bias), Linear(inter, H, bias=c.mlp_bias)
        elif c.fused_qkv:
            self.gate_up_proj, self.down_proj = Linear(H, 2 * inter, bias=c.mlp_bias), Linear(inter, H, bias=c.mlp_bias)
        else:
            self.gate_proj, self.up_proj = Linear(H, inter, bias=c.mlp_bias), Linear(H, inter, bias=c.mlp_bias)
            self.down_proj = Linear(inter, H, bias=c.mlp_bias)
        self.fn = _act(c.act)

    def forward(self, x):
        if not self.c.gated_mlp:
            return self.fc2(self.fn(self.fc1(x)))
        if self.c.fused_qkv:
            g, u = self.gate_up_proj(x).chunk(2, -1)
            return self.down_proj(_glu(g, u, self.c.act, self.fn))
        return self.down_proj(_glu(self.gate_proj(x), self.up_proj(x), self.c.act, self.fn))


class Experts(nn.Module):
    """Stacked expert weights in the checkpoint's own layout."""

    def __init__(self, c: ArchConfig):
        super().__init__()
        self.c = c
        E, H, I = c.num_experts, c.hidden_size, c.moe_intermediate
        if c.expert_layout == "out_in":
            self.gate_up_proj, self.down_proj = nn.Parameter(torch.empty(E, 2 * I, H)), nn.Parameter(torch.empty(E, H, I))
        else:
            self.gate_up_proj, self.down_proj = nn.Parameter(torch.empty(E, H, 2 * I)), nn.Parameter(torch.empty(E, I, H))
        if c.expert_bias:
            self.gate_up_proj_bias, self.down_proj_bias = nn.Parameter(torch.zeros(E, 2 * I)), nn.Parameter(torch.zeros(E, H))
        for p in (self.gate_up_proj, self.down_proj):
            nn.init.normal_(p, std=0.02)

    def one(self, e: int, x: torch.Tensor) -> torch.Tensor:
        c = self.c
        wgu, wd = self.gate_up_proj[e], self.down_proj[e]
        gu = x @ (wgu.t() if c.expert_layout == "out_in" else wgu)
        if c.expert_bias:
            gu = gu + self.gate_up_proj_bias[e]
        if c.expert_act == "oss":
            g, u = gu[..., 0::2].clamp(max=7.0), gu[..., 1::2].clamp(-7.0, 7.0)
            h = (u + 1.0) * (g * torch.sigmoid(g * 1.702))
        else:
            g, u = gu.chunk(2, -1)
            h = _act(c.act)(g) * u
        y = h @ (wd.t() if c.expert_layout == "out_in" else wd)
        if c.expert_bias:
            y = y + self.down_proj_bias[e]
        return y


class _Router(nn.Module):
    def __init__(self, c: ArchConfig):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(c.num_experts, c.hidden_size))
        nn.init.normal_(self.weight, std=0.02)
        if c.router_bias:
            self.bias = nn.Parameter(torch.zeros(c.num_experts))
        if c.router == "sigmoid_group":
            self.register_buffer("e_score_correction_bias", torch.zeros(c.num_experts))


class _RouterHolder(nn.Module):          # granitemoe stores the router weight under ``router.layer``
    def __init__(self, c):
        super().__init__()
        self.layer = _Router(c)


def route(c: ArchConfig, logits: torch.Tensor, bias: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """logits [N, E] -> (weights [N, k] fp32, expert ids [N, k]) under the configured routing rule."""
    k = c.top_k
    lf = logits.float()
    if c.router == "softmax_topk":
        w, idx = torch.topk(torch.softmax(lf, -1), k, -1)
        if c.norm_topk_prob:
            w = w / w.sum(-1, keepdim=True)
        return w, idx
    if c.router == "topk_softmax":
        top, idx = torch.topk(lf, k, -1)
        return torch.softmax(top, -1), idx
    if c.router == "sigmoid_input":
        top, idx = torch.topk(lf, k, -1)
        return torch.sigmoid(top), idx
    scores = torch.sigmoid(lf) if c.router == "sigmoid_group" else torch.softmax(lf, -1)
    choice = scores + bias.float() if (bias is not None and c.router == "sigmoid_group") else scores
    if c.n_group > 1:
        N, E = choice.shape
        grp = choice.view(N, c.n_group, E // c.n_group)
        gs = grp.topk(2, -1)[0].sum(-1) if c.group_score == "top2sum" else grp.max(-1)[0]
        keep = torch.zeros_like(gs).scatter_(1, gs.topk(c.topk_group, -1, sorted=False)[1], 1.0)
        keep = keep[:, :, None].expand(N, c.n_group, E // c.n_group).reshape(N, E).bool()
        choice = choice.masked_fill(~keep, 0.0 if c.router == "sigmoid_group" else 0.0)
    idx = torch.topk(choice, k, -1, sorted=False)[1]
    w = scores.gather(1, idx)
    if c.norm_topk_prob and k > 1:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return w * c.routed_scale, idx


class MoE(nn.Module):
    def __init__(self, c: ArchConfig):
        super().__init__()
        self.c = c
        if "." in c.router_name:
            self.router = _RouterHolder(c)
            self._router = lambda: self.router.layer
        else:
            setattr(self, c.router_name, _Router(c))
            self._router = lambda: getattr(self, c.router_name)
        if c.moe_name == "block_sparse_moe":            # granitemoe: input_linear / output_linear
            E, H, I = c.num_experts, c.hidden_size, c.moe_intermediate
            self.input_linear = nn.Module()
            self.input_linear.weight = nn.Parameter(torch.empty(E, 2 * I, H).normal_(std=0.02))
            self.output_linear = nn.Module()
            self.output_linear.weight = nn.Parameter(torch.empty(E, H, I).normal_(std=0.02))
        else:
            self.experts = Experts(c)
        if c.n_shared_experts:
            shared = MLP(_dense_view(c), c.shared_intermediate or c.moe_intermediate * c.n_shared_experts)
            setattr(self, c.shared_name, shared)
            if c.shared_gate:
                self.shared_expert_gate = Linear(c.hidden_size, 1, bias=False)

    def _expert(self, e: int, x: torch.Tensor) -> torch.Tensor:
        if self.c.moe_name == "block_sparse_moe":
            g, u = (x @ self.input_linear.weight[e].t()).chunk(2, -1)
            return (_act(self.c.act)(g) * u) @ self.output_linear.weight[e].t()
        return self.experts.one(e, x)

    def forward(self, x):
        c = self.c
        shape = x.shape
        xf = x.reshape(-1, shape[-1])
        r = self._router()
        logits = F.linear(xf, r.weight, getattr(r, "bias", None))
        w, idx = route(c, logits, getattr(r, "e_score_correction_bias", None))
        out = torch.zeros_like(xf, dtype=torch.float32)
        for e in idx.unique().tolist():
            tok, slot = (idx == e).nonzero(as_tuple=True)
            xe = xf[tok]
            if c.router == "sigmoid_input":
                y = self._expert(e, xe * w[tok, slot, None].to(xe.dtype)).float()
            else:
                y = self._expert(e, xe).float() * w[tok, slot, None]
            out.index_add_(0, tok, y)
        out = out.to(x.dtype)
        if c.n_shared_experts:
            s = getattr(self, c.shared_name)(xf)
            if c.shared_gate:
                s = torch.sigmoid(self.shared_expert_gate(xf)) * s
            out = out + s
        return out.view(shape)


def _dense_view(c: ArchConfig) -> ArchConfig:
    """The config a shared expert's MLP sees: gated, unfused, without bias."""
    import copy
    d = copy.copy(c)
    d.gated_mlp, d.fused_qkv, d.mlp_bias = True, False, False
    return d


class Block(nn.Module):
    def __init__(self, c: ArchConfig, idx: int):
        super().__init__()
        self.c = c
        if c.layer_type(idx) == "linear":
            self.linear_attn = GatedDeltaNet(c, idx)
        else:
            self.self_attn = LatentAttention(c, idx) if c.mla else Attention(c, idx)
        self._mix = lambda: self.linear_attn if c.layer_type(idx) == "linear" else self.self_attn
        if c.mlp_type(idx) == "moe":
            setattr(self, c.moe_name, MoE(c))
            self._ff = lambda: getattr(self, c.moe_name)
        else:
            name = c.moe_name if c.moe_name == "feed_forward" else "mlp"
            setattr(self, name, MLP(c, c.dense_intermediate or c.intermediate_size))
            self._ff = lambda: getattr(self, name)
        H, n, e = c.hidden_size, c.norm, c.norm_eps
        if c.block != "post":
            self.input_layernorm = Norm(H, n, e)
        if c.block in ("sequential", "sandwich", "post"):
            self.post_attention_layernorm = Norm(H, n, e)
        if c.block == "sandwich":
            self.pre_feedforward_layernorm, self.post_feedforward_layernorm = Norm(H, n, e), Norm(H, n, e)
        if c.block == "post":
            self.post_feedforward_layernorm = Norm(H, n, e)

    def forward(self, x, rope, positions, cache, k_positions):
        c, rm = self.c, self.c.residual_multiplier
        ff = self._ff()
        if c.block == "parallel":
            n = self.input_layernorm(x)
            return x + self._mix()(n, rope, positions, cache, k_positions) + ff(n)
        if c.block == "sandwich":
            x = x + self.post_attention_layernorm(self._mix()(self.input_layernorm(x), rope, positions, cache, k_positions))
            return x + self.post_feedforward_layernorm(ff(self.pre_feedforward_layernorm(x)))
        if c.block == "post":
            x = x + self.post_attention_layernorm(self._mix()(x, rope, positions, cache, k_positions))
            return x + self.post_feedforward_layernorm(ff(x))
        x = x + rm * self._mix()(self.input_layernorm(x), rope, positions, cache, k_positions)
        return x + rm * ff(self.post_attention_layernorm(x))


class _Backbone(nn.Module):
    def __init__(self, c: ArchConfig):
        super().__init__()
        self.embed_tokens = nn.Embedding(c.vocab_size, c.hidden_size)
        self.layers = nn.ModuleList([Block(c, i) for i in range(c.num_layers)])
        setattr(self, c.final_norm_name, Norm(c.hidden_size, c.norm, c.norm_eps))


class GenericDecoderLM(nn.Module):
    def __init__(self, c: ArchConfig):
        super().__init__()
        self.c = c
        self.model = _Backbone(c)
        if not c.tie_embeddings:
            self.lm_head = Linear(c.hidden_size, c.vocab_size, bias=c.lm_head_bias)
        rd = c.rope_dim or c.head_dim
        inv, att = rope_inv_freq(rd, c.rope_theta, c.rope_scaling, c.max_position)
        self.register_buffer("inv_freq", inv, persistent=False)
        self.attention_factor = att
        if c.rope_local_theta:
            self.register_buffer("inv_freq_local", rope_inv_freq(rd, c.rope_local_theta, None, c.max_position)[0], persistent=False)

    @classmethod
    def from_hf_config(cls, d: dict) -> "GenericDecoderLM":
        return cls(arch_config_from_hf(d))

    def init_weights(self, std: float = 0.02, seed: int = 0) -> "GenericDecoderLM":
        g = torch.Generator().manual_seed(seed)
        for n, p in self.named_parameters():
            if p.dim() >= 2:
                p.data.copy_(torch.randn(p.shape, generator=g) * std)
        return self

    def _rope(self, positions: torch.Tensor) -> dict:
        out = {"attention_factor": self.attention_factor}
        ang = positions[:, :, None].float() * self.inv_freq[None, None].float()
        out["global"] = (torch.cos(ang) * self.attention_factor, torch.sin(ang) * self.attention_factor)
        if self.c.rope_local_theta:
            a2 = positions[:, :, None].float() * self.inv_freq_local[None, None].float()
            out["local"] = (torch.cos(a2), torch.sin(a2))
        # the attention factor already multiplies cos/sin (as the checkpoints' own code does), so the score scale stays
        out["attention_factor"] = 1.0 if not self.c.mla else self._mla_mscale()
        return out

    def _mla_mscale(self) -> float:
        sc = self.c.rope_scaling or {}
        if sc.get("rope_type") == "yarn" and sc.get("mscale_all_dim"):
            f, m = float(sc.get("factor", 1.0)), float(sc["mscale_all_dim"])
            return 1.0 if f <= 1 else 0.1 * m * math.log(f) + 1.0
        return 1.0

    def forward_hidden(self, input_ids: torch.Tensor, cache: Optional[KVCache] = None,
                       positions: Optional[torch.Tensor] = None, attn_mask: Optional[torch.Tensor] = None,
                       doc_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``attn_mask`` (bool [B, 1, Tq, Tk], True = attend) replaces the position-derived causal mask in every layer
        (tree-structured verification); full-attention models only. ``doc_ids`` [B, T] marks packed rows: tokens attend
        inside their own document only (on top of the causal / sliding / chunked rule of each layer) and ``positions``
        should restart at every document; recurrent layers (Mamba, gated delta net) are not reset at the boundaries."""
        c = self.c
        if input_ids.dim() == 1:
            input_ids = input_ids[None]
        B, T = input_ids.shape
        past = cache.length() if cache is not None else 0
        default_positions = positions is None
        if positions is None:
            positions = torch.arange(past, past + T, device=input_ids.device)[None].expand(B, T)
        k_positions = torch.arange(0, past + T, device=input_ids.device)[None].expand(B, past + T) if cache is not None \
            else positions
        x = self.model.embed_tokens(input_ids)
        if c.embed_scale != 1.0:
            x = x * torch.tensor(c.embed_scale, dtype=x.dtype)
        rope = self._rope(positions)
        rope["mask"] = attn_mask
        rope["doc_ids"] = doc_ids if cache is None else None
        rope["contiguous"] = default_positions and past == 0       # every row is a whole sequence starting at position 0
        for layer in self.model.layers:
            x = layer(x, rope, positions, cache, k_positions)
        return getattr(self.model, c.final_norm_name)(x)

    def logits(self, h: torch.Tensor) -> torch.Tensor:
        c = self.c
        z = F.linear(h, self.model.embed_tokens.weight) if c.tie_embeddings else self.lm_head(h)
        if c.logit_scale != 1.0:
            z = z * c.logit_scale
        if c.logits_divisor != 1.0:
            z = z / c.logits_divisor
        if c.final_softcap > 0:
            z = torch.tanh(z / c.final_softcap) * c.final_softcap
        return z

    def loss_head(self):
        """(head matrix [V, H], factor on the logits, soft cap) when the read-out is one bias-free matrix, so that a trainer
        can fuse it with the cross entropy instead of materialising [tokens, V] logits; None otherwise."""
        c = self.c
        if c.tie_embeddings:
            w = self.model.embed_tokens.weight
        else:
            head = self.lm_head
            if type(head).__name__ not in ("Linear",) or getattr(head, "bias", None) is not None:
                return None
            w = head.weight
        return w, c.logit_scale / c.logits_divisor, c.final_softcap

    def forward(self, input_ids, cache: Optional[KVCache] = None, positions=None, attn_mask=None, doc_ids=None) -> torch.Tensor:
        return self.logits(self.forward_hidden(input_ids, cache, positions, attn_mask, doc_ids))

    def new_cache(self, kv_bits: Optional[int] = None, kv_group: int = 64, turbo: bool = False, qjl: bool = False) -> KVCache:
        """``kv_bits`` None: keys and values in the model dtype; 8 / 4: group-quantised; with ``turbo`` 2 / 4 / 8 bit
        rotation + codebook compression."""
        if kv_bits is None:
            return KVCache(self.c.num_layers)
        return QuantKVCache(self.c.num_layers, kv_bits, kv_group, turbo, qjl)

    @torch.no_grad()
    def generate(self, prompt: List[int], max_new_tokens: int = 32, eos_token_id: Optional[int] = None,
                 kv_bits: Optional[int] = None) -> List[int]:
        """Greedy decoding with the contiguous cache."""
        dev = self.model.embed_tokens.weight.device
        cache = self.new_cache(kv_bits)
        ids = torch.tensor([prompt], device=dev)
        out: List[int] = []
        for _ in range(max_new_tokens):
            nxt = int(self.forward(ids, cache)[0, -1].argmax())
            out.append(nxt)
            if eos_token_id is not None and nxt == eos_token_id:
                break
            ids = torch.tensor([[nxt]], device=dev)
        return out


def convert_legacy_expert_keys(sd: Dict[str, torch.Tensor], c: ArchConfig) -> Dict[str, torch.Tensor]:
    """Checkpoints that store one tensor per expert (``...experts.N.{w1,w3,w2}`` or ``{gate,up,down}_proj``) are
    restacked into the fused ``experts.gate_up_proj`` / ``experts.down_proj`` parameters."""
    import re
    pat = re.compile(r"^(.*)\.(?:block_sparse_moe|mlp)\.experts\.(\d+)\.(w1|w2|w3|gate_proj|up_proj|down_proj)\.weight$")
    groups: Dict[str, Dict[int, Dict[str, torch.Tensor]]] = {}
    out: Dict[str, torch.Tensor] = {}
    for k, v in sd.items():
        m = pat.match(k)
        if not m:
            out[k.replace(".block_sparse_moe.gate.", ".mlp.gate.")] = v
            continue
        role = {"w1": "gate", "gate_proj": "gate", "w3": "up", "up_proj": "up", "w2": "down", "down_proj": "down"}[m.group(3)]
        groups.setdefault(m.group(1), {}).setdefault(int(m.group(2)), {})[role] = v
    for prefix, ex in groups.items():
        order = sorted(ex)
        out[f"{prefix}.mlp.experts.gate_up_proj"] = torch.stack([torch.cat((ex[e]["gate"], ex[e]["up"]), 0) for e in order])
        out[f"{prefix}.mlp.experts.down_proj"] = torch.stack([ex[e]["down"] for e in order])
    return out
