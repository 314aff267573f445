"""Gemma 4 text decoder.

Differs from the earlier Gemma generations enough to have its own module (the reference does the same:
crates/pmetal-models/src/architectures/gemma4.rs:1-60 lists the features, :274-440 the config helpers, :634-870 the
attention, :873-1000 the decoder layer):

* sliding and full-attention layers have different head sizes (``head_dim`` / ``global_head_dim``) and rotary tables:
  the sliding layers rotate every pair with theta 1e4, the full layers rotate the first quarter of the pairs with theta
  1e6 ("proportional" RoPE: the exponent's denominator stays the full head size and the other pairs get angle 0);
* ``attention_k_eq_v``: full-attention layers have no value projection, the values are the raw key projection (before the
  key norm and rotation), and they may use ``num_global_key_value_heads`` heads;
* a value norm without a learnable scale; score scale 1.0 (the q/k norms carry the scale);
* the last ``num_kv_shared_layers`` layers own no keys/values and read those of the last earlier layer of their kind;
  their MLP is twice as wide when ``use_double_wide_mlp`` is set;
* per-layer inputs: a second embedding table yields a small vector per (token, layer); it is mixed with a projection of the
  main embedding and gates a low-rank residual branch at the end of every layer;
* an optional sparse expert block that runs in parallel with the dense MLP (router on the un-normalised residual);
* a per-layer output scalar and a tanh soft-cap on the final logits.

Parameter names match the published checkpoints, so a Hugging Face state dict loads directly; a multimodal checkpoint's
``model.language_model.`` prefix is stripped by :meth:`Gemma4LM.load_hf_state_dict`."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .fast import Linear

from .generic import KVCache, _act, apply_rope, attend, build_mask


@dataclass
class Gemma4Config:
    vocab_size: int = 262144
    hidden_size: int = 2304
    intermediate_size: int = 9216
    num_layers: int = 30
    num_heads: int = 8
    num_kv_heads: int = 4
    head_dim: int = 256
    global_head_dim: int = 512
    num_global_kv_heads: Optional[int] = None
    k_eq_v: bool = False
    activation: str = "gelu_pytorch_tanh"
    eps: float = 1e-6
    sliding_window: int = 512
    layer_types: List[str] = field(default_factory=list)
    rope_local: Dict = field(default_factory=lambda: {"rope_type": "default", "rope_theta": 10000.0})
    rope_global: Dict = field(default_factory=lambda: {"rope_type": "proportional", "partial_rotary_factor": 0.25,
                                                       "rope_theta": 1000000.0})
    final_softcap: float = 0.0
    vocab_size_per_layer: int = 262144
    per_layer_dim: int = 256
    num_kv_shared_layers: int = 0
    double_wide_mlp: bool = False
    moe: bool = False
    num_experts: int = 0
    top_k: int = 0
    moe_intermediate_size: int = 0
    attention_bias: bool = False
    tie_embeddings: bool = True

    @classmethod
    def from_hf(cls, d: dict) -> "Gemma4Config":
        d = d.get("text_config", d)
        L = d.get("num_hidden_layers", 30)
        types = d.get("layer_types") or ["sliding_attention" if (i + 1) % 6 else "full_attention" for i in range(L)]
        types = list(types)
        types[-1] = "full_attention"                  # the published configuration forces a global last layer
        c = cls(vocab_size=d.get("vocab_size", 262144), hidden_size=d.get("hidden_size", 2304),
                intermediate_size=d.get("intermediate_size", 9216), num_layers=L,
                num_heads=d.get("num_attention_heads", 8), num_kv_heads=d.get("num_key_value_heads", 4),
                head_dim=d.get("head_dim", 256), global_head_dim=d.get("global_head_dim") or d.get("head_dim", 256),
                num_global_kv_heads=d.get("num_global_key_value_heads"), k_eq_v=bool(d.get("attention_k_eq_v", False)),
                activation=d.get("hidden_activation", "gelu_pytorch_tanh"), eps=d.get("rms_norm_eps", 1e-6),
                sliding_window=d.get("sliding_window", 512), layer_types=types,
                final_softcap=float(d.get("final_logit_softcapping") or 0.0),
                vocab_size_per_layer=d.get("vocab_size_per_layer_input", d.get("vocab_size", 262144)),
                per_layer_dim=int(d.get("hidden_size_per_layer_input") or 0),
                num_kv_shared_layers=int(d.get("num_kv_shared_layers") or 0),
                double_wide_mlp=bool(d.get("use_double_wide_mlp", False)), moe=bool(d.get("enable_moe_block", False)),
                num_experts=int(d.get("num_experts") or 0), top_k=int(d.get("top_k_experts") or 0),
                moe_intermediate_size=int(d.get("moe_intermediate_size") or 0),
                attention_bias=bool(d.get("attention_bias", False)), tie_embeddings=bool(d.get("tie_word_embeddings", True)))
        rp = d.get("rope_parameters") or {}
        if rp.get("sliding_attention"):
            c.rope_local = dict(rp["sliding_attention"])
        if rp.get("full_attention"):
            c.rope_global = dict(rp["full_attention"])
        return c

    # ---- per-layer geometry
    def is_full(self, i: int) -> bool:
        return self.layer_types[i] == "full_attention"

    def layer_head_dim(self, i: int) -> int:
        return self.global_head_dim if self.is_full(i) and self.global_head_dim else self.head_dim

    def layer_k_eq_v(self, i: int) -> bool:
        return self.k_eq_v and self.is_full(i)

    def layer_kv_heads(self, i: int) -> int:
        return (self.num_global_kv_heads or self.num_kv_heads) if self.layer_k_eq_v(i) else self.num_kv_heads

    @property
    def first_shared(self) -> int:
        return self.num_layers - self.num_kv_shared_layers

    def kv_source(self, i: int) -> Optional[int]:
        """The layer whose keys/values layer ``i`` reads, or None when it computes its own."""
        if self.num_kv_shared_layers <= 0 or i < self.first_shared:
            return None
        for j in range(self.first_shared - 1, -1, -1):
            if self.layer_types[j] == self.layer_types[i]:
                return j
        raise ValueError(f"layer {i} shares keys/values but no earlier {self.layer_types[i]} layer exists")


def rope_table(params: Dict, head_dim: int) -> torch.Tensor:
    """Inverse frequencies [head_dim/2] of one layer kind. ``proportional`` rotates only the first
    ``partial_rotary_factor`` of the pairs, keeps ``head_dim`` in the exponent and leaves the rest at angle 0."""
    theta = float(params.get("rope_theta", 10000.0))
    kind = params.get("rope_type", "default")
    if kind == "proportional":
        n = int(float(params.get("partial_rotary_factor", 1.0)) * head_dim // 2)
        inv = 1.0 / (theta ** (torch.arange(0, 2 * n, 2, dtype=torch.float32) / head_dim))
        inv = torch.cat((inv, torch.zeros(head_dim // 2 - n)))
        return inv / float(params.get("factor", 1.0))
    if kind == "linear":
        return 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim)) / float(params.get("factor", 1.0))
    if kind != "default":
        raise ValueError(f"unsupported rope type {kind!r} for Gemma 4")
    return 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))


class RMSNorm(nn.Module):
    """fp32 RMS norm with a plain (not 1 + w) scale, or none at all."""

    def __init__(self, dim: int, eps: float, with_scale: bool = True):
        super().__init__()
        self.eps = eps
        if with_scale:
            self.weight = nn.Parameter(torch.ones(dim))
        else:
            self.register_parameter("weight", None)

    def forward(self, x):
        xf = x.float()
        y = xf * torch.pow(xf.pow(2).mean(-1, keepdim=True) + self.eps, -0.5)
        if self.weight is not None:
            y = y * self.weight.float()
        return y.to(x.dtype)


class Gemma4Attention(nn.Module):
    def __init__(self, c: Gemma4Config, idx: int):
        super().__init__()
        self.c, self.idx = c, idx
        self.full = c.is_full(idx)
        self.d = c.layer_head_dim(idx)
        self.hkv = c.layer_kv_heads(idx)
        self.source = c.kv_source(idx)
        H, b = c.hidden_size, c.attention_bias
        self.q_proj = Linear(H, c.num_heads * self.d, bias=b)
        self.k_proj = Linear(H, self.hkv * self.d, bias=b)
        self.v_proj = None if c.layer_k_eq_v(idx) else Linear(H, self.hkv * self.d, bias=b)
        self.o_proj = Linear(c.num_heads * self.d, H, bias=b)
        self.q_norm = RMSNorm(self.d, c.eps)
        self.k_norm = RMSNorm(self.d, c.eps)
        self.v_norm = RMSNorm(self.d, c.eps, with_scale=False)

    def forward(self, x, rope, positions, cache: Optional[KVCache], k_positions, shared: Dict[int, Tuple]):
        B, T, _ = x.shape
        cos, sin = rope
        q = self.q_norm(self.q_proj(x).view(B, T, -1, self.d)).transpose(1, 2)
        q = apply_rope(q, cos, sin, False)
        if self.source is not None and self.source in shared:
            k, v = shared[self.source]
        else:
            kr = self.k_proj(x).view(B, T, self.hkv, self.d)
            vr = self.v_proj(x).view(B, T, self.hkv, self.d) if self.v_proj is not None else kr
            k = apply_rope(self.k_norm(kr).transpose(1, 2), cos, sin, False)
            v = self.v_norm(vr).transpose(1, 2)
            if cache is not None:
                k, v = cache.append(self.idx, k, v)
            shared[self.idx] = (k, v)
        kind = "causal" if self.full else "sliding"
        mask = build_mask(kind, positions, k_positions, self.c.sliding_window, 0)
        y = attend(q, k, v, mask, 1.0)
        return self.o_proj(y.transpose(1, 2).reshape(B, T, -1))


class Gemma4MLP(nn.Module):
    def __init__(self, c: Gemma4Config, idx: int):
        super().__init__()
        wide = c.double_wide_mlp and c.kv_source(idx) is not None
        inter = c.intermediate_size * (2 if wide else 1)
        self.gate_proj = Linear(c.hidden_size, inter, bias=False)
        self.up_proj = Linear(c.hidden_size, inter, bias=False)
        self.down_proj = Linear(inter, c.hidden_size, bias=False)
        self.act = _act(c.activation)

    def forward(self, x):
        return self.down_proj(self.act(self.gate_proj(x)) * self.up_proj(x))


class Gemma4Router(nn.Module):
    """Scale-free RMS norm, a learned per-channel scale times hidden^-0.5, softmax, top-k renormalised to sum 1, then a
    learned per-expert multiplier."""

    def __init__(self, c: Gemma4Config):
        super().__init__()
        self.c = c
        self.norm = RMSNorm(c.hidden_size, c.eps, with_scale=False)
        self.proj = Linear(c.hidden_size, c.num_experts, bias=False)
        self.scale = nn.Parameter(torch.ones(c.hidden_size))
        self.per_expert_scale = nn.Parameter(torch.ones(c.num_experts))

    def forward(self, x):
        h = self.norm(x) * self.scale * (self.c.hidden_size ** -0.5)
        p = torch.softmax(self.proj(h), -1)
        w, idx = torch.topk(p, self.c.top_k, -1)
        w = w / w.sum(-1, keepdim=True)
        return w * self.per_expert_scale[idx], idx


class Gemma4Experts(nn.Module):
    def __init__(self, c: Gemma4Config):
        super().__init__()
        E, H, I = c.num_experts, c.hidden_size, c.moe_intermediate_size
        self.gate_up_proj = nn.Parameter(torch.zeros(E, 2 * I, H))
        self.down_proj = nn.Parameter(torch.zeros(E, H, I))
        self.act = _act(c.activation)

    def forward(self, x, idx, w):
        """x [N, H], idx/w [N, k]: tokens grouped per expert (sorted by expert id), one pair of GEMMs per used expert."""
        N, k = idx.shape
        flat = idx.reshape(-1)
        order = torch.argsort(flat, stable=True)
        counts = torch.bincount(flat, minlength=self.gate_up_proj.shape[0]).tolist()
        tok = torch.div(order, k, rounding_mode="floor")
        out = torch.zeros_like(x)
        start = 0
        for e, n in enumerate(counts):
            if n == 0:
                continue
            sel = order[start:start + n]
            t = tok[start:start + n]
            g, u = F.linear(x[t], self.gate_up_proj[e]).chunk(2, -1)
            y = F.linear(self.act(g) * u, self.down_proj[e]) * w.reshape(-1)[sel, None]
            out.index_add_(0, t, y.to(out.dtype))
            start += n
        return out


class Gemma4Layer(nn.Module):
    def __init__(self, c: Gemma4Config, idx: int):
        super().__init__()
        self.c = c
        H = c.hidden_size
        self.self_attn = Gemma4Attention(c, idx)
        self.mlp = Gemma4MLP(c, idx)
        self.input_layernorm = RMSNorm(H, c.eps)
        self.post_attention_layernorm = RMSNorm(H, c.eps)
        self.pre_feedforward_layernorm = RMSNorm(H, c.eps)
        self.post_feedforward_layernorm = RMSNorm(H, c.eps)
        self.register_buffer("layer_scalar", torch.ones(1))
        if c.per_layer_dim:
            self.per_layer_input_gate = Linear(H, c.per_layer_dim, bias=False)
            self.per_layer_projection = Linear(c.per_layer_dim, H, bias=False)
            self.post_per_layer_input_norm = RMSNorm(H, c.eps)
            self.act = _act(c.activation)
        if c.moe:
            self.router = Gemma4Router(c)
            self.experts = Gemma4Experts(c)
            self.post_feedforward_layernorm_1 = RMSNorm(H, c.eps)
            self.post_feedforward_layernorm_2 = RMSNorm(H, c.eps)
            self.pre_feedforward_layernorm_2 = RMSNorm(H, c.eps)

    def forward(self, x, per_layer, rope, positions, cache, k_positions, shared):
        x = x + self.post_attention_layernorm(self.self_attn(self.input_layernorm(x), rope, positions, cache, k_positions, shared))
        r = x
        h = self.mlp(self.pre_feedforward_layernorm(x))
        if self.c.moe:
            flat = r.reshape(-1, r.shape[-1])
            w, idx = self.router(flat)
            h2 = self.experts(self.pre_feedforward_layernorm_2(flat), idx, w).reshape(r.shape)
            h = self.post_feedforward_layernorm_1(h) + self.post_feedforward_layernorm_2(h2)
        x = r + self.post_feedforward_layernorm(h)
        if self.c.per_layer_dim:
            g = self.act(self.per_layer_input_gate(x)) * per_layer
            x = x + self.post_per_layer_input_norm(self.per_layer_projection(g))
        return x * self.layer_scalar.to(x.dtype)


class _Backbone(nn.Module):
    def __init__(self, c: Gemma4Config):
        super().__init__()
        self.embed_tokens = nn.Embedding(c.vocab_size, c.hidden_size)
        self.layers = nn.ModuleList(Gemma4Layer(c, i) for i in range(c.num_layers))
        self.norm = RMSNorm(c.hidden_size, c.eps)
        if c.per_layer_dim:
            self.embed_tokens_per_layer = nn.Embedding(c.vocab_size_per_layer, c.num_layers * c.per_layer_dim)
            self.per_layer_model_projection = Linear(c.hidden_size, c.num_layers * c.per_layer_dim, bias=False)
            self.per_layer_projection_norm = RMSNorm(c.per_layer_dim, c.eps)


class Gemma4LM(nn.Module):
    def __init__(self, c: Gemma4Config):
        super().__init__()
        self.c = c
        self.model = _Backbone(c)
        if not c.tie_embeddings:
            self.lm_head = Linear(c.hidden_size, c.vocab_size, bias=False)
        self.register_buffer("inv_local", rope_table(c.rope_local, c.head_dim), persistent=False)
        self.register_buffer("inv_global", rope_table(c.rope_global, c.global_head_dim or c.head_dim), persistent=False)

    @classmethod
    def from_hf_config(cls, d: dict) -> "Gemma4LM":
        return cls(Gemma4Config.from_hf(d))

    def init_weights(self, std: float = 0.02, seed: int = 0) -> "Gemma4LM":
        g = torch.Generator().manual_seed(seed)
        for _, p in self.named_parameters():
            if p.dim() >= 2:
                p.data.copy_(torch.randn(p.shape, generator=g) * std)
        return self

    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor], strict: bool = True):
        """Accepts text-only checkpoints (``model.layers…``) and the text tower of a multimodal one
        (``model.language_model.layers…``); vision/audio tower tensors are dropped."""
        out = {}
        for k, v in sd.items():
            if k.startswith("model.language_model."):
                out["model." + k[len("model.language_model."):]] = v
            elif k.startswith(("model.vision_tower.", "model.audio_tower.", "model.embed_vision.", "model.embed_audio.")):
                continue
            else:
                out[k] = v
        if self.c.tie_embeddings:
            out.pop("lm_head.weight", None)
        return self.load_state_dict(out, strict=strict)

    def per_layer_inputs(self, input_ids: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        """[B, T, L, P]: (norm(projection of the scaled main embedding) + scaled per-layer embedding) / sqrt(2)."""
        c, m = self.c, self.model
        B, T = input_ids.shape
        emb = m.embed_tokens_per_layer(input_ids) * torch.tensor(c.per_layer_dim ** 0.5, dtype=x.dtype)
        proj = m.per_layer_model_projection(x) * (c.hidden_size ** -0.5)
        proj = m.per_layer_projection_norm(proj.view(B, T, c.num_layers, c.per_layer_dim))
        return (proj + emb.view(B, T, c.num_layers, c.per_layer_dim)) * (2.0 ** -0.5)

    def forward_hidden(self, input_ids: torch.Tensor, cache: Optional[KVCache] = None,
                       positions: Optional[torch.Tensor] = None) -> torch.Tensor:
        c = self.c
        if input_ids.dim() == 1:
            input_ids = input_ids[None]
        B, T = input_ids.shape
        dev = input_ids.device
        past = cache.length() if cache is not None else 0
        if positions is None:
            positions = torch.arange(past, past + T, device=dev)[None].expand(B, T)
        k_positions = torch.arange(0, past + T, device=dev)[None].expand(B, past + T) if cache is not None else positions
        x = self.model.embed_tokens(input_ids)
        x = x * torch.tensor(c.hidden_size ** 0.5, dtype=x.dtype)
        per_layer = self.per_layer_inputs(input_ids, x) if c.per_layer_dim else None
        pos = positions[:, :, None].float()
        a_l, a_g = pos * self.inv_local[None, None].float(), pos * self.inv_global[None, None].float()
        ropes = {False: (torch.cos(a_l), torch.sin(a_l)), True: (torch.cos(a_g), torch.sin(a_g))}
        shared: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        for i, layer in enumerate(self.model.layers):
            x = layer(x, per_layer[:, :, i] if per_layer is not None else None, ropes[c.is_full(i)], positions, cache,
                      k_positions, shared)
        return self.model.norm(x)

    def logits(self, h: torch.Tensor) -> torch.Tensor:
        z = F.linear(h, self.model.embed_tokens.weight) if self.c.tie_embeddings else self.lm_head(h)
        if self.c.final_softcap > 0:
            z = torch.tanh(z / self.c.final_softcap) * self.c.final_softcap
        return z

    def forward(self, input_ids, cache: Optional[KVCache] = None, positions=None) -> torch.Tensor:
        return self.logits(self.forward_hidden(input_ids, cache, positions))

    def new_cache(self) -> KVCache:
        return KVCache(self.c.num_layers)

    @torch.no_grad()
    def generate(self, prompt: List[int], max_new_tokens: int = 32, eos_token_id: Optional[int] = None) -> List[int]:
        dev = self.model.embed_tokens.weight.device
        cache = self.new_cache()
        ids = torch.tensor([prompt], device=dev)
        out: List[int] = []
        for _ in range(max_new_tokens):
            nxt = int(self.forward(ids, cache)[0, -1].argmax())
            out.append(nxt)
            if eos_token_id is not None and nxt == eos_token_id:
                break
            ids = torch.tensor([[nxt]], device=dev)
        return out
