"""Llama 3.2 Vision (mllama): a tiled vision encoder feeding cross-attention layers interleaved in a Llama decoder.

Reference: crates/pmetal-models/src/architectures/mllama.rs:25-135 (configs), :138-430 (gated embeddings, vision layers
and model), :431-608 (cross attention and decoder layers), :609-830 (projector, text model, wrapper).

Vision tower: every image is cut into up to ``max_num_tiles`` tiles; a tile is patch-embedded, gets a class token, a
gated mix of one shared position table and a per-aspect-ratio tile position table, runs through the local transformer,
then (with another aspect-ratio embedding) through a tanh-gated global transformer that attends over all tiles. The
output concatenates the final state with the states after the ``intermediate_layers_indices`` local layers.

Text model: a Llama decoder (vocabulary + 8 special rows) in which the layers listed in ``cross_attention_layers``
replace self-attention by attention over the projected vision states (per-head RMS-normed q/k, tanh gates on both
residual branches, rows with no visible tile have their MLP branch zeroed). Cross-attention keys/values are computed
once per image and kept in the cache.

Parameter names match the published checkpoints (``model.vision_model.…``, ``model.language_model.…``,
``model.multi_modal_projector.…``, ``lm_head.weight``)."""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .fast import Linear

from .generic import KVCache, apply_rope, attend, rope_inv_freq


# ------------------------------------------------------------------------------------------------ vision tower
def _max_ratio_id(v: dict) -> int:
    """Aspect-ratio ids are 1-based indices into ``supported_aspect_ratios`` (0 = no image)."""
    return int(v.get("max_aspect_ratio_id") or len(v.get("supported_aspect_ratios") or [0] * 8))


class _AspectRatioEmbedding(nn.Module):
    """One learned vector per (aspect-ratio id, tile), added to every patch of the tile through a tanh gate."""

    def __init__(self, v: dict):
        super().__init__()
        self.tiles, self.dim = v["max_num_tiles"], v["hidden_size"]
        self.embedding = nn.Embedding(_max_ratio_id(v) + 1, self.tiles * self.dim)
        self.gate = nn.Parameter(torch.zeros(1))

    def forward(self, x, ids):
        return x + self.embedding(ids).reshape(-1, self.tiles, 1, self.dim) * self.gate.tanh()


class _PositionEmbedding(nn.Module):
    """(1 - tanh g) * shared patch positions + tanh g * per-aspect-ratio tile positions."""

    def __init__(self, v: dict):
        super().__init__()
        self.tiles, self.dim = v["max_num_tiles"], v["hidden_size"]
        self.patches = (v["image_size"] // v["patch_size"]) ** 2 + 1
        self.gate = nn.Parameter(torch.zeros(1))
        self.embedding = nn.Parameter(torch.randn(self.patches, self.dim) * self.dim ** -0.5)
        self.tile_embedding = nn.Embedding(_max_ratio_id(v) + 1, self.tiles * self.patches * self.dim)

    def forward(self, x, ids):
        g = self.gate.tanh()
        x = x + (1 - g) * self.embedding.view(1, 1, self.patches, self.dim)
        return x + g * self.tile_embedding(ids).reshape(x.shape[0], self.tiles, self.patches, self.dim)


class _VisionAttention(nn.Module):
    def __init__(self, v: dict):
        super().__init__()
        D, self.h = v["hidden_size"], v["attention_heads"]
        self.q_proj, self.k_proj = Linear(D, D, bias=False), Linear(D, D, bias=False)
        self.v_proj, self.o_proj = Linear(D, D, bias=False), Linear(D, D, bias=False)

    def forward(self, x, bias):
        B, N, D = x.shape
        q, k, v = (p(x).view(B, N, self.h, D // self.h).transpose(1, 2) for p in (self.q_proj, self.k_proj, self.v_proj))
        y = F.scaled_dot_product_attention(q, k, v, attn_mask=bias)
        return self.o_proj(y.transpose(1, 2).reshape(B, N, D))


class _VisionMLP(nn.Module):
    def __init__(self, v: dict):
        super().__init__()
        self.fc1 = Linear(v["hidden_size"], v["intermediate_size"])
        self.fc2 = Linear(v["intermediate_size"], v["hidden_size"])
        self.tanh_approx = v.get("hidden_act", "gelu") in ("gelu_pytorch_tanh", "gelu_new")

    def forward(self, x):
        return self.fc2(F.gelu(self.fc1(x), approximate="tanh" if self.tanh_approx else "none"))


class _VisionLayer(nn.Module):
    def __init__(self, v: dict, gated: bool):
        super().__init__()
        self.self_attn, self.mlp = _VisionAttention(v), _VisionMLP(v)
        self.input_layernorm = nn.LayerNorm(v["hidden_size"], eps=v.get("norm_eps", 1e-5))
        self.post_attention_layernorm = nn.LayerNorm(v["hidden_size"], eps=v.get("norm_eps", 1e-5))
        self.gated = gated
        if gated:
            self.gate_attn = nn.Parameter(torch.full((1,), math.pi / 4))
            self.gate_ffn = nn.Parameter(torch.full((1,), math.pi / 4))

    def forward(self, x, bias):
        a = self.self_attn(self.input_layernorm(x), bias)
        x = x + (self.gate_attn.tanh() * a if self.gated else a)
        m = self.mlp(self.post_attention_layernorm(x))
        return x + (self.gate_ffn.tanh() * m if self.gated else m)


class _VisionStack(nn.Module):
    def __init__(self, v: dict, n: int, gated: bool):
        super().__init__()
        self.layers = nn.ModuleList(_VisionLayer(v, gated) for _ in range(n))


class MllamaVision(nn.Module):
    """pixel_values [B, images, tiles, C, H, W] -> [B, images, tiles, patches + 1, hidden * (1 + len(intermediate))]."""

    def __init__(self, v: dict):
        super().__init__()
        self.v = v
        D = v["hidden_size"]
        self.patches = (v["image_size"] // v["patch_size"]) ** 2 + 1
        self.patch_embedding = nn.Conv2d(v.get("num_channels", 3), D, v["patch_size"], v["patch_size"], bias=False)
        self.class_embedding = nn.Parameter(torch.randn(D) * D ** -0.5)
        self.gated_positional_embedding = _PositionEmbedding(v)
        self.pre_tile_positional_embedding = _AspectRatioEmbedding(v)
        self.post_tile_positional_embedding = _AspectRatioEmbedding(v)
        self.layernorm_pre, self.layernorm_post = nn.LayerNorm(D), nn.LayerNorm(D)
        self.transformer = _VisionStack(v, v["num_hidden_layers"], False)
        self.global_transformer = _VisionStack(v, v["num_global_layers"], True)
        self.intermediate = list(v["intermediate_layers_indices"])

    @staticmethod
    def padding_bias(tile_mask: torch.Tensor, patches: int, padded: int, dtype) -> torch.Tensor:
        """Additive [N, 1, tiles*padded, tiles*padded] bias. A position is "padding" when its tile is absent or it is one
        of the rows added to round the patch count up to a multiple of 8; a score is pushed to the dtype minimum only
        where BOTH the query and the key are padding (the published model was trained with exactly this mask)."""
        N, tiles = tile_mask.shape
        keep = tile_mask.view(N, tiles, 1).to(dtype).repeat(1, 1, padded)
        if padded > patches:
            keep[:, :, patches:] = 0
        pad = (1 - keep).reshape(N, tiles * padded, 1)
        return (pad @ pad.transpose(1, 2) * torch.finfo(dtype).min)[:, None]

    def forward(self, pixel_values, aspect_ratio_ids, aspect_ratio_mask):
        B, M, Tl, C, Hh, Ww = pixel_values.shape
        N = B * M
        ids = aspect_ratio_ids.reshape(N, -1)
        x = self.patch_embedding(pixel_values.reshape(N * Tl, C, Hh, Ww).to(self.patch_embedding.weight.dtype))
        x = x.flatten(2).transpose(1, 2)
        D = x.shape[-1]
        x = self.pre_tile_positional_embedding(x.reshape(N, Tl, -1, D), ids).reshape(N * Tl, -1, D)
        x = torch.cat((self.class_embedding.expand(N * Tl, 1, D), x), 1)
        P = x.shape[1]
        x = self.layernorm_pre(self.gated_positional_embedding(x.reshape(N, Tl, P, D), ids))
        extra = (8 - P % 8) % 8
        x = F.pad(x, (0, 0, 0, extra))
        bias = self.padding_bias(aspect_ratio_mask.reshape(N, -1), self.patches, P + extra, x.dtype)
        x = x.reshape(N, -1, D)
        taps = []
        for i, layer in enumerate(self.transformer.layers):
            x = layer(x, bias)
            if i in self.intermediate:
                taps.append(x)
        x = self.layernorm_post(x)
        x = self.post_tile_positional_embedding(x.reshape(N, Tl, P + extra, D), ids).reshape(N, -1, D)
        for layer in self.global_transformer.layers:
            x = layer(x, bias)
        x = x.reshape(N, Tl, P + extra, D)[:, :, :P].reshape(B, M, Tl, P, D)
        mid = torch.stack(taps, -1).reshape(N, Tl, P + extra, -1)[:, :, :P].reshape(B, M, Tl, P, -1)
        return torch.cat((x, mid), -1)


# ------------------------------------------------------------------------------------------------ text model
class _RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight, self.eps = nn.Parameter(torch.ones(dim)), eps

    def forward(self, x):
        xf = x.float()
        return self.weight * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype)


class _TextMLP(nn.Module):
    def __init__(self, t: dict):
        super().__init__()
        H, I = t["hidden_size"], t["intermediate_size"]
        self.gate_proj, self.up_proj = Linear(H, I, bias=False), Linear(H, I, bias=False)
        self.down_proj = Linear(I, H, bias=False)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class _Proj(nn.Module):
    def __init__(self, t: dict):
        super().__init__()
        H, self.h, self.hkv = t["hidden_size"], t["num_attention_heads"], t.get("num_key_value_heads") or t["num_attention_heads"]
        self.d = H // self.h
        self.q_proj = Linear(H, self.h * self.d, bias=False)
        self.k_proj = Linear(H, self.hkv * self.d, bias=False)
        self.v_proj = Linear(H, self.hkv * self.d, bias=False)
        self.o_proj = Linear(self.h * self.d, H, bias=False)


class _SelfAttention(_Proj):
    def forward(self, x, rope, mask, cache: Optional[KVCache], idx: int):
        B, T, _ = x.shape
        q = apply_rope(self.q_proj(x).view(B, T, self.h, self.d).transpose(1, 2), *rope, False)
        k = apply_rope(self.k_proj(x).view(B, T, self.hkv, self.d).transpose(1, 2), *rope, False)
        v = self.v_proj(x).view(B, T, self.hkv, self.d).transpose(1, 2)
        if cache is not None:
            k, v = cache.append(idx, k, v)
        y = attend(q, k, v, mask, self.d ** -0.5)
        return self.o_proj(y.transpose(1, 2).reshape(B, T, -1))


class _CrossAttention(_Proj):
    def __init__(self, t: dict):
        super().__init__(t)
        self.q_norm, self.k_norm = _RMSNorm(self.d, t.get("rms_norm_eps", 1e-5)), _RMSNorm(self.d, t.get("rms_norm_eps", 1e-5))

    def forward(self, x, states: Optional[torch.Tensor], bias, cache: Optional[KVCache], idx: int):
        B, T, _ = x.shape
        q = self.q_norm(self.q_proj(x).view(B, T, self.h, self.d).transpose(1, 2))
        if states is not None:
            k = self.k_norm(self.k_proj(states).view(B, -1, self.hkv, self.d).transpose(1, 2))
            v = self.v_proj(states).view(B, -1, self.hkv, self.d).transpose(1, 2)
            if cache is not None:
                cache.state[("cross", idx)] = (k, v)
        else:
            k, v = cache.state[("cross", idx)]
        g = self.h // self.hkv
        if g > 1:
            k, v = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
        y = F.scaled_dot_product_attention(q, k, v, attn_mask=bias)
        return self.o_proj(y.transpose(1, 2).reshape(B, T, -1))


class _SelfLayer(nn.Module):
    cross = False

    def __init__(self, t: dict, idx: int):
        super().__init__()
        self.idx = idx
        self.self_attn, self.mlp = _SelfAttention(t), _TextMLP(t)
        self.input_layernorm = _RMSNorm(t["hidden_size"], t.get("rms_norm_eps", 1e-5))
        self.post_attention_layernorm = _RMSNorm(t["hidden_size"], t.get("rms_norm_eps", 1e-5))

    def forward(self, x, rope, mask, cache):
        x = x + self.self_attn(self.input_layernorm(x), rope, mask, cache, self.idx)
        return x + self.mlp(self.post_attention_layernorm(x))


class _CrossLayer(nn.Module):
    cross = True

    def __init__(self, t: dict, idx: int):
        super().__init__()
        self.idx = idx
        self.cross_attn, self.mlp = _CrossAttention(t), _TextMLP(t)
        self.input_layernorm = _RMSNorm(t["hidden_size"], t.get("rms_norm_eps", 1e-5))
        self.post_attention_layernorm = _RMSNorm(t["hidden_size"], t.get("rms_norm_eps", 1e-5))
        self.cross_attn_attn_gate = nn.Parameter(torch.zeros(1))
        self.cross_attn_mlp_gate = nn.Parameter(torch.zeros(1))

    def forward(self, x, states, bias, row_mask, cache):
        x = x + self.cross_attn_attn_gate.tanh() * self.cross_attn(self.input_layernorm(x), states, bias, cache, self.idx)
        m = self.mlp(self.post_attention_layernorm(x))
        if row_mask is not None:
            m = row_mask[:, 0] * m
        return x + self.cross_attn_mlp_gate.tanh() * m


class MllamaText(nn.Module):
    def __init__(self, t: dict):
        super().__init__()
        self.t = t
        self.cross_layers = set(t.get("cross_attention_layers") or [])
        self.embed_tokens = nn.Embedding(t["vocab_size"] + 8, t["hidden_size"])
        self.layers = nn.ModuleList((_CrossLayer if i in self.cross_layers else _SelfLayer)(t, i)
                                    for i in range(t["num_hidden_layers"]))
        self.norm = _RMSNorm(t["hidden_size"], t.get("rms_norm_eps", 1e-5))
        rp = t.get("rope_parameters") or t.get("rope_scaling") or {}
        theta = float(rp.get("rope_theta", t.get("rope_theta", 500000.0)))
        scaling = rp if rp.get("rope_type", "default") != "default" else None
        inv, _ = rope_inv_freq(t["hidden_size"] // t["num_attention_heads"], theta, scaling, t.get("max_position_embeddings", 131072))
        self.register_buffer("inv_freq", inv, persistent=False)

    def forward(self, input_ids, states, cross_bias, row_mask, cache: Optional[KVCache]):
        B, T = input_ids.shape
        dev = input_ids.device
        past = int(cache.state.get("length", 0)) if cache is not None else 0
        pos = torch.arange(past, past + T, device=dev)
        ang = pos[None, :, None].float() * self.inv_freq[None, None].float()
        rope = (torch.cos(ang).expand(B, -1, -1), torch.sin(ang).expand(B, -1, -1))
        mask = (torch.arange(past + T, device=dev)[None, :] <= pos[:, None])[None, None]
        x = self.embed_tokens(input_ids)
        have_cross = states is not None or (cache is not None and any(isinstance(k, tuple) for k in cache.state))
        for layer in self.layers:
            if layer.cross:
                if have_cross:
                    x = layer(x, states, cross_bias, row_mask, cache)
            else:
                x = layer(x, rope, mask, cache)
        if cache is not None:
            cache.state["length"] = past + T
        return self.norm(x)


class _MllamaBody(nn.Module):
    def __init__(self, config: dict):
        super().__init__()
        v, t = config["vision_config"], config["text_config"]
        self.vision_model = MllamaVision(v)
        self.language_model = MllamaText(t)
        self.multi_modal_projector = Linear(v["vision_output_dim"], t["hidden_size"])


def prepare_cross_mask(cross_attention_mask: torch.Tensor, vision_tokens: int, dtype) -> Tuple[torch.Tensor, torch.Tensor]:
    """[B, T, images, tiles] 0/1 -> additive bias [B, 1, T, images*tiles*vision_tokens] and the per-row flag
    [B, 1, T, 1] (0 for a token that sees no tile at all: its bias row is cleared, so it attends uniformly, and its
    cross-layer MLP branch is zeroed)."""
    B, T = cross_attention_mask.shape[:2]
    m = cross_attention_mask.repeat_interleave(vision_tokens, 3).view(B, T, -1)[:, None].to(dtype)
    lo = torch.finfo(dtype).min
    bias = (1.0 - m).masked_fill((1.0 - m).bool(), lo)
    rows = (bias != lo).any(-1, keepdim=True).to(dtype)
    return bias * rows, rows


class MllamaForConditionalGeneration(nn.Module):
    def __init__(self, config: dict):
        super().__init__()
        self.config = config
        self.model = _MllamaBody(config)
        t = config["text_config"]
        self.lm_head = Linear(t["hidden_size"], t["vocab_size"], bias=False)

    def encode_images(self, pixel_values, aspect_ratio_ids, aspect_ratio_mask) -> torch.Tensor:
        """Projected vision states [B, images*tiles*patches, hidden] for the cross-attention layers."""
        f = self.model.vision_model(pixel_values, aspect_ratio_ids, aspect_ratio_mask)
        H = self.config["text_config"]["hidden_size"]
        return self.model.multi_modal_projector(f).reshape(-1, f.shape[-2], H).reshape(pixel_values.shape[0], -1, H)

    def new_cache(self) -> KVCache:
        return KVCache(self.config["text_config"]["num_hidden_layers"])

    def forward(self, input_ids, pixel_values=None, aspect_ratio_ids=None, aspect_ratio_mask=None,
                cross_attention_mask=None, cache: Optional[KVCache] = None) -> torch.Tensor:
        """``cross_attention_mask`` covers the whole sequence so far ([B, total length, images, tiles]); the rows of the
        tokens in this call are selected from it. Without images and without cached image keys the cross-attention
        layers are skipped (text-only use)."""
        states = None
        if pixel_values is not None:
            states = self.encode_images(pixel_values, aspect_ratio_ids, aspect_ratio_mask)
        bias = rows = None
        if cross_attention_mask is not None:
            dtype = self.model.multi_modal_projector.weight.dtype
            bias, rows = prepare_cross_mask(cross_attention_mask, self.model.vision_model.patches, dtype)
            past = int(cache.state.get("length", 0)) if cache is not None else 0
            sel = slice(past, past + input_ids.shape[1])
            bias, rows = bias[:, :, sel], rows[:, :, sel]
        h = self.model.language_model(input_ids, states, bias, rows, cache)
        return self.lm_head(h)

    @torch.no_grad()
    def generate(self, prompt: List[int], max_new_tokens: int = 16, eos_token_id: Optional[int] = None, **image_inputs):
        """Greedy decoding; image inputs (and a cross-attention mask for the prompt) are given once, later tokens reuse the
        cached cross keys and repeat the last mask row."""
        dev = self.lm_head.weight.device
        cache = self.new_cache()
        ids = torch.tensor([prompt], device=dev)
        cam = image_inputs.pop("cross_attention_mask", None)
        out: List[int] = []
        for step in range(max_new_tokens):
            kw = image_inputs if step == 0 else {}
            if cam is not None and step > 0:
                cam = torch.cat((cam, cam[:, -1:]), 1)
            nxt = int(self.forward(ids, cross_attention_mask=cam, cache=cache, **kw)[0, -1].argmax())
            out.append(nxt)
            if eos_token_id is not None and nxt == eos_token_id:
                break
            ids = torch.tensor([[nxt]], device=dev)
        return out
