"""Vision towers and the vision-language wrapper: Pixtral (ViT with two-dimensional rotary embedding, RMSNorm, gated
MLP), the Qwen2-VL tower (3-D patch embedding, rotary over (row, column) in merge-group order, patch merger), and a
wrapper that projects image features and splices them into the text embeddings of a decoder at the image-token
positions (crates/pmetal-models/src/architectures/{pixtral,qwen2_vl,mllama}.rs). Parameter names follow the Hugging
Face checkpoints of the towers."""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from .fast import Linear

from .generic import Norm


def _rotate_half(x):
    a, b = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-b, a), -1)


def _block_diag_mask(lengths: Sequence[int], device) -> Optional[torch.Tensor]:
    """Attention only inside each image of a packed patch sequence; None for a single image."""
    if len(lengths) <= 1:
        return None
    ids = torch.repeat_interleave(torch.arange(len(lengths), device=device), torch.tensor(list(lengths), device=device))
    return (ids[:, None] == ids[None, :])[None, None]


# ------------------------------------------------------------------------------------------------ Pixtral
class _PixAttention(nn.Module):
    def __init__(self, H, h, d):
        super().__init__()
        self.h, self.d = h, d
        self.q_proj, self.k_proj, self.v_proj = (Linear(H, h * d, bias=False) for _ in range(3))
        self.o_proj = Linear(h * d, H, bias=False)

    def forward(self, x, cos, sin, mask):
        B, T, _ = x.shape
        q, k, v = (f(x).view(B, T, self.h, self.d).transpose(1, 2) for f in (self.q_proj, self.k_proj, self.v_proj))
        q = q * cos + _rotate_half(q) * sin
        k = k * cos + _rotate_half(k) * sin
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
        return self.o_proj(o.transpose(1, 2).reshape(B, T, self.h * self.d))


class _PixMlp(nn.Module):
    def __init__(self, H, I, act):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = Linear(H, I, bias=False), Linear(H, I, bias=False), Linear(I, H, bias=False)
        self.fn = {"gelu": F.gelu, "silu": F.silu}[act]

    def forward(self, x):
        return self.down_proj(self.fn(self.gate_proj(x)) * self.up_proj(x))


class _PixLayer(nn.Module):
    def __init__(self, c):
        super().__init__()
        H = c["hidden_size"]
        d = c.get("head_dim") or H // c["num_attention_heads"]
        self.attention_norm, self.ffn_norm = Norm(H, "rms", 1e-5), Norm(H, "rms", 1e-5)
        self.attention = _PixAttention(H, c["num_attention_heads"], d)
        self.feed_forward = _PixMlp(H, c["intermediate_size"], c.get("hidden_act", "gelu"))

    def forward(self, x, cos, sin, mask):
        x = x + self.attention(self.attention_norm(x), cos, sin, mask)
        return x + self.feed_forward(self.ffn_norm(x))


class _PixTransformer(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.layers = nn.ModuleList([_PixLayer(c) for _ in range(c["num_hidden_layers"])])


class PixtralVision(nn.Module):
    """Images of different sizes are patchified separately, packed into one sequence, and attend only within their own
    patches; rotary frequencies alternate between the row and the column index of a patch."""

    def __init__(self, c: dict):
        super().__init__()
        self.c = c
        H, P = c["hidden_size"], c["patch_size"]
        self.patch_conv = nn.Conv2d(c.get("num_channels", 3), H, P, P, bias=False)
        self.ln_pre = Norm(H, "rms", 1e-5)
        self.transformer = _PixTransformer(c)
        d = c.get("head_dim") or H // c["num_attention_heads"]
        theta = (c.get("rope_parameters") or {}).get("rope_theta", c.get("rope_theta", 10000.0))
        side = c["image_size"] // P
        freqs = 1.0 / (theta ** (torch.arange(0, d, 2).float() / d))
        fh = torch.outer(torch.arange(side).float(), freqs[::2])
        fw = torch.outer(torch.arange(side).float(), freqs[1::2])
        inv = torch.cat((fh[:, None, :].repeat(1, side, 1), fw[None, :, :].repeat(side, 1, 1)), -1).reshape(-1, d // 2)
        self.register_buffer("inv_freq", torch.cat((inv, inv), -1), persistent=False)
        self.side = side

    def forward(self, images: Sequence[torch.Tensor]) -> torch.Tensor:
        """images: list of [C, H, W] tensors (H, W multiples of the patch size). Returns [total_patches, hidden]."""
        embeds, pos, lens = [], [], []
        for img in images:
            e = self.patch_conv(img[None].to(self.patch_conv.weight.dtype))[0]        # [H, h, w]
            hh, ww = e.shape[-2:]
            embeds.append(e.flatten(1).t())
            grid = torch.arange(hh, device=e.device)[:, None] * self.side + torch.arange(ww, device=e.device)[None, :]
            pos.append(grid.reshape(-1))
            lens.append(hh * ww)
        x = self.ln_pre(torch.cat(embeds)[None])
        ang = self.inv_freq[torch.cat(pos)]
        cos, sin = ang.cos()[None, None].to(x.dtype), ang.sin()[None, None].to(x.dtype)
        mask = _block_diag_mask(lens, x.device)
        for layer in self.transformer.layers:
            x = layer(x, cos, sin, mask)
        return x[0]


# ------------------------------------------------------------------------------------------------ Qwen2-VL tower
class _QvAttention(nn.Module):
    def __init__(self, D, h):
        super().__init__()
        self.h = h
        self.qkv, self.proj = Linear(D, 3 * D), Linear(D, D)

    def forward(self, x, cos, sin, mask):
        T, D = x.shape
        q, k, v = self.qkv(x).view(T, 3, self.h, D // self.h).permute(1, 0, 2, 3).unbind(0)      # [T, h, d]
        q = (q.float() * cos + _rotate_half(q.float()) * sin).to(x.dtype)
        k = (k.float() * cos + _rotate_half(k.float()) * sin).to(x.dtype)
        o = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None],
                                           attn_mask=mask)
        return self.proj(o[0].transpose(0, 1).reshape(T, D))


class _QvMlp(nn.Module):
    def __init__(self, D, I, act):
        super().__init__()
        self.fc1, self.fc2 = Linear(D, I), Linear(I, D)
        self.fn = {"quick_gelu": lambda x: x * torch.sigmoid(1.702 * x), "gelu": F.gelu, "silu": F.silu}[act]

    def forward(self, x):
        return self.fc2(self.fn(self.fc1(x)))


class _QvBlock(nn.Module):
    def __init__(self, D, h, I, act):
        super().__init__()
        self.norm1, self.norm2 = nn.LayerNorm(D, eps=1e-6), nn.LayerNorm(D, eps=1e-6)
        self.attn, self.mlp = _QvAttention(D, h), _QvMlp(D, I, act)

    def forward(self, x, cos, sin, mask):
        x = x + self.attn(self.norm1(x), cos, sin, mask)
        return x + self.mlp(self.norm2(x))


class _QvPatchEmbed(nn.Module):
    def __init__(self, C, D, tp, P):
        super().__init__()
        self.shape = (C, tp, P, P)
        self.proj = nn.Conv3d(C, D, (tp, P, P), (tp, P, P), bias=False)

    def forward(self, x):
        return self.proj(x.view(-1, *self.shape).to(self.proj.weight.dtype)).view(-1, self.proj.out_channels)


class _QvMerger(nn.Module):
    def __init__(self, out_dim, D, merge):
        super().__init__()
        self.width = D * merge * merge
        self.ln_q = nn.LayerNorm(D, eps=1e-6)
        self.mlp = nn.Sequential(Linear(self.width, self.width), nn.GELU(), Linear(self.width, out_dim))

    def forward(self, x):
        return self.mlp(self.ln_q(x).view(-1, self.width))


class Qwen2VLVision(nn.Module):
    """Input: flattened patches [n, C * temporal * P * P] in merge-group order plus ``grid_thw`` [(t, h, w)] per image /
    video; output: one feature per ``merge x merge`` group of patches, in the language model's width."""

    def __init__(self, c: dict):
        super().__init__()
        D, h = c["embed_dim"], c["num_heads"]
        self.merge = c.get("spatial_merge_size", 2)
        self.patch_embed = _QvPatchEmbed(c.get("in_channels", c.get("in_chans", 3)), D, c.get("temporal_patch_size", 2), c["patch_size"])
        self.blocks = nn.ModuleList([_QvBlock(D, h, int(D * c.get("mlp_ratio", 4)), c.get("hidden_act", "quick_gelu"))
                                     for _ in range(c["depth"])])
        self.merger = _QvMerger(c["hidden_size"], D, self.merge)
        rd = D // h // 2
        self.register_buffer("inv_freq", 1.0 / (10000.0 ** (torch.arange(0, rd, 2).float() / rd)), persistent=False)

    def _positions(self, grid_thw) -> torch.Tensor:
        m, out = self.merge, []
        for t, h, w in grid_thw:
            hp = torch.arange(h)[:, None].expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            wp = torch.arange(w)[None, :].expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            out.append(torch.stack((hp, wp), -1).repeat(t, 1))
        return torch.cat(out)

    def forward(self, patches: torch.Tensor, grid_thw: Sequence[Sequence[int]]) -> torch.Tensor:
        x = self.patch_embed(patches)
        pos = self._positions(grid_thw).to(x.device)
        freqs = pos[..., None].float() * self.inv_freq                   # [n, 2, rd/2]
        ang = freqs.flatten(1)
        ang = torch.cat((ang, ang), -1)
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        lens = [h * w for t, h, w in grid_thw for _ in range(t)]
        mask = _block_diag_mask(lens, x.device)
        for blk in self.blocks:
            x = blk(x, cos, sin, mask)
        return self.merger(x)


# ------------------------------------------------------------------------------------------------ wrapper
class VisionLanguageModel(nn.Module):
    """Text decoder + vision tower + projector. Image features replace the embeddings of the image placeholder
    tokens (one feature per placeholder, in order)."""

    def __init__(self, decoder: nn.Module, tower: nn.Module, projector: Optional[nn.Module], image_token_id: int):
        super().__init__()
        self.language_model, self.vision_tower, self.multi_modal_projector = decoder, tower, projector
        self.image_token_id = image_token_id

    def embed(self, input_ids: torch.Tensor, image_features: Optional[torch.Tensor]) -> torch.Tensor:
        emb = self.language_model.model.embed_tokens(input_ids)
        if image_features is not None:
            feats = self.multi_modal_projector(image_features) if self.multi_modal_projector is not None else image_features
            where = input_ids == self.image_token_id
            if int(where.sum()) != feats.shape[0]:
                raise ValueError(f"{int(where.sum())} image placeholders but {feats.shape[0]} image features")
            emb = emb.masked_scatter(where[..., None], feats.to(emb.dtype))
        return emb

    def forward(self, input_ids, image_features=None):
        lm = self.language_model
        x = self.embed(input_ids, image_features)
        B, T = input_ids.shape
        pos = torch.arange(T, device=input_ids.device)[None].expand(B, T)
        if lm.c.embed_scale != 1.0:
            x = x * lm.c.embed_scale
        rope = lm._rope(pos)
        for layer in lm.model.layers:
            x = layer(x, rope, pos, None, pos)
        return lm.logits(getattr(lm.model, lm.c.final_norm_name)(x))


class _LlavaProjector(nn.Module):
    def __init__(self, vin, vout, act="gelu", bias=True):
        super().__init__()
        self.linear_1, self.linear_2 = Linear(vin, vout, bias=bias), Linear(vout, vout, bias=bias)
        self.fn = {"gelu": F.gelu, "silu": F.silu}[act]

    def forward(self, x):
        return self.linear_2(self.fn(self.linear_1(x)))


def build_vision_language(config: dict) -> VisionLanguageModel:
    """Pixtral / Llava-style (``vision_config`` + ``text_config`` + MLP projector), Qwen2-VL (tower with merger) and
    mllama (tiled tower + cross-attention decoder, its own class)."""
    from .generic import GenericDecoderLM
    mt = config.get("model_type", "")
    text = config.get("text_config") or {k: v for k, v in config.items() if k != "vision_config"}
    if mt == "qwen2_vl":
        text = dict(text, model_type="qwen2")
        tower = Qwen2VLVision(config["vision_config"])
        return VisionLanguageModel(GenericDecoderLM.from_hf_config(text), tower, None, config.get("image_token_id", 151655))
    if mt == "mllama":
        from .mllama import MllamaForConditionalGeneration
        return MllamaForConditionalGeneration(config)
    vis = config["vision_config"]
    tower = PixtralVision(vis)
    proj = _LlavaProjector(vis["hidden_size"], text["hidden_size"], config.get("projector_hidden_act", "gelu"),
                           config.get("multimodal_projector_bias", True))
    return VisionLanguageModel(GenericDecoderLM.from_hf_config(text), tower, proj, config.get("image_token_index", 10))
