"""FLUX rectified-flow transformer and the latent autoencoder (crates/pmetal-models/src/architectures/{flux,vae}.rs).

``FluxTransformer``: image latents (packed 2x2 patches) and text tokens are embedded into one width; ``num_layers``
double-stream blocks keep separate weights for the two streams but attend jointly, ``num_single_layers`` single-stream
blocks run on the concatenation with a fused attention + MLP projection. Every block is modulated by the pooled
conditioning vector (timestep, optional guidance, pooled text) through adaptive LayerNorm with gates; positions enter
through a rotary embedding over (index, row, column) axes. Parameter names follow the diffusers checkpoints
(``transformer_blocks.N.attn.to_q`` ...). ``AutoencoderKL`` is the convolutional VAE that maps images to 16-channel
latents and back. ``flow_match_sample`` is the Euler sampler over the flow's time grid."""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .fast import Linear


# ------------------------------------------------------------------------------------------------ embeddings
def timestep_embedding(t: torch.Tensor, dim: int = 256, max_period: float = 10000.0) -> torch.Tensor:
    """Sinusoidal features [cos | sin] of ``t`` (already scaled to [0, 1000])."""
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t.float()[:, None] * freqs[None]
    return torch.cat((torch.cos(args), torch.sin(args)), -1)


class _MlpEmbedder(nn.Module):
    def __init__(self, din, dout):
        super().__init__()
        self.linear_1, self.linear_2 = Linear(din, dout), Linear(dout, dout)

    def forward(self, x):
        return self.linear_2(F.silu(self.linear_1(x)))


class _TimeTextEmbed(nn.Module):
    def __init__(self, dim, pooled_dim, guidance: bool):
        super().__init__()
        self.timestep_embedder = _MlpEmbedder(256, dim)
        if guidance:
            self.guidance_embedder = _MlpEmbedder(256, dim)
        self.text_embedder = _MlpEmbedder(pooled_dim, dim)
        self.guidance = guidance

    def forward(self, t, guidance, pooled):
        e = self.timestep_embedder(timestep_embedding(t).to(pooled.dtype))
        if self.guidance:
            e = e + self.guidance_embedder(timestep_embedding(guidance).to(pooled.dtype))
        return e + self.text_embedder(pooled)


def rope_nd(ids: torch.Tensor, axes_dim: Sequence[int], theta: float = 10000.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """ids [T, n_axes] -> (cos, sin) [T, sum(axes_dim) / 2]: each axis rotates its own slice of the head dimension."""
    cos, sin = [], []
    for a, d in enumerate(axes_dim):
        freqs = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32, device=ids.device) / d))
        ang = ids[:, a].float()[:, None] * freqs[None]
        cos.append(ang.cos())
        sin.append(ang.sin())
    return torch.cat(cos, -1), torch.cat(sin, -1)


def _apply_rope(x, cos, sin):
    """x [B, h, T, d] with interleaved pairs (2i, 2i+1)."""
    a, b = x.float()[..., 0::2], x.float()[..., 1::2]
    return torch.stack((a * cos - b * sin, a * sin + b * cos), -1).flatten(-2).to(x.dtype)


class _RmsNorm(nn.Module):
    def __init__(self, d, eps=1e-6):
        super().__init__()
        self.weight, self.eps = nn.Parameter(torch.ones(d)), eps

    def forward(self, x):
        return (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


class _AdaNorm(nn.Module):
    """LayerNorm without affine parameters, scaled and shifted by projections of the conditioning vector; ``n`` chunks
    (shift, scale, gate per sub-layer)."""

    def __init__(self, dim, n):
        super().__init__()
        self.linear = Linear(dim, n * dim)
        self.n = n

    def forward(self, x, emb):
        parts = self.linear(F.silu(emb))[:, None].chunk(self.n, -1)
        return F.layer_norm(x, x.shape[-1:], eps=1e-6) * (1 + parts[1]) + parts[0], parts[2:]


class _FeedForward(nn.Module):
    def __init__(self, dim):
        super().__init__()
        proj = nn.Module()
        proj.proj = Linear(dim, 4 * dim)
        self.net = nn.ModuleList([proj, nn.Identity(), Linear(4 * dim, dim)])

    def forward(self, x):
        return self.net[2](F.gelu(self.net[0].proj(x), approximate="tanh"))


class _JointAttention(nn.Module):
    def __init__(self, dim, heads, joint: bool):
        super().__init__()
        self.h, self.joint = heads, joint
        d = dim // heads
        self.to_q, self.to_k, self.to_v = Linear(dim, dim), Linear(dim, dim), Linear(dim, dim)
        self.norm_q, self.norm_k = _RmsNorm(d), _RmsNorm(d)
        if joint:
            self.add_q_proj, self.add_k_proj, self.add_v_proj = Linear(dim, dim), Linear(dim, dim), Linear(dim, dim)
            self.norm_added_q, self.norm_added_k = _RmsNorm(d), _RmsNorm(d)
            self.to_out = nn.ModuleList([Linear(dim, dim), nn.Identity()])
            self.to_add_out = Linear(dim, dim)

    def _split(self, x):
        B, T, D = x.shape
        return x.view(B, T, self.h, D // self.h).transpose(1, 2)

    def forward(self, x, ctx, cos, sin):
        q, k, v = self.norm_q(self._split(self.to_q(x))), self.norm_k(self._split(self.to_k(x))), self._split(self.to_v(x))
        if self.joint:
            cq = self.norm_added_q(self._split(self.add_q_proj(ctx)))
            ck = self.norm_added_k(self._split(self.add_k_proj(ctx)))
            cv = self._split(self.add_v_proj(ctx))
            q, k, v = torch.cat((cq, q), 2), torch.cat((ck, k), 2), torch.cat((cv, v), 2)      # text tokens first
        q, k = _apply_rope(q, cos, sin), _apply_rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).flatten(2)
        if self.joint:
            n = ctx.shape[1]
            return self.to_out[0](o[:, n:]), self.to_add_out(o[:, :n])
        return o


class _DoubleBlock(nn.Module):
    def __init__(self, dim, heads):
        super().__init__()
        self.norm1, self.norm1_context = _AdaNorm(dim, 6), _AdaNorm(dim, 6)
        self.attn = _JointAttention(dim, heads, True)
        self.ff, self.ff_context = _FeedForward(dim), _FeedForward(dim)

    def forward(self, x, ctx, emb, cos, sin):
        nx, (gate_a, shift_m, scale_m, gate_m) = self.norm1(x, emb)
        nc, (cgate_a, cshift_m, cscale_m, cgate_m) = self.norm1_context(ctx, emb)
        ax, ac = self.attn(nx, nc, cos, sin)
        x = x + gate_a * ax
        x = x + gate_m * self.ff(F.layer_norm(x, x.shape[-1:], eps=1e-6) * (1 + scale_m) + shift_m)
        ctx = ctx + cgate_a * ac
        ctx = ctx + cgate_m * self.ff_context(F.layer_norm(ctx, ctx.shape[-1:], eps=1e-6) * (1 + cscale_m) + cshift_m)
        return x, ctx


class _SingleBlock(nn.Module):
    def __init__(self, dim, heads):
        super().__init__()
        self.norm = _AdaNorm(dim, 3)
        self.proj_mlp = Linear(dim, 4 * dim)
        self.proj_out = Linear(5 * dim, dim)
        self.attn = _JointAttention(dim, heads, False)

    def forward(self, x, emb, cos, sin):
        n, (gate,) = self.norm(x, emb)
        a = self.attn(n, None, cos, sin)
        return x + gate * self.proj_out(torch.cat((a, F.gelu(self.proj_mlp(n), approximate="tanh")), -1))


class _AdaNormOut(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.linear = Linear(dim, 2 * dim)

    def forward(self, x, emb):
        scale, shift = self.linear(F.silu(emb))[:, None].chunk(2, -1)
        return F.layer_norm(x, x.shape[-1:], eps=1e-6) * (1 + scale) + shift


class FluxTransformer(nn.Module):
    def __init__(self, cfg: dict):
        super().__init__()
        self.cfg = cfg
        heads, hd = cfg.get("num_attention_heads", 24), cfg.get("attention_head_dim", 128)
        dim = heads * hd
        self.axes_dim = list(cfg.get("axes_dims_rope", (16, 56, 56)))
        assert sum(self.axes_dim) == hd
        cin = cfg.get("in_channels", 64)
        self.x_embedder = Linear(cin, dim)
        self.context_embedder = Linear(cfg.get("joint_attention_dim", 4096), dim)
        self.time_text_embed = _TimeTextEmbed(dim, cfg.get("pooled_projection_dim", 768), bool(cfg.get("guidance_embeds", False)))
        self.transformer_blocks = nn.ModuleList([_DoubleBlock(dim, heads) for _ in range(cfg.get("num_layers", 19))])
        self.single_transformer_blocks = nn.ModuleList([_SingleBlock(dim, heads) for _ in range(cfg.get("num_single_layers", 38))])
        self.norm_out = _AdaNormOut(dim)
        self.proj_out = Linear(dim, cfg.get("out_channels") or cin)

    def forward(self, latents, text, pooled, timestep, img_ids, txt_ids, guidance: Optional[torch.Tensor] = None):
        """latents [B, T_img, C_in] (packed patches), text [B, T_txt, D_txt], pooled [B, D_pool], timestep [B] in [0, 1],
        img_ids [T_img, 3], txt_ids [T_txt, 3]. Returns the predicted velocity [B, T_img, C_out]."""
        x, ctx = self.x_embedder(latents), self.context_embedder(text)
        g = guidance * 1000.0 if guidance is not None else torch.zeros_like(timestep)
        emb = self.time_text_embed(timestep * 1000.0, g, pooled)
        cos, sin = rope_nd(torch.cat((txt_ids, img_ids)), self.axes_dim, self.cfg.get("rope_theta", 10000.0))
        for blk in self.transformer_blocks:
            x, ctx = blk(x, ctx, emb, cos, sin)
        n = ctx.shape[1]
        h = torch.cat((ctx, x), 1)
        for blk in self.single_transformer_blocks:
            h = blk(h, emb, cos, sin)
        return self.proj_out(self.norm_out(h[:, n:], emb))


def pack_latents(z: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """[B, C, H, W] -> packed 2x2 patches [B, H/2 * W/2, 4 C] and their (0, row, column) ids."""
    B, C, H, W = z.shape
    p = z.view(B, C, H // 2, 2, W // 2, 2).permute(0, 2, 4, 1, 3, 5).reshape(B, (H // 2) * (W // 2), C * 4)
    ids = torch.zeros(H // 2, W // 2, 3, device=z.device)
    ids[..., 1] = torch.arange(H // 2, device=z.device)[:, None]
    ids[..., 2] = torch.arange(W // 2, device=z.device)[None, :]
    return p, ids.view(-1, 3)


def unpack_latents(p: torch.Tensor, H: int, W: int) -> torch.Tensor:
    B, _, D = p.shape
    C = D // 4
    return p.view(B, H // 2, W // 2, C, 2, 2).permute(0, 3, 1, 4, 2, 5).reshape(B, C, H, W)


def flow_sigmas(steps: int, shift: float = 1.0) -> torch.Tensor:
    """Time grid 1 -> 0 with the resolution-dependent shift s: sigma' = s sigma / (1 + (s - 1) sigma)."""
    s = torch.linspace(1.0, 0.0, steps + 1)
    return shift * s / (1 + (shift - 1) * s)


@torch.no_grad()
def flow_match_sample(model: FluxTransformer, noise: torch.Tensor, text, pooled, steps: int = 4, shift: float = 1.0,
                      guidance: Optional[float] = None) -> torch.Tensor:
    """Euler integration of dx/dt = v(x, t) from pure noise [B, C, H, W] at t = 1 to the latent at t = 0."""
    B, C, H, W = noise.shape
    x, ids = pack_latents(noise)
    txt_ids = torch.zeros(text.shape[1], 3, device=noise.device)
    sig = flow_sigmas(steps, shift).to(noise.device)
    g = None if guidance is None else torch.full((B,), guidance, device=noise.device)
    for i in range(steps):
        t = sig[i].expand(B)
        v = model(x, text, pooled, t, ids, txt_ids, g)
        x = x + (sig[i + 1] - sig[i]) * v
    return unpack_latents(x, H, W)


# ------------------------------------------------------------------------------------------------ autoencoder
class _ResBlock(nn.Module):
    def __init__(self, cin, cout, groups=32):
        super().__init__()
        self.norm1, self.conv1 = nn.GroupNorm(groups, cin, eps=1e-6), nn.Conv2d(cin, cout, 3, padding=1)
        self.norm2, self.conv2 = nn.GroupNorm(groups, cout, eps=1e-6), nn.Conv2d(cout, cout, 3, padding=1)
        if cin != cout:
            self.conv_shortcut = nn.Conv2d(cin, cout, 1)

    def forward(self, x):
        h = self.conv1(F.silu(self.norm1(x)))
        h = self.conv2(F.silu(self.norm2(h)))
        return (self.conv_shortcut(x) if hasattr(self, "conv_shortcut") else x) + h


class _VaeAttention(nn.Module):
    def __init__(self, c, groups=32):
        super().__init__()
        self.group_norm = nn.GroupNorm(groups, c, eps=1e-6)
        self.to_q, self.to_k, self.to_v = Linear(c, c), Linear(c, c), Linear(c, c)
        self.to_out = nn.ModuleList([Linear(c, c), nn.Identity()])

    def forward(self, x):
        B, C, H, W = x.shape
        h = self.group_norm(x).flatten(2).transpose(1, 2)
        o = F.scaled_dot_product_attention(self.to_q(h)[:, None], self.to_k(h)[:, None], self.to_v(h)[:, None])[:, 0]
        return x + self.to_out[0](o).transpose(1, 2).view(B, C, H, W)


class _Mid(nn.Module):
    def __init__(self, c, groups):
        super().__init__()
        self.resnets = nn.ModuleList([_ResBlock(c, c, groups), _ResBlock(c, c, groups)])
        self.attentions = nn.ModuleList([_VaeAttention(c, groups)])

    def forward(self, x):
        return self.resnets[1](self.attentions[0](self.resnets[0](x)))


class _Down(nn.Module):
    def __init__(self, cin, cout, n, down, groups):
        super().__init__()
        self.resnets = nn.ModuleList([_ResBlock(cin if i == 0 else cout, cout, groups) for i in range(n)])
        if down:
            ds = nn.Module()
            ds.conv = nn.Conv2d(cout, cout, 3, stride=2)
            self.downsamplers = nn.ModuleList([ds])

    def forward(self, x):
        for r in self.resnets:
            x = r(x)
        if hasattr(self, "downsamplers"):
            x = self.downsamplers[0].conv(F.pad(x, (0, 1, 0, 1)))
        return x


class _Up(nn.Module):
    def __init__(self, cin, cout, n, up, groups):
        super().__init__()
        self.resnets = nn.ModuleList([_ResBlock(cin if i == 0 else cout, cout, groups) for i in range(n)])
        if up:
            us = nn.Module()
            us.conv = nn.Conv2d(cout, cout, 3, padding=1)
            self.upsamplers = nn.ModuleList([us])

    def forward(self, x):
        for r in self.resnets:
            x = r(x)
        if hasattr(self, "upsamplers"):
            x = self.upsamplers[0].conv(F.interpolate(x, scale_factor=2.0, mode="nearest"))
        return x


class _Encoder(nn.Module):
    def __init__(self, cin, chans, layers, latent, groups):
        super().__init__()
        self.conv_in = nn.Conv2d(cin, chans[0], 3, padding=1)
        self.down_blocks = nn.ModuleList([_Down(chans[max(i - 1, 0)], c, layers, i < len(chans) - 1, groups)
                                          for i, c in enumerate(chans)])
        self.mid_block = _Mid(chans[-1], groups)
        self.conv_norm_out, self.conv_out = nn.GroupNorm(groups, chans[-1], eps=1e-6), nn.Conv2d(chans[-1], 2 * latent, 3, padding=1)

    def forward(self, x):
        x = self.conv_in(x)
        for b in self.down_blocks:
            x = b(x)
        return self.conv_out(F.silu(self.conv_norm_out(self.mid_block(x))))


class _Decoder(nn.Module):
    def __init__(self, cout, chans, layers, latent, groups):
        super().__init__()
        rev = list(reversed(chans))
        self.conv_in = nn.Conv2d(latent, rev[0], 3, padding=1)
        self.mid_block = _Mid(rev[0], groups)
        self.up_blocks = nn.ModuleList([_Up(rev[max(i - 1, 0)], c, layers + 1, i < len(rev) - 1, groups)
                                        for i, c in enumerate(rev)])
        self.conv_norm_out, self.conv_out = nn.GroupNorm(groups, rev[-1], eps=1e-6), nn.Conv2d(rev[-1], cout, 3, padding=1)

    def forward(self, z):
        x = self.mid_block(self.conv_in(z))
        for b in self.up_blocks:
            x = b(x)
        return self.conv_out(F.silu(self.conv_norm_out(x)))


class AutoencoderKL(nn.Module):
    """Convolutional variational autoencoder: ``encode`` -> (mean, log-variance) of the latent, ``decode`` -> image.
    Latents are stored as ``(z - shift_factor) * scaling_factor``."""

    def __init__(self, cfg: dict):
        super().__init__()
        chans = list(cfg.get("block_out_channels", (128, 256, 512, 512)))
        latent, groups = cfg.get("latent_channels", 16), cfg.get("norm_num_groups", 32)
        self.encoder = _Encoder(cfg.get("in_channels", 3), chans, cfg.get("layers_per_block", 2), latent, groups)
        self.decoder = _Decoder(cfg.get("out_channels", 3), chans, cfg.get("layers_per_block", 2), latent, groups)
        self.scaling, self.shift = cfg.get("scaling_factor", 0.3611), cfg.get("shift_factor", 0.1159) or 0.0
        if cfg.get("use_quant_conv", False):
            self.quant_conv, self.post_quant_conv = nn.Conv2d(2 * latent, 2 * latent, 1), nn.Conv2d(latent, latent, 1)

    def encode(self, x, sample: bool = False, generator=None):
        h = self.encoder(x)
        if hasattr(self, "quant_conv"):
            h = self.quant_conv(h)
        mean, logvar = h.chunk(2, 1)
        z = mean + torch.exp(0.5 * logvar.clamp(-30, 20)) * torch.randn(mean.shape, generator=generator, device=mean.device) \
            if sample else mean
        return (z - self.shift) * self.scaling

    def decode(self, z):
        z = z / self.scaling + self.shift
        if hasattr(self, "post_quant_conv"):
            z = self.post_quant_conv(z)
        return self.decoder(z)
