"""Nemotron-H: a stack of single-mixer blocks (Mamba-2 state-space mixer, attention without position encoding, or a
squared-ReLU MLP or mixture of such experts), each ``x + mixer(norm(x))`` (crates/pmetal-models/src/architectures/nemotron_h.rs). Parameter names
follow the Hugging Face checkpoints (``backbone.layers.N.mixer.*``).

The Mamba-2 mixer here is the plain recurrence (one state update per token): per head h with head_dim P and state N,
    S <- exp(dt A_h) S + dt x B^T,   y = S C + D_h x,
after a short causal depthwise convolution over (x, B, C) and followed by a gated group RMSNorm. It is the portable
definition used for loading, evaluation and generation with a per-layer (convolution window, state) cache."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .fast import Linear

from .generic import ArchConfig, KVCache, Norm, attend, build_mask, route


class Mamba2Mixer(nn.Module):
    def __init__(self, c: dict, idx: int):
        super().__init__()
        self.idx = idx
        self.heads, self.hd, self.N = c["mamba_num_heads"], c["mamba_head_dim"], c["ssm_state_size"]
        self.groups, self.kw = c.get("n_groups", 8), c.get("conv_kernel", 4)
        self.inner = self.heads * self.hd
        self.conv_dim = self.inner + 2 * self.groups * self.N
        self.dt_min = c.get("time_step_min", 0.001)
        self.conv1d = nn.Conv1d(self.conv_dim, self.conv_dim, self.kw, groups=self.conv_dim, padding=self.kw - 1,
                                bias=c.get("use_conv_bias", True))
        self.in_proj = Linear(c["hidden_size"], self.inner + self.conv_dim + self.heads, bias=c.get("use_bias", False))
        self.dt_bias = nn.Parameter(torch.ones(self.heads))
        self.A_log = nn.Parameter(torch.log(torch.arange(1, self.heads + 1).float()))
        self.D = nn.Parameter(torch.ones(self.heads))
        self.norm = nn.Module()
        self.norm.weight = nn.Parameter(torch.ones(self.inner))
        self.eps = c.get("layer_norm_epsilon", 1e-5)
        self.out_proj = Linear(self.inner, c["hidden_size"], bias=c.get("use_bias", False))

    def forward(self, x, cache: Optional[KVCache]):
        B, T, _ = x.shape
        z, xbc, dt = self.in_proj(x).split((self.inner, self.conv_dim, self.heads), -1)
        st = cache.state.get(self.idx) if cache is not None else None
        xbc = xbc.transpose(1, 2)
        prev = st[0] if st is not None else xbc.new_zeros(B, self.conv_dim, self.kw - 1)
        full = torch.cat((prev, xbc), -1)
        conv = F.silu(F.conv1d(full, self.conv1d.weight, self.conv1d.bias, groups=self.conv_dim))[:, :, -T:].transpose(1, 2)
        xs, Bm, Cm = conv.split((self.inner, self.groups * self.N, self.groups * self.N), -1)
        xs = xs.reshape(B, T, self.heads, self.hd).float()
        rep = self.heads // self.groups
        Bm = Bm.reshape(B, T, self.groups, self.N).float().repeat_interleave(rep, 2)
        Cm = Cm.reshape(B, T, self.groups, self.N).float().repeat_interleave(rep, 2)
        dt = torch.clamp(F.softplus(dt.float() + self.dt_bias), min=self.dt_min)              # [B, T, heads]
        decay = torch.exp(dt * (-torch.exp(self.A_log.float())))                               # [B, T, heads]
        S = st[1].float() if st is not None else xs.new_zeros(B, self.heads, self.hd, self.N)
        ys = []
        for t in range(T):
            S = S * decay[:, t, :, None, None] + (dt[:, t, :, None] * xs[:, t])[..., None] * Bm[:, t, :, None, :]
            ys.append(torch.einsum("bhpn,bhn->bhp", S, Cm[:, t]))
        y = torch.stack(ys, 1) + xs * self.D[None, None, :, None]
        if cache is not None:
            cache.state[self.idx] = (full[:, :, -(self.kw - 1):].detach(), S)
        y = y.reshape(B, T, self.inner) * F.silu(z.float())                                    # gate, then group norm
        g = y.view(B, T, self.groups, self.inner // self.groups)
        y = (g * torch.rsqrt(g.pow(2).mean(-1, keepdim=True) + self.eps)).view(B, T, self.inner)
        return self.out_proj((self.norm.weight * y.to(x.dtype)))


class _Attention(nn.Module):
    def __init__(self, c: dict, idx: int):
        super().__init__()
        self.idx = idx
        H, self.h, self.hkv = c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"]
        self.d = c.get("head_dim") or H // self.h
        bias = c.get("attention_bias", False)
        self.q_proj, self.k_proj = Linear(H, self.h * self.d, bias=bias), Linear(H, self.hkv * self.d, bias=bias)
        self.v_proj, self.o_proj = Linear(H, self.hkv * self.d, bias=bias), Linear(self.h * self.d, H, bias=bias)

    def forward(self, x, cache, positions, k_positions):
        B, T, _ = x.shape
        q = self.q_proj(x).view(B, T, self.h, self.d).transpose(1, 2)
        k = self.k_proj(x).view(B, T, self.hkv, self.d).transpose(1, 2)
        v = self.v_proj(x).view(B, T, self.hkv, self.d).transpose(1, 2)
        if cache is not None:
            k, v = cache.append(self.idx, k, v)
        o = attend(q, k, v, build_mask("full", positions, k_positions, 0, 0), self.d ** -0.5)
        return self.o_proj(o.transpose(1, 2).reshape(B, T, self.h * self.d))


class _Mlp(nn.Module):
    def __init__(self, c: dict):
        super().__init__()
        bias = c.get("mlp_bias", False)
        self.up_proj = Linear(c["hidden_size"], c["intermediate_size"], bias=bias)
        self.down_proj = Linear(c["intermediate_size"], c["hidden_size"], bias=bias)

    def forward(self, x):
        return self.down_proj(F.relu(self.up_proj(x)).square())


class _Experts(nn.Module):
    def __init__(self, E, I, inp):
        super().__init__()
        self.up_proj = nn.Parameter(torch.empty(E, I, inp).normal_(std=0.02))
        self.down_proj = nn.Parameter(torch.empty(E, inp, I).normal_(std=0.02))


class _Gate(nn.Module):
    def __init__(self, E, H):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(E, H).normal_(std=0.02))
        self.register_buffer("e_score_correction_bias", torch.zeros(E))


class _Moe(nn.Module):
    """Routed squared-ReLU experts (sigmoid scores, group-limited top-k with a selection bias, as DeepSeek-V3) plus a
    shared expert; optionally the routed path runs in a smaller latent width."""

    def __init__(self, c: dict):
        super().__init__()
        H, E = c["hidden_size"], c["n_routed_experts"]
        latent = c.get("moe_latent_size")
        self.rc = ArchConfig(num_experts=E, top_k=c["num_experts_per_tok"], router="sigmoid_group",
                             norm_topk_prob=bool(c.get("norm_topk_prob", True)),
                             routed_scale=float(c.get("routed_scaling_factor", 1.0)), n_group=c.get("n_group") or 1,
                             topk_group=c.get("topk_group") or 1, group_score="top2sum")
        self.experts = _Experts(E, c["moe_intermediate_size"], latent or H)
        self.gate = _Gate(E, H)
        self.shared_experts = _Mlp(dict(c, intermediate_size=c["moe_shared_expert_intermediate_size"]))
        if latent:
            bias = c.get("mlp_bias", False)
            self.fc1_latent_proj, self.fc2_latent_proj = Linear(H, latent, bias=bias), Linear(latent, H, bias=bias)
        self.latent = bool(latent)

    def forward(self, x):
        shape = x.shape
        xf = x.reshape(-1, shape[-1])
        w, idx = route(self.rc, F.linear(xf.float(), self.gate.weight.float()), self.gate.e_score_correction_bias)
        hin = self.fc1_latent_proj(xf) if self.latent else xf
        out = torch.zeros_like(hin, dtype=torch.float32)
        for e in idx.unique().tolist():
            tok, slot = (idx == e).nonzero(as_tuple=True)
            y = F.relu(hin[tok] @ self.experts.up_proj[e].t()).square() @ self.experts.down_proj[e].t()
            out.index_add_(0, tok, y.float() * w[tok, slot, None])
        out = out.to(x.dtype)
        if self.latent:
            out = self.fc2_latent_proj(out)
        return (out + self.shared_experts(xf)).view(shape)


class _Block(nn.Module):
    def __init__(self, c: dict, idx: int, kind: str):
        super().__init__()
        self.kind = kind
        self.norm = Norm(c["hidden_size"], "rms", c.get("layer_norm_epsilon", 1e-5))
        if kind == "mamba":
            self.mixer = Mamba2Mixer(c, idx)
        elif kind == "attention":
            self.mixer = _Attention(c, idx)
        elif kind == "mlp":
            self.mixer = _Mlp(c)
        elif kind == "moe":
            self.mixer = _Moe(c)
        else:
            raise NotImplementedError(f"Nemotron-H block type {kind!r}")

    def forward(self, x, cache, positions, k_positions):
        n = self.norm(x)
        if self.kind == "mamba":
            return x + self.mixer(n, cache)
        if self.kind == "attention":
            return x + self.mixer(n, cache, positions, k_positions)
        return x + self.mixer(n)


class _Backbone(nn.Module):
    def __init__(self, c: dict, kinds: List[str]):
        super().__init__()
        self.embeddings = nn.Embedding(c["vocab_size"], c["hidden_size"])
        self.layers = nn.ModuleList([_Block(c, i, k) for i, k in enumerate(kinds)])
        self.norm_f = Norm(c["hidden_size"], "rms", c.get("layer_norm_epsilon", 1e-5))


def block_types(cfg: dict) -> List[str]:
    kinds = cfg.get("layers_block_type") or cfg.get("layer_types")
    if kinds:
        return list(kinds)
    pattern = cfg.get("hybrid_override_pattern", "")
    table = {"M": "mamba", "*": "attention", "-": "mlp", "E": "moe"}
    return [table[ch] for ch in pattern]


class NemotronHLM(nn.Module):
    def __init__(self, cfg: dict):
        super().__init__()
        self.cfg = cfg
        self.kinds = block_types(cfg)
        self.backbone = _Backbone(cfg, self.kinds)
        self.lm_head = Linear(cfg["hidden_size"], cfg["vocab_size"], bias=False)

    def new_cache(self) -> KVCache:
        return KVCache(len(self.kinds))

    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor], strict: bool = True):
        """Checkpoints name the stack either ``backbone.`` (original release) or ``model.``; both load."""
        sd = {("backbone." + k[len("model."):] if k.startswith("model.") else k): v for k, v in sd.items()}
        return self.load_state_dict(sd, strict=strict)

    def forward(self, input_ids, cache: Optional[KVCache] = None) -> torch.Tensor:
        if input_ids.dim() == 1:
            input_ids = input_ids[None]
        B, T = input_ids.shape
        past = int(cache.state.get("length", 0)) if cache is not None else 0
        positions = torch.arange(past, past + T, device=input_ids.device)[None].expand(B, T)
        k_positions = torch.arange(0, past + T, device=input_ids.device)[None].expand(B, past + T)
        x = self.backbone.embeddings(input_ids)
        for layer in self.backbone.layers:
            x = layer(x, cache, positions, k_positions if cache is not None else positions)
        if cache is not None:
            cache.state["length"] = past + T
        return self.lm_head(self.backbone.norm_f(x))

    @torch.no_grad()
    def generate(self, prompt: List[int], max_new_tokens: int = 32) -> List[int]:
        cache = self.new_cache()
        ids = torch.tensor([prompt], device=self.lm_head.weight.device)
        out: List[int] = []
        for _ in range(max_new_tokens):
            nxt = int(self.forward(ids, cache)[0, -1].argmax())
            out.append(nxt)
            ids = torch.tensor([[nxt]], device=ids.device)
        return out
