"""Encoder and encoder-decoder families: BERT-style text encoders (embedding models), T5, CLIP and Whisper.

The reference carries one Rust module per family (crates/pmetal-models/src/architectures/{bert,t5,clip,whisper}.rs) plus
sentence pooling (crates/pmetal-models/src/pooling.rs). These are the portable PyTorch counterparts with the parameter
names of the Hugging Face checkpoints, so a checkpoint's state dict loads without renaming. Attention goes through
``scaled_dot_product_attention`` (flash kernels on GPU); nothing here is on the training benchmark's hot path."""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .fast import Linear


def _act(name: str):
    return {"gelu": F.gelu, "relu": F.relu, "silu": F.silu, "gelu_new": lambda x: F.gelu(x, approximate="tanh"),
            "quick_gelu": lambda x: x * torch.sigmoid(1.702 * x), "gelu_pytorch_tanh": lambda x: F.gelu(x, approximate="tanh")}[name]


def _heads(x: torch.Tensor, h: int) -> torch.Tensor:
    B, T, D = x.shape
    return x.view(B, T, h, D // h).transpose(1, 2)


def _merge(x: torch.Tensor) -> torch.Tensor:
    B, h, T, d = x.shape
    return x.transpose(1, 2).reshape(B, T, h * d)


# ------------------------------------------------------------------------------------------------ BERT
class _BertSelf(nn.Module):
    def __init__(self, H, h):
        super().__init__()
        self.h = h
        self.query, self.key, self.value = Linear(H, H), Linear(H, H), Linear(H, H)

    def forward(self, x, mask):
        q, k, v = (_heads(f(x), self.h) for f in (self.query, self.key, self.value))
        return _merge(F.scaled_dot_product_attention(q, k, v, attn_mask=mask))


class _BertOut(nn.Module):
    def __init__(self, inp, H, eps):
        super().__init__()
        self.dense = Linear(inp, H)
        self.LayerNorm = nn.LayerNorm(H, eps=eps)

    def forward(self, x, residual):
        return self.LayerNorm(self.dense(x) + residual)


class _BertAttention(nn.Module):
    def __init__(self, H, h, eps):
        super().__init__()
        self.self = _BertSelf(H, h)
        self.output = _BertOut(H, H, eps)

    def forward(self, x, mask):
        return self.output(self.self(x, mask), x)


class _BertIntermediate(nn.Module):
    def __init__(self, H, I):
        super().__init__()
        self.dense = Linear(H, I)


class _BertLayer(nn.Module):
    def __init__(self, H, h, I, eps, act):
        super().__init__()
        self.attention = _BertAttention(H, h, eps)
        self.intermediate = _BertIntermediate(H, I)
        self.output = _BertOut(I, H, eps)
        self.fn = _act(act)

    def forward(self, x, mask):
        x = self.attention(x, mask)
        return self.output(self.fn(self.intermediate.dense(x)), x)


class _BertEmbeddings(nn.Module):
    def __init__(self, V, H, P, types, eps, pad_offset):
        super().__init__()
        self.word_embeddings = nn.Embedding(V, H)
        self.position_embeddings = nn.Embedding(P, H)
        self.token_type_embeddings = nn.Embedding(types, H)
        self.LayerNorm = nn.LayerNorm(H, eps=eps)
        self.pad_offset = pad_offset

    def forward(self, ids, type_ids, mask):
        B, T = ids.shape
        if self.pad_offset:      # RoBERTa: positions count real tokens and start after the padding index
            pos = torch.cumsum(mask.long(), 1) * mask.long() + self.pad_offset
        else:
            pos = torch.arange(T, device=ids.device)[None].expand(B, T)
        x = self.word_embeddings(ids) + self.position_embeddings(pos) + self.token_type_embeddings(type_ids)
        return self.LayerNorm(x)


class _BertEncoder(nn.Module):
    def __init__(self, n, *a):
        super().__init__()
        self.layer = nn.ModuleList([_BertLayer(*a) for _ in range(n)])


class _BertPooler(nn.Module):
    def __init__(self, H):
        super().__init__()
        self.dense = Linear(H, H)


class BertModel(nn.Module):
    """BERT / RoBERTa / XLM-R encoder with the sentence pooling modes used for embedding models
    (crates/pmetal-models/src/architectures/bert.rs, crates/pmetal-models/src/pooling.rs)."""

    def __init__(self, cfg: dict):
        super().__init__()
        H, h = cfg["hidden_size"], cfg["num_attention_heads"]
        eps = cfg.get("layer_norm_eps", 1e-12)
        roberta = cfg.get("model_type", "bert") in ("roberta", "xlm-roberta", "xlm_roberta")
        self.embeddings = _BertEmbeddings(cfg["vocab_size"], H, cfg.get("max_position_embeddings", 512),
                                          cfg.get("type_vocab_size", 2), eps, cfg.get("pad_token_id", 1) if roberta else 0)
        self.encoder = _BertEncoder(cfg["num_hidden_layers"], H, h, cfg["intermediate_size"], eps, cfg.get("hidden_act", "gelu"))
        self.pooler = _BertPooler(H)

    def forward(self, input_ids, attention_mask: Optional[torch.Tensor] = None, token_type_ids=None) -> torch.Tensor:
        if attention_mask is None:
            attention_mask = torch.ones_like(input_ids)
        if token_type_ids is None:
            token_type_ids = torch.zeros_like(input_ids)
        x = self.embeddings(input_ids, token_type_ids, attention_mask)
        mask = attention_mask[:, None, None, :].bool()
        for layer in self.encoder.layer:
            x = layer(x, mask)
        return x

    def pool(self, hidden: torch.Tensor, attention_mask: torch.Tensor, mode: str = "mean", normalize: bool = True):
        m = attention_mask.to(hidden.dtype)[..., None]
        if mode == "cls":
            out = hidden[:, 0]
        elif mode == "pooler":
            out = torch.tanh(self.pooler.dense(hidden[:, 0]))
        elif mode == "max":
            out = hidden.masked_fill(m == 0, float("-inf")).max(1)[0]
        elif mode == "last":
            idx = attention_mask.long().sum(1) - 1
            out = hidden[torch.arange(hidden.shape[0], device=hidden.device), idx]
        else:
            out = (hidden * m).sum(1) / m.sum(1).clamp(min=1e-9)
        return F.normalize(out, dim=-1) if normalize else out


# ------------------------------------------------------------------------------------------------ T5
class _T5Norm(nn.Module):
    def __init__(self, d, eps):
        super().__init__()
        self.weight, self.eps = nn.Parameter(torch.ones(d)), eps

    def forward(self, x):
        v = x.float().pow(2).mean(-1, keepdim=True)
        return self.weight * (x.float() * torch.rsqrt(v + self.eps)).to(x.dtype)


def _t5_bucket(rel: torch.Tensor, bidirectional: bool, num_buckets: int, max_distance: int) -> torch.Tensor:
    ret = torch.zeros_like(rel)
    if bidirectional:
        num_buckets //= 2
        ret = ret + (rel > 0).long() * num_buckets
        rel = rel.abs()
    else:
        rel = -torch.min(rel, torch.zeros_like(rel))
    max_exact = num_buckets // 2
    is_small = rel < max_exact
    large = max_exact + (torch.log(rel.float().clamp(min=1) / max_exact) / math.log(max_distance / max_exact)
                         * (num_buckets - max_exact)).long()
    large = torch.min(large, torch.full_like(large, num_buckets - 1))
    return ret + torch.where(is_small, rel, large)


class _T5Attention(nn.Module):
    def __init__(self, c, has_bias: bool, bidirectional: bool):
        super().__init__()
        inner = c["num_heads"] * c["d_kv"]
        self.h, self.bidirectional = c["num_heads"], bidirectional
        self.buckets, self.max_dist = c.get("relative_attention_num_buckets", 32), c.get("relative_attention_max_distance", 128)
        self.q, self.k, self.v = (Linear(c["d_model"], inner, bias=False) for _ in range(3))
        self.o = Linear(inner, c["d_model"], bias=False)
        if has_bias:
            self.relative_attention_bias = nn.Embedding(self.buckets, self.h)

    def bias(self, Tq, Tk, device):
        ctx = torch.arange(Tq, device=device)[:, None] + (Tk - Tq)
        mem = torch.arange(Tk, device=device)[None, :]
        b = _t5_bucket(mem - ctx, self.bidirectional, self.buckets, self.max_dist)
        return self.relative_attention_bias(b).permute(2, 0, 1)[None]          # [1, h, Tq, Tk]

    def forward(self, x, kv, bias):
        q, k, v = _heads(self.q(x), self.h), _heads(self.k(kv), self.h), _heads(self.v(kv), self.h)
        s = torch.matmul(q, k.transpose(-1, -2)).float()                          # T5 does not scale the scores
        if bias is not None:
            s = s + bias
        return self.o(_merge(torch.matmul(torch.softmax(s, -1).to(v.dtype), v)))


class _T5LayerSelf(nn.Module):
    def __init__(self, c, has_bias, bidir):
        super().__init__()
        self.SelfAttention = _T5Attention(c, has_bias, bidir)
        self.layer_norm = _T5Norm(c["d_model"], c.get("layer_norm_epsilon", 1e-6))


class _T5LayerCross(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.EncDecAttention = _T5Attention(c, False, True)
        self.layer_norm = _T5Norm(c["d_model"], c.get("layer_norm_epsilon", 1e-6))


class _T5Dense(nn.Module):
    def __init__(self, c):
        super().__init__()
        proj = c.get("feed_forward_proj", "relu")
        self.gated = proj.startswith("gated-")
        self.fn = _act({"gelu": "gelu_new"}.get(proj.replace("gated-", ""), proj.replace("gated-", "")))
        if self.gated:
            self.wi_0, self.wi_1 = Linear(c["d_model"], c["d_ff"], bias=False), Linear(c["d_model"], c["d_ff"], bias=False)
        else:
            self.wi = Linear(c["d_model"], c["d_ff"], bias=False)
        self.wo = Linear(c["d_ff"], c["d_model"], bias=False)

    def forward(self, x):
        return self.wo(self.fn(self.wi_0(x)) * self.wi_1(x)) if self.gated else self.wo(self.fn(self.wi(x)))


class _T5LayerFF(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.DenseReluDense = _T5Dense(c)
        self.layer_norm = _T5Norm(c["d_model"], c.get("layer_norm_epsilon", 1e-6))


class _T5Block(nn.Module):
    def __init__(self, c, first: bool, decoder: bool):
        super().__init__()
        layers = [_T5LayerSelf(c, first, not decoder)]
        if decoder:
            layers.append(_T5LayerCross(c))
        layers.append(_T5LayerFF(c))
        self.layer = nn.ModuleList(layers)


class _T5Stack(nn.Module):
    def __init__(self, c, decoder: bool, n: int):
        super().__init__()
        self.decoder = decoder
        self.embed_tokens = nn.Embedding(c["vocab_size"], c["d_model"])
        self.block = nn.ModuleList([_T5Block(c, i == 0, decoder) for i in range(n)])
        self.final_layer_norm = _T5Norm(c["d_model"], c.get("layer_norm_epsilon", 1e-6))

    def forward(self, ids, enc: Optional[torch.Tensor] = None, mask: Optional[torch.Tensor] = None,
                enc_mask: Optional[torch.Tensor] = None):
        x = self.embed_tokens(ids)
        T = x.shape[1]
        bias = self.block[0].layer[0].SelfAttention.bias(T, T, x.device).float()
        if self.decoder:
            bias = bias + torch.full((T, T), float("-inf"), device=x.device).triu(1)
        if mask is not None:
            bias = bias + (1.0 - mask[:, None, None, :].float()) * torch.finfo(torch.float32).min
        cross = None if enc_mask is None else (1.0 - enc_mask[:, None, None, :].float()) * torch.finfo(torch.float32).min
        for blk in self.block:
            sa = blk.layer[0]
            x = x + sa.SelfAttention(sa.layer_norm(x), sa.layer_norm(x), bias)
            if self.decoder:
                ca = blk.layer[1]
                x = x + ca.EncDecAttention(ca.layer_norm(x), enc, cross)
            ff = blk.layer[-1]
            x = x + ff.DenseReluDense(ff.layer_norm(x))
        return self.final_layer_norm(x)


class T5Model(nn.Module):
    """T5 / Flan-T5 encoder-decoder with bucketed relative position bias
    (crates/pmetal-models/src/architectures/t5.rs). ``forward`` returns vocabulary logits of the decoder tokens."""

    def __init__(self, cfg: dict):
        super().__init__()
        self.cfg = cfg
        self.shared = nn.Embedding(cfg["vocab_size"], cfg["d_model"])
        self.encoder = _T5Stack(cfg, False, cfg["num_layers"])
        self.decoder = _T5Stack(cfg, True, cfg.get("num_decoder_layers") or cfg["num_layers"])
        self.encoder.embed_tokens = self.shared
        self.decoder.embed_tokens = self.shared
        self.tied = bool(cfg.get("tie_word_embeddings", True))
        if not self.tied:
            self.lm_head = Linear(cfg["d_model"], cfg["vocab_size"], bias=False)

    def encode(self, input_ids, attention_mask=None):
        return self.encoder(input_ids, mask=attention_mask)

    def forward(self, input_ids, decoder_input_ids, attention_mask=None):
        enc = self.encode(input_ids, attention_mask)
        h = self.decoder(decoder_input_ids, enc=enc, enc_mask=attention_mask)
        if self.tied:
            return F.linear(h * self.cfg["d_model"] ** -0.5, self.shared.weight)
        return self.lm_head(h)


# ------------------------------------------------------------------------------------------------ CLIP
class _PreLnAttention(nn.Module):
    """Bias-carrying multi-head attention with q/k/v/out projections (CLIP and Whisper naming)."""

    def __init__(self, H, h, k_bias: bool = True):
        super().__init__()
        self.h = h
        self.q_proj, self.v_proj, self.out_proj = Linear(H, H), Linear(H, H), Linear(H, H)
        self.k_proj = Linear(H, H, bias=k_bias)

    def forward(self, x, kv=None, causal: bool = False):
        kv = x if kv is None else kv
        q, k, v = _heads(self.q_proj(x), self.h), _heads(self.k_proj(kv), self.h), _heads(self.v_proj(kv), self.h)
        return self.out_proj(_merge(F.scaled_dot_product_attention(q, k, v, is_causal=causal and q.shape[2] > 1)))


class _ClipMlp(nn.Module):
    def __init__(self, H, I, act):
        super().__init__()
        self.fc1, self.fc2, self.fn = Linear(H, I), Linear(I, H), _act(act)

    def forward(self, x):
        return self.fc2(self.fn(self.fc1(x)))


class _ClipLayer(nn.Module):
    def __init__(self, H, h, I, act, eps):
        super().__init__()
        self.self_attn = _PreLnAttention(H, h)
        self.layer_norm1, self.layer_norm2 = nn.LayerNorm(H, eps=eps), nn.LayerNorm(H, eps=eps)
        self.mlp = _ClipMlp(H, I, act)

    def forward(self, x, causal):
        x = x + self.self_attn(self.layer_norm1(x), causal=causal)
        return x + self.mlp(self.layer_norm2(x))


class _ClipEncoder(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.layers = nn.ModuleList([_ClipLayer(c["hidden_size"], c["num_attention_heads"], c["intermediate_size"],
                                                c.get("hidden_act", "quick_gelu"), c.get("layer_norm_eps", 1e-5))
                                     for _ in range(c["num_hidden_layers"])])


class _ClipTextEmb(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.token_embedding = nn.Embedding(c["vocab_size"], c["hidden_size"])
        self.position_embedding = nn.Embedding(c["max_position_embeddings"], c["hidden_size"])


class _ClipText(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.embeddings, self.encoder = _ClipTextEmb(c), _ClipEncoder(c)
        self.final_layer_norm = nn.LayerNorm(c["hidden_size"], eps=c.get("layer_norm_eps", 1e-5))
        self.eos = c.get("eos_token_id", 2)

    def forward(self, ids):
        T = ids.shape[1]
        x = self.embeddings.token_embedding(ids) + self.embeddings.position_embedding(torch.arange(T, device=ids.device))
        for layer in self.encoder.layers:
            x = layer(x, True)
        x = self.final_layer_norm(x)
        # pooled output: the end-of-text position (highest id in the original vocabulary, else the first eos)
        idx = ids.argmax(-1) if self.eos == 2 else (ids == self.eos).int().argmax(-1)
        return x, x[torch.arange(x.shape[0], device=x.device), idx]


class _ClipVisionEmb(nn.Module):
    def __init__(self, c):
        super().__init__()
        H, P = c["hidden_size"], c["patch_size"]
        self.class_embedding = nn.Parameter(torch.randn(H))
        self.patch_embedding = nn.Conv2d(c.get("num_channels", 3), H, P, P, bias=False)
        self.position_embedding = nn.Embedding((c["image_size"] // P) ** 2 + 1, H)


class _ClipVision(nn.Module):
    def __init__(self, c):
        super().__init__()
        eps = c.get("layer_norm_eps", 1e-5)
        self.embeddings, self.encoder = _ClipVisionEmb(c), _ClipEncoder(c)
        self.pre_layrnorm, self.post_layernorm = nn.LayerNorm(c["hidden_size"], eps=eps), nn.LayerNorm(c["hidden_size"], eps=eps)

    def forward(self, pixels):
        e = self.embeddings
        p = e.patch_embedding(pixels).flatten(2).transpose(1, 2)
        x = torch.cat((e.class_embedding.expand(p.shape[0], 1, -1), p), 1)
        x = self.pre_layrnorm(x + e.position_embedding.weight[None, : x.shape[1]])
        for layer in self.encoder.layers:
            x = layer(x, False)
        return x, self.post_layernorm(x[:, 0])


class ClipModel(nn.Module):
    """CLIP text and vision towers with the joint projection (crates/pmetal-models/src/architectures/clip.rs)."""

    def __init__(self, cfg: dict):
        super().__init__()
        t, v = cfg["text_config"], cfg["vision_config"]
        dim = cfg.get("projection_dim", 512)
        self.text_model, self.vision_model = _ClipText(t), _ClipVision(v)
        self.visual_projection = Linear(v["hidden_size"], dim, bias=False)
        self.text_projection = Linear(t["hidden_size"], dim, bias=False)
        self.logit_scale = nn.Parameter(torch.tensor(cfg.get("logit_scale_init_value", 2.6592)))

    def text_embeds(self, ids):
        return F.normalize(self.text_projection(self.text_model(ids)[1]), dim=-1)

    def image_embeds(self, pixels):
        return F.normalize(self.visual_projection(self.vision_model(pixels)[1]), dim=-1)

    def forward(self, input_ids, pixel_values) -> Tuple[torch.Tensor, torch.Tensor]:
        t, i = self.text_embeds(input_ids), self.image_embeds(pixel_values)
        per_text = self.logit_scale.exp() * t @ i.t()
        return per_text.t(), per_text                       # (logits per image, logits per text)


# ------------------------------------------------------------------------------------------------ Whisper
class _WhisperLayer(nn.Module):
    def __init__(self, D, h, ffn, cross: bool, act):
        super().__init__()
        self.self_attn = _PreLnAttention(D, h, k_bias=False)
        self.self_attn_layer_norm = nn.LayerNorm(D)
        if cross:
            self.encoder_attn = _PreLnAttention(D, h, k_bias=False)
            self.encoder_attn_layer_norm = nn.LayerNorm(D)
        self.fc1, self.fc2, self.final_layer_norm, self.fn = Linear(D, ffn), Linear(ffn, D), nn.LayerNorm(D), _act(act)

    def forward(self, x, enc=None):
        x = x + self.self_attn(self.self_attn_layer_norm(x), causal=enc is not None)
        if enc is not None:
            x = x + self.encoder_attn(self.encoder_attn_layer_norm(x), kv=enc)
        return x + self.fc2(self.fn(self.fc1(self.final_layer_norm(x))))


class _WhisperEncoder(nn.Module):
    def __init__(self, c):
        super().__init__()
        D = c["d_model"]
        self.conv1 = nn.Conv1d(c["num_mel_bins"], D, 3, padding=1)
        self.conv2 = nn.Conv1d(D, D, 3, stride=2, padding=1)
        self.embed_positions = nn.Embedding(c["max_source_positions"], D)
        self.layers = nn.ModuleList([_WhisperLayer(D, c["encoder_attention_heads"], c["encoder_ffn_dim"], False,
                                                   c.get("activation_function", "gelu")) for _ in range(c["encoder_layers"])])
        self.layer_norm = nn.LayerNorm(D)

    def forward(self, mel):
        x = F.gelu(self.conv2(F.gelu(self.conv1(mel)))).transpose(1, 2)
        x = x + self.embed_positions.weight[: x.shape[1]]
        for layer in self.layers:
            x = layer(x)
        return self.layer_norm(x)


class _WhisperDecoder(nn.Module):
    def __init__(self, c):
        super().__init__()
        D = c["d_model"]
        self.embed_tokens = nn.Embedding(c["vocab_size"], D)
        self.embed_positions = nn.Embedding(c["max_target_positions"], D)
        self.layers = nn.ModuleList([_WhisperLayer(D, c["decoder_attention_heads"], c["decoder_ffn_dim"], True,
                                                   c.get("activation_function", "gelu")) for _ in range(c["decoder_layers"])])
        self.layer_norm = nn.LayerNorm(D)

    def forward(self, ids, enc):
        x = self.embed_tokens(ids) + self.embed_positions.weight[: ids.shape[1]]
        for layer in self.layers:
            x = layer(x, enc)
        return self.layer_norm(x)


class _WhisperCore(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.encoder, self.decoder = _WhisperEncoder(c), _WhisperDecoder(c)


class WhisperModel(nn.Module):
    """Whisper speech-to-text transformer: convolutional front end over log-mel frames, encoder, decoder with cross
    attention, output projection tied to the token embedding (crates/pmetal-models/src/architectures/whisper.rs)."""

    def __init__(self, cfg: dict):
        super().__init__()
        self.model = _WhisperCore(cfg)

    def forward(self, input_features, decoder_input_ids):
        enc = self.model.encoder(input_features)
        return F.linear(self.model.decoder(decoder_input_ids, enc), self.model.decoder.embed_tokens.weight)

    @torch.no_grad()
    def transcribe(self, input_features, start_ids, max_new_tokens: int = 32, eos_token_id: Optional[int] = None):
        enc = self.model.encoder(input_features)
        ids = torch.tensor([list(start_ids)], device=input_features.device)
        for _ in range(max_new_tokens):
            nxt = F.linear(self.model.decoder(ids, enc)[:, -1], self.model.decoder.embed_tokens.weight).argmax(-1)
            ids = torch.cat((ids, nxt[:, None]), 1)
            if eos_token_id is not None and int(nxt) == eos_token_id:
                break
        return ids[0].tolist()
