"""Decoder-only transformer (Qwen3 / Qwen2 / Llama / Mistral family, dense or MoE).

Behaviour follows the reference's Qwen3 implementation
(crates/pmetal-models/src/architectures/qwen3.rs:235-545): pre-norm blocks, GQA,
optional per-head RMSNorm on q and k before half-split RoPE, SwiGLU MLP, optional
tied output embedding; the MoE variant follows qwen3_moe.rs:390-640.

Physical layout differs from the Hugging Face checkpoint layout on purpose: q, k, v
are one row-stacked weight (one GEMM), as are gate and up, and every frozen weight
can keep a transposed copy so that the input-gradient GEMM reads a K-major operand.
Activations are a flat token stream [T, hidden] with ``cu_seqlens`` document
boundaries; a padded batch is the special case of equal-length documents.
``load_hf_state_dict`` / ``hf_state_dict`` translate to and from checkpoint names.
"""
from __future__ import annotations

import math
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as ops
from .config import ModelArgs

ATTN_PROJ = ("q_proj", "k_proj", "v_proj", "o_proj")
MLP_PROJ = ("gate_proj", "up_proj", "down_proj")
ALL_PROJ = ATTN_PROJ + MLP_PROJ


# rows up to which linear layers run on the bandwidth-bound mat-vec kernel instead of tensor-core tiles (decode)
DECODE_MEGA = os.environ.get("PMETAL_DECODE_MEGA", "1") == "1"
GEMV_MAX_ROWS = int(os.environ.get("PMETAL_GEMV_MAX_ROWS", "16"))


class FusedLinear(nn.Module):
    """A row-stacked group of projections sharing one input, with optional LoRA.

    ``weight`` is [sum(seg_sizes), in]. LoRA factors are stored stacked as
    ``lora_a`` [n_seg·r, in] and ``lora_b`` [sum(seg_sizes), r] in fp32 (the reference keeps
    adapters in f32, crates/pmetal-lora/src/lora.rs:268-289). ``active`` marks which
    segments are LoRA targets; inactive ones keep zero factors and receive no update.
    """

    def __init__(self, in_features: int, seg_names: Sequence[str], seg_sizes: Sequence[int], bias: bool = False,
                 dtype=torch.float32, device=None):
        super().__init__()
        self.in_features = in_features
        self.seg_names = tuple(seg_names)
        self.seg_sizes = tuple(int(s) for s in seg_sizes)
        self.out_features = sum(self.seg_sizes)
        self.weight = nn.Parameter(torch.empty(self.out_features, in_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(self.out_features, dtype=dtype, device=device)) if bias else None
        self.weight_t: Optional[torch.Tensor] = None
        self.lora_a: Optional[nn.Parameter] = None
        self.lora_b: Optional[nn.Parameter] = None
        self.r = 0
        self.scale = 0.0
        self.active: Tuple[bool, ...] = tuple(False for _ in self.seg_sizes)
        self.batched = None             # lora.batched.BatchedLoraAdapters: several adapters, one index per input row
        self.adapter_rows: Optional[torch.Tensor] = None

    # -- LoRA management
    def add_lora(self, r: int, scale: float, active: Sequence[bool], use_rslora: bool = False,
                 generator: Optional[torch.Generator] = None) -> None:
        if r <= 0 or not any(active):
            return
        dev = self.weight.device
        n = len(self.seg_sizes)
        a = torch.zeros(n * r, self.in_features, dtype=torch.float32)
        # A ~ U(±sqrt(3/in)) (rsLoRA: ±sqrt(1/r)), B = 0  (crates/pmetal-lora/src/lora.rs:268-289)
        bound = math.sqrt(1.0 / r) if use_rslora else math.sqrt(3.0 / self.in_features)
        for i, on in enumerate(active):
            if on:
                a[i * r:(i + 1) * r].uniform_(-bound, bound, generator=generator)
        self.lora_a = nn.Parameter(a.to(dev))
        self.lora_b = nn.Parameter(torch.zeros(self.out_features, r, dtype=torch.float32, device=dev))
        self.r, self.scale, self.active = r, float(scale), tuple(bool(x) for x in active)
        if not all(self.active):
            mask_a = torch.zeros(n * r, 1, device=dev)
            mask_b = torch.zeros(self.out_features, 1, device=dev)
            o = 0
            for i, (on, sz) in enumerate(zip(self.active, self.seg_sizes)):
                if on:
                    mask_a[i * r:(i + 1) * r] = 1
                    mask_b[o:o + sz] = 1
                o += sz
            # the fused backward accumulates straight into .grad and hands autograd None
            self.lora_a.register_hook(lambda g, m=mask_a: None if g is None else g * m)
            self.lora_b.register_hook(lambda g, m=mask_b: None if g is None else g * m)

    def seg_slice(self, name: str) -> Tuple[int, slice]:
        i = self.seg_names.index(name)
        o = sum(self.seg_sizes[:i])
        return i, slice(o, o + self.seg_sizes[i])

    def prepare_transposed(self) -> None:
        """Keep Wᵀ for the input-gradient GEMM (frozen weights only)."""
        if self.weight.is_cuda and not self.weight.requires_grad:
            self.weight_t = self.weight.detach().t().contiguous()

    def merged_weight(self) -> torch.Tensor:
        q = getattr(self, "qweight", None)
        if q is not None:
            from ..lora.nf4 import dequantize
            w = dequantize(q, torch.float32)
        else:
            w = self.weight.detach().to(torch.float32, copy=True)     # never alias the stored weight (fp32 models)
        if self.lora_a is not None:
            o = 0
            for i, sz in enumerate(self.seg_sizes):
                a = self.lora_a[i * self.r:(i + 1) * self.r].float()
                w[o:o + sz] += self.scale * (self.lora_b[o:o + sz].float() @ a)
                o += sz
        return w

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.batched is not None and self.adapter_rows is not None and self.bias is None:
            from ..lora.batched import batched_lora_linear
            return batched_lora_linear(x, self.weight, self.batched, self.adapter_rows, residual)
        if self.weight.requires_grad and self.bias is None and self.lora_a is None:
            sh = getattr(self.weight, "shadow", None)           # full-parameter training: bf16 shadow of the fp32 master
            if sh is not None and ops.use_native(x) and self.in_features % 8 == 0 and self.out_features % 8 == 0:
                return ops.dense_linear(x, self.weight, sh, residual)
        if self.bias is not None or self.weight.requires_grad:
            y = F.linear(x, self.weight, self.bias)
            if self.lora_a is not None:
                y = y + self._lora_delta(x)
            return y if residual is None else y + residual
        return ops.lora_linear(x, self.weight, self.weight_t, self.lora_a, self.lora_b, self.seg_sizes, self.r,
                               self.scale, residual, getattr(self, "lora_a_c", None), getattr(self, "lora_b_c", None),
                               getattr(self, "qweight", None))

    def gemv_ok(self, m: int) -> bool:
        """Decode fast path: a few rows, no bias, and either a plain bf16 weight or a 4-bit (NF4 / FP4) packed weight
        that the mat-vec kernel expands on the fly."""
        if m > GEMV_MAX_ROWS or self.bias is not None or (self.batched is not None and self.adapter_rows is not None):
            return False
        rows = 4 if m <= 4 else (8 if m <= 8 else 16)
        if rows * self.in_features * 2 > 200 * 1024:        # the kernel stages the token rows in shared memory
            return False
        q = getattr(self, "qweight", None)
        if q is not None:
            return (q.scheme in ("nf4", "fp4") and q.data.is_cuda and q.block_size % 32 == 0 and self.in_features % 32 == 0)
        return (self.weight.is_cuda and self.weight.dtype == torch.bfloat16 and not self.weight.requires_grad
                and self.in_features % 8 == 0)

    def gemv_forward(self, x: torch.Tensor, norm_w=None, eps: float = 1e-6, residual=None, swiglu: bool = False):
        """y = norm(x) W^T (+ LoRA) (+ residual), optionally SwiGLU over the (gate, up) halves; one or two launches of
        the skinny mat-vec kernel."""
        from ..ops import native as nat
        t = None
        if self.lora_a is not None:
            a_c = getattr(self, "lora_a_c", None)
            if a_c is None:
                a_c = self.lora_a.detach().to(torch.bfloat16)
            t = nat.gemv(x, a_c, norm_w, eps, alpha=self.scale)
        q = getattr(self, "qweight", None)
        kw = dict(t=t, lora_b=self.lora_b.detach(), r=self.r, seg_sizes=self.seg_sizes) if t is not None else {}
        if q is not None:
            return nat.gemv_q4(x, q, norm_w, eps, residual, swiglu, **kw)
        return nat.gemv(x, self.weight, norm_w, eps, residual, swiglu, **kw)

    def _lora_delta(self, x: torch.Tensor) -> torch.Tensor:
        outs, o = [], 0
        for i, sz in enumerate(self.seg_sizes):
            t = F.linear(x, self.lora_a[i * self.r:(i + 1) * self.r].to(x.dtype))
            outs.append(self.scale * F.linear(t, self.lora_b[o:o + sz].to(x.dtype)))
            o += sz
        return torch.cat(outs, -1)


class Attention(nn.Module):
    def __init__(self, cfg: ModelArgs, layer_idx: int, dtype, device):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        d = cfg.head_dim
        self.qkv_proj = FusedLinear(cfg.hidden_size, ("q_proj", "k_proj", "v_proj"),
                                    (cfg.q_size, cfg.kv_size, cfg.kv_size), cfg.attention_bias, dtype, device)
        self.o_proj = FusedLinear(cfg.q_size, ("o_proj",), (cfg.hidden_size,), False, dtype, device)
        if cfg.qk_norm:
            self.q_norm = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
            self.k_norm = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        else:
            self.q_norm = self.k_norm = None
        self.window = cfg.sliding_window if cfg.uses_sliding_window(layer_idx) else 0

    def forward(self, x_normed, residual, rope, cu_seqlens, seq_start):
        cfg = self.cfg
        qkv = self.qkv_proj(x_normed)
        qn, kn = (ops.live(self.q_norm), ops.live(self.k_norm)) if self.q_norm is not None else (None, None)
        o = ops.attention_block(qkv, qn, kn, rope[0], rope[1], cu_seqlens, seq_start,
                                cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps,
                                None, self.window, cfg.attn_logit_softcap)
        return self.o_proj(o, residual)


class MLP(nn.Module):
    def __init__(self, cfg: ModelArgs, inter: int, dtype, device):
        super().__init__()
        self.gate_up_proj = FusedLinear(cfg.hidden_size, ("gate_proj", "up_proj"), (inter, inter), cfg.mlp_bias,
                                        dtype, device)
        self.down_proj = FusedLinear(inter, ("down_proj",), (cfg.hidden_size,), cfg.mlp_bias, dtype, device)

    def forward(self, x_normed, residual):
        return self.down_proj(ops.swiglu(self.gate_up_proj(x_normed)), residual)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelArgs, layer_idx: int, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.self_attn = Attention(cfg, layer_idx, dtype, device)
        if cfg.is_moe_layer(layer_idx):
            from .moe import SparseMoeBlock
            self.mlp = SparseMoeBlock(cfg, dtype, device)
        else:
            self.mlp = MLP(cfg, cfg.intermediate_size, dtype, device)
        self.input_layernorm = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device))
        self.post_attention_layernorm = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device))

    def forward(self, x, rope, cu_seqlens, seq_start):
        """x -> x + attn(norm(x)) -> (+ mlp(norm(.))). The residual adds run in the epilogue of the
        o_proj / down_proj GEMMs."""
        eps = self.cfg.rms_norm_eps
        # the norm hands back the stream it read: using that alias for the residual branch lets its gradient be
        # summed inside the norm's backward kernel
        n1, x = ops.add_rms_norm(x, None, ops.live(self.input_layernorm), eps)
        h = self.self_attn(n1, x, rope, cu_seqlens, seq_start)
        n2, h = ops.add_rms_norm(h, None, ops.live(self.post_attention_layernorm), eps)
        return self.mlp(n2, h)


class DecoderLM(nn.Module):
    def __init__(self, cfg: ModelArgs, dtype=torch.float32, device=None):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device))
        self.layers = nn.ModuleList([DecoderLayer(cfg, i, dtype, device) for i in range(cfg.num_hidden_layers)])
        self.norm = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device))
        self.lm_head = None if cfg.tie_word_embeddings else nn.Parameter(
            torch.empty(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device))
        self.head_t: Optional[torch.Tensor] = None
        self.gradient_checkpointing = 0
        self._rope_schedule = None      # (inv_freq on the device, attention factor) for non-linear rope_scaling

    def rope(self, positions: torch.Tensor):
        """cos/sin tables of this batch: plain or linearly scaled RoPE straight from theta, every other
        schedule (llama3, yarn, dynamic NTK, longrope) from its frequency vector built once per device."""
        cfg = self.cfg
        if not cfg.rope_scaling:
            return ops.rope_table(positions, cfg.head_dim, cfg.rope_theta, cfg.rope_scale)
        sched = self._rope_schedule
        if sched is None or sched[0].device != positions.device:
            from .rope import rope_inv_freq
            inv, att = rope_inv_freq(cfg.head_dim, cfg.rope_theta, cfg.rope_scaling, cfg.max_position_embeddings)
            sched = self._rope_schedule = (inv.to(positions.device).contiguous(), float(att))
        return ops.rope_table_scheduled(positions, sched[0], sched[1])

    # ------------------------------------------------------------------ init / freeze
    @torch.no_grad()
    def init_weights(self, std: float = 0.02, seed: int = 0) -> "DecoderLM":
        """N(0, std) for every matrix, ones for norms. Drawn on CPU in fp32 in parameter order so the
        result is identical for any target device/dtype."""
        g = torch.Generator().manual_seed(seed)
        for name, p in self.named_parameters():
            if "lora_" in name:
                continue
            if p.dim() >= 2:
                p.copy_(torch.empty(p.shape, dtype=torch.float32).normal_(0.0, std, generator=g).to(p.dtype))
            elif name.endswith("bias"):
                p.zero_()
            else:
                p.fill_(1.0)
        return self

    @torch.no_grad()
    def init_weights_on_device(self, std: float = 0.02, seed: int = 0) -> "DecoderLM":
        """Same distribution as ``init_weights`` but drawn on the parameters' own device (large models: seconds
        instead of minutes); the values differ from the CPU-drawn ones."""
        g = torch.Generator(device=self.embed_tokens.device).manual_seed(seed)
        for name, p in self.named_parameters():
            if "lora_" in name:
                continue
            if p.dim() >= 2:
                p.normal_(0.0, std, generator=g)
            elif name.endswith("bias"):
                p.zero_()
            else:
                p.fill_(1.0)
        return self

    def freeze_base(self) -> None:
        for name, p in self.named_parameters():
            p.requires_grad_("lora_" in name or "magnitude" in name)

    def fused_linears(self):
        for i, layer in enumerate(self.layers):
            yield i, "self_attn", layer.self_attn.qkv_proj
            yield i, "self_attn", layer.self_attn.o_proj
            if isinstance(layer.mlp, MLP):
                yield i, "mlp", layer.mlp.gate_up_proj
                yield i, "mlp", layer.mlp.down_proj

    def prepare_for_training(self) -> None:
        """Build the transposed copies the input-gradient GEMMs read."""
        for _, _, fl in self.fused_linears():
            fl.prepare_transposed()
        hw = self.head_weight()
        if hw.is_cuda and not hw.requires_grad:
            self.head_t = hw.detach().t().contiguous()

    def head_weight(self) -> torch.Tensor:
        return self.embed_tokens if self.lm_head is None else self.lm_head

    # ------------------------------------------------------------------ forward
    def forward_hidden(self, input_ids: torch.Tensor, positions: Optional[torch.Tensor] = None,
                       cu_seqlens: Optional[torch.Tensor] = None, seq_start: Optional[torch.Tensor] = None,
                       layer_range: Optional[Tuple[int, int]] = None,
                       hidden_in: Optional[torch.Tensor] = None) -> torch.Tensor:
        """input_ids [T] (flat packed stream) or [B, L] → final-normed hidden [T, H]."""
        if input_ids.dim() == 2:
            B, L = input_ids.shape
            input_ids = input_ids.reshape(-1)
            if cu_seqlens is None:
                cu_seqlens = torch.arange(0, (B + 1) * L, L, dtype=torch.int32, device=input_ids.device)
            if positions is None:
                positions = torch.arange(L, device=input_ids.device, dtype=torch.int32).repeat(B)
        T = input_ids.shape[0]
        if cu_seqlens is None:
            cu_seqlens = torch.tensor([0, T], dtype=torch.int32, device=input_ids.device)
        if positions is None:
            from ..ops.reference import seq_starts_from_cu
            ss = seq_start if seq_start is not None else seq_starts_from_cu(cu_seqlens, T)
            positions = torch.arange(T, device=input_ids.device, dtype=torch.int32) - ss
        lo, hi = layer_range if layer_range is not None else (0, len(self.layers))
        x = hidden_in if hidden_in is not None else F.embedding(input_ids, ops.live(self.embed_tokens))
        rope = self.rope(positions)
        policies = getattr(self, "layer_policies", None) if self.training else None      # utils/offload.py plan
        ready = getattr(self, "grad_ready_hook", None) if torch.is_grad_enabled() else None   # parallel/overlap.py
        for i in range(lo, hi):
            layer = self.layers[i]
            if ready is not None and x.requires_grad:     # fires once the gradient w.r.t. this layer's input exists
                x.register_hook(lambda g, i=i: ready(i))
            pol = policies[i] if policies is not None else None
            if pol == "recompute" or (pol is None and self.gradient_checkpointing and self.training
                                      and (i % self.gradient_checkpointing == 0)):
                from torch.utils.checkpoint import checkpoint
                x = checkpoint(layer, x, rope, cu_seqlens, seq_start, use_reentrant=False)
            elif pol in ("offload_cpu", "offload_disk") and getattr(self, "activation_offloader", None) is not None:
                with self.activation_offloader:       # what this block saves for backward waits in host memory
                    x = layer(x, rope, cu_seqlens, seq_start)
            else:
                x = layer(x, rope, cu_seqlens, seq_start)
        if hi < len(self.layers):
            return x
        return ops.rms_norm(x, ops.live(self.norm), self.cfg.rms_norm_eps)

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        out = F.linear(hidden, self.head_weight())
        cap = self.cfg.final_logit_softcap
        return cap * torch.tanh(out / cap) if cap > 0 else out

    def forward(self, input_ids, positions=None, cu_seqlens=None, seq_start=None) -> torch.Tensor:
        shape = input_ids.shape
        h = self.forward_hidden(input_ids, positions, cu_seqlens, seq_start)
        return self.logits(h).view(*shape, -1)

    def loss(self, input_ids: torch.Tensor, labels: torch.Tensor, positions=None, cu_seqlens=None,
             seq_start=None) -> torch.Tensor:
        """Causal-LM loss. ``labels`` are unshifted (label[t] is the id at t, −100 = ignore); the shift by
        one happens here (crates/pmetal-bridge/src/training.rs:120). In a packed stream the caller masks
        the first token of each non-first document so no prediction crosses a boundary."""
        h = self.forward_hidden(input_ids, positions, cu_seqlens, seq_start)
        flat = labels.reshape(-1)
        if input_ids.dim() == 2:
            B, L = input_ids.shape
            tgt = torch.full_like(labels, -100)
            tgt[:, :-1] = labels[:, 1:]
            tgt = tgt.reshape(-1)
        else:
            tgt = torch.full_like(flat, -100)
            tgt[:-1] = flat[1:]
        return ops.causal_lm_loss(h, self.head_weight(), tgt, -100, self.head_t, self.cfg.final_logit_softcap)

    # ------------------------------------------------------------------ cached (paged) forward
    @torch.no_grad()
    def forward_paged(self, input_ids: torch.Tensor, cache, meta, all_logits: bool = False,
                      return_hidden: bool = False) -> torch.Tensor:
        """Forward over the new tokens of several sequences with a paged KV cache.

        ``input_ids`` [total_q] are the new tokens in ``meta`` order; keys/values are appended to ``cache`` and
        attention reads the block table directly. Returns logits for the last new token of every sequence
        ([n_seq, V]) or for every new token ([total_q, V], speculative verification)."""
        cfg = self.cfg
        ch = getattr(self, "step_channel", None)
        if ch is not None and ch.leader and not ch.muted:
            ch.publish_paged(input_ids, meta, all_logits, return_hidden)      # the other ranks repeat this call
        hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        x = F.embedding(input_ids, self.embed_tokens)
        native = ops.use_native(x) and d == 128
        rope = self.rope(meta.positions)
        T = x.shape[0]
        skinny = native and T <= GEMV_MAX_ROWS
        layers = self.layers
        plain_cache = cache.quant is None and cache.window == 0      # bf16 blocks, nothing recycled
        if (skinny and DECODE_MEGA and plain_cache and meta.max_q == 1 and T == meta.block_table.shape[0]
                and self._mega_ok(T)):
            # every layer of the step in one cooperative launch (csrc/decode_mega.cu)
            from ..ops import native as nat
            table = self._mega_table(cache)
            ns = nat.decode_splits(T, hkv, meta.max_kv)
            sc = self._mega_scratch.get((T, ns))
            if sc is None:
                sc = self._mega_scratch[(T, ns)] = nat.decode_scratch(T, cfg.hidden_size, hq, hkv, cfg.intermediate_size,
                                                                      ns, x.device)
            x = nat.decode_layers(table, len(self.layers), x.contiguous(), sc, rope[0], rope[1], meta, hq, hkv,
                                  cfg.intermediate_size, cfg.rms_norm_eps, d ** -0.5)
            layers = ()
        for li, layer in enumerate(layers):
            at = layer.self_attn
            if getattr(self, "tp_world", 1) > 1:
                x = self._layer_paged_sharded(li, layer, x, rope, cache, meta, native)
                continue
            if skinny and at.qkv_proj.gemv_ok(T) and at.o_proj.gemv_ok(T):
                # decode: six launches per dense layer (norm+qkv, qk-norm+rope+cache append, attention, o+residual,
                # norm+gate/up+SwiGLU, down+residual); mixture-of-experts layers share the attention half
                from ..ops import native as nat
                eps = cfg.rms_norm_eps
                qkv = at.qkv_proj.gemv_forward(x, layer.input_layernorm, eps)
                if cache.quant is None:
                    q = nat.qknorm_rope_cache(qkv, at.q_norm, at.k_norm, rope[0], rope[1], hq, hkv, eps, cache.k[li],
                                              cache.v[li], meta.slots)
                else:
                    q, k = nat.qknorm_rope_fwd(qkv, at.q_norm, at.k_norm, rope[0], rope[1], hq, hkv, eps)
                    cache.append(li, k, qkv[:, (hq + hkv) * d:].view(T, hkv, d), meta.slots)
                o = cache.attention(li, q, meta, d ** -0.5, at.window).view(T, hq * d)
                h = at.o_proj.gemv_forward(o, residual=x)
                if isinstance(layer.mlp, MLP) and layer.mlp.gate_up_proj.gemv_ok(T) and layer.mlp.down_proj.gemv_ok(T):
                    act = layer.mlp.gate_up_proj.gemv_forward(h, layer.post_attention_layernorm, eps, swiglu=True)
                    x = layer.mlp.down_proj.gemv_forward(act, residual=h)
                else:
                    x = layer.mlp(ops.rms_norm(h, layer.post_attention_layernorm, eps), h)
                continue
            n1 = ops.rms_norm(x, layer.input_layernorm, cfg.rms_norm_eps)
            qkv = at.qkv_proj(n1)
            if native:
                from ..ops import native as nat
                q, k = nat.qknorm_rope_fwd(qkv, at.q_norm, at.k_norm, rope[0], rope[1], hq, hkv, cfg.rms_norm_eps)
                v = qkv[:, (hq + hkv) * d:].view(T, hkv, d)
                cache.append(li, k, v, meta.slots)
                o = cache.attention(li, q, meta, d ** -0.5, at.window).view(T, hq * d)
            else:
                o = self._paged_attention_reference(qkv, at, rope, cache, meta, li)
            h = at.o_proj(o, x)
            n2 = ops.rms_norm(h, layer.post_attention_layernorm, cfg.rms_norm_eps)
            x = layer.mlp(n2, h)
        if not all_logits:
            last = (meta.q_start + meta.q_lens - 1).long()
            x = x[last]               # RMSNorm is per row, so selecting rows first is equivalent
        head = self.head_weight()
        if (skinny and not return_hidden and x.shape[0] <= GEMV_MAX_ROWS and cfg.final_logit_softcap <= 0
                and head.dtype == torch.bfloat16 and not head.requires_grad):
            from ..ops import native as nat
            return nat.gemv(x.contiguous(), head, self.norm, cfg.rms_norm_eps)      # final norm fused into the head
        x = ops.rms_norm(x, self.norm, cfg.rms_norm_eps)
        return x if return_hidden else self.logits(x)

    def _layer_paged_sharded(self, li, layer, x, rope, cache, meta, native: bool):
        """One layer of the cached forward on a model cut by ``parallel.tp_model.shard_for_serving``: this rank's
        heads and experts (or feed-forward channels) on replicated activations; the two partial results are summed over
        the ranks. The residual enters each sum once, through the epilogue of rank 0's projection."""
        cfg = self.cfg
        at = layer.self_attn
        hq, hkv, d, eps = at.hq_local, at.hkv_local, cfg.head_dim, cfg.rms_norm_eps
        T = x.shape[0]
        first = self.tp_rank == 0
        if native and T <= GEMV_MAX_ROWS and at.qkv_proj.gemv_ok(T) and at.o_proj.gemv_ok(T):
            # a handful of rows: the mat-vec kernels with the norm, the cache append and the residual fused in
            from ..ops import native as nat
            qkv = at.qkv_proj.gemv_forward(x, layer.input_layernorm, eps)
            if cache.quant is None:
                q = nat.qknorm_rope_cache(qkv, at.q_norm, at.k_norm, rope[0], rope[1], hq, hkv, eps, cache.k[li],
                                          cache.v[li], meta.slots)
            else:
                q, k = nat.qknorm_rope_fwd(qkv, at.q_norm, at.k_norm, rope[0], rope[1], hq, hkv, eps)
                cache.append(li, k, qkv[:, (hq + hkv) * d:].view(T, hkv, d), meta.slots)
            o = cache.attention(li, q, meta, d ** -0.5, at.window).view(T, hq * d)
            h = at.tp_reduce(at.o_proj.gemv_forward(o, residual=x if first else None))
            if isinstance(layer.mlp, MLP) and layer.mlp.gate_up_proj.gemv_ok(T) and layer.mlp.down_proj.gemv_ok(T):
                act = layer.mlp.gate_up_proj.gemv_forward(h, layer.post_attention_layernorm, eps, swiglu=True)
                return layer.mlp.tp_reduce(layer.mlp.down_proj.gemv_forward(act, residual=h if first else None))
        else:
            qkv = at.qkv_proj(ops.rms_norm(x, layer.input_layernorm, eps))
            if native:
                from ..ops import native as nat
                q, k = nat.qknorm_rope_fwd(qkv, at.q_norm, at.k_norm, rope[0], rope[1], hq, hkv, eps)
                cache.append(li, k, qkv[:, (hq + hkv) * d:].view(T, hkv, d), meta.slots)
                o = cache.attention(li, q, meta, d ** -0.5, at.window).view(T, hq * d)
            else:
                o = self._paged_attention_reference(qkv, at, rope, cache, meta, li, hq, hkv)
            h = at.tp_reduce(at.o_proj(o, x if first else None))
        n2 = ops.rms_norm(h, layer.post_attention_layernorm, eps)
        if isinstance(layer.mlp, MLP):
            y = layer.mlp.down_proj(ops.swiglu(layer.mlp.gate_up_proj(n2)), h if first else None)
            return layer.mlp.tp_reduce(y)
        from ..parallel.tp_model import moe_local_forward
        return moe_local_forward(layer.mlp, n2, h)

    def _mega_ok(self, T: int) -> bool:
        """The whole-step kernel covers dense layers with plain bf16 weights: no adapters, biases, sliding windows or
        soft-capping."""
        if not hasattr(self, "_mega_scratch"):
            self._mega_scratch = {}
            self._mega_tables = {}
        cfg = self.cfg
        ok = cfg.attn_logit_softcap <= 0 and cfg.head_dim == 128 and getattr(self, "tp_world", 1) == 1
        if ok:            # checked on every call: adapters or packed weights may have been attached since the last one
            for layer in self.layers:
                at = layer.self_attn
                if not isinstance(layer.mlp, MLP) or at.window:
                    ok = False
                    break
                for lin in (at.qkv_proj, at.o_proj, layer.mlp.gate_up_proj, layer.mlp.down_proj):
                    if (lin.lora_a is not None or getattr(lin, "qweight", None) is not None or not lin.gemv_ok(1)
                            or not lin.weight.is_contiguous()):
                        ok = False
                        break
                if not ok:
                    break
        if not ok:
            return False
        from ..ops import native as nat
        cfg = self.cfg
        return nat.decode_layers_supported(T, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                                           cfg.intermediate_size)

    def _mega_table(self, cache) -> torch.Tensor:
        """Per-layer pointer table of the whole-step kernel for this cache. Entries are tied to the cache object by a
        weak reference, so a new cache that happens to reuse the id of a freed one gets a fresh table."""
        import weakref
        ent = self._mega_tables.get(id(cache))
        sig = (self.layers[0].self_attn.qkv_proj.weight.data_ptr(), self.layers[-1].mlp.down_proj.weight.data_ptr(),
               cache.k[0].data_ptr())
        if ent is not None and ent[0]() is cache and ent[2] == sig:      # same cache object, weights not re-allocated
            return ent[1]
        for key in [k for k, e in self._mega_tables.items() if e[0]() is None]:
            del self._mega_tables[key]
        rows = []
        for li, layer in enumerate(self.layers):
            at, mlp = layer.self_attn, layer.mlp
            rows.append([layer.input_layernorm.data_ptr(), at.qkv_proj.weight.data_ptr(),
                         at.q_norm.data_ptr() if at.q_norm is not None else 0,
                         at.k_norm.data_ptr() if at.k_norm is not None else 0, at.o_proj.weight.data_ptr(),
                         layer.post_attention_layernorm.data_ptr(), mlp.gate_up_proj.weight.data_ptr(),
                         mlp.down_proj.weight.data_ptr(), cache.k[li].data_ptr(), cache.v[li].data_ptr()])
        t = torch.tensor(rows, dtype=torch.int64, device=self.embed_tokens.device)
        self._mega_tables[id(cache)] = (weakref.ref(cache), t, sig)
        return t

    def _paged_attention_reference(self, qkv, at, rope, cache, meta, li, hq=None, hkv=None):
        from ..ops import reference as ref
        cfg = self.cfg
        d = cfg.head_dim
        hq = hq if hq is not None else cfg.num_attention_heads
        hkv = hkv if hkv is not None else cfg.num_key_value_heads
        T = qkv.shape[0]
        q = qkv[:, :hq * d].view(T, hq, d)
        k = qkv[:, hq * d:(hq + hkv) * d].view(T, hkv, d)
        v = qkv[:, (hq + hkv) * d:].view(T, hkv, d)
        if at.q_norm is not None:
            q, k = ref.rms_norm(q, at.q_norm, cfg.rms_norm_eps), ref.rms_norm(k, at.k_norm, cfg.rms_norm_eps)
        q, k = ref.apply_rope(q, rope[0], rope[1]), ref.apply_rope(k, rope[0], rope[1])
        cache.write_reference(li, k, v, meta.slots)
        win = min(w for w in (at.window, cache.window) if w > 0) if (at.window > 0 or cache.window > 0) else 0
        sink = cache.sink if cache.window > 0 else 0
        out = torch.empty(T, hq, d, dtype=qkv.dtype, device=qkv.device)
        qs, ql, sl = meta.q_start.tolist(), meta.q_lens.tolist(), meta.seq_lens.tolist()
        rep = hq // hkv
        for i in range(len(ql)):
            K, V = cache.gather_blocks(li, meta.block_table[i], sl[i])      # from the metadata alone: ranks that follow
            # another rank's scheduler hold no per-sequence state
            L, n = K.shape[0], ql[i]
            qq = q[qs[i]:qs[i] + n].transpose(0, 1).float()
            kk = K.transpose(0, 1).float().repeat_interleave(rep, 0)
            vv = V.transpose(0, 1).float().repeat_interleave(rep, 0)
            sc = torch.matmul(qq, kk.transpose(1, 2)) * d ** -0.5
            qpos = torch.arange(L - n, L, device=qkv.device)[:, None]
            kpos = torch.arange(L, device=qkv.device)[None, :]
            mask = kpos <= qpos
            if win > 0:
                mask &= (kpos > qpos - win) | (kpos < sink)
            sc = sc.masked_fill(~mask, float("-inf"))
            out[qs[i]:qs[i] + n] = torch.matmul(sc.softmax(-1), vv).transpose(0, 1).to(out.dtype)
        return out.view(T, hq * d)

    def new_cache(self, num_blocks: int, dtype=None, device=None, quant=None, window: int = 0, sink: int = 0):
        from .kv_cache import PagedKVCache
        p = self.embed_tokens
        return PagedKVCache(self.cfg.num_hidden_layers, getattr(self, "kv_heads_local", self.cfg.num_key_value_heads),
                            self.cfg.head_dim, num_blocks, dtype or p.dtype, device or p.device, quant=quant,
                            window=window, sink=sink)

    # ------------------------------------------------------------------ checkpoint name mapping
    def hf_state_dict(self, merged: bool = False) -> Dict[str, torch.Tensor]:
        sd: Dict[str, torch.Tensor] = {"model.embed_tokens.weight": self.embed_tokens.detach(),
                                       "model.norm.weight": self.norm.detach()}
        if self.lm_head is not None:
            sd["lm_head.weight"] = self.lm_head.detach()
        for i, layer in enumerate(self.layers):
            p = f"model.layers.{i}."
            sd[p + "input_layernorm.weight"] = layer.input_layernorm.detach()
            sd[p + "post_attention_layernorm.weight"] = layer.post_attention_layernorm.detach()
            at = layer.self_attn
            if at.q_norm is not None:
                sd[p + "self_attn.q_norm.weight"] = at.q_norm.detach()
                sd[p + "self_attn.k_norm.weight"] = at.k_norm.detach()
            groups = [("self_attn.", at.qkv_proj), ("self_attn.", at.o_proj)]
            if isinstance(layer.mlp, MLP):
                groups += [("mlp.", layer.mlp.gate_up_proj), ("mlp.", layer.mlp.down_proj)]
            else:
                sd.update({p + "mlp." + k: v for k, v in layer.mlp.hf_state_dict().items()})
            for pre, fl in groups:
                w = fl.merged_weight().to(fl.weight.dtype) if merged else fl.weight.detach()
                o = 0
                for nm, sz in zip(fl.seg_names, fl.seg_sizes):
                    sd[p + pre + nm + ".weight"] = w[o:o + sz]
                    if fl.bias is not None:
                        sd[p + pre + nm + ".bias"] = fl.bias.detach()[o:o + sz]
                    o += sz
        return sd

    @torch.no_grad()
    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor], strict: bool = True) -> List[str]:
        """Copy tensors named like a Hugging Face checkpoint into the fused layout. Returns unused keys."""
        used = set()

        def take(name, dst):
            if name not in sd:
                if strict:
                    raise KeyError(f"missing weight {name}")
                return
            dst.copy_(sd[name].to(dst.dtype))
            used.add(name)

        take("model.embed_tokens.weight", self.embed_tokens)
        take("model.norm.weight", self.norm)
        if self.lm_head is not None:
            if "lm_head.weight" in sd:
                take("lm_head.weight", self.lm_head)
            else:
                self.lm_head.copy_(self.embed_tokens)
        for i, layer in enumerate(self.layers):
            p = f"model.layers.{i}."
            take(p + "input_layernorm.weight", layer.input_layernorm)
            take(p + "post_attention_layernorm.weight", layer.post_attention_layernorm)
            at = layer.self_attn
            if at.q_norm is not None:
                take(p + "self_attn.q_norm.weight", at.q_norm)
                take(p + "self_attn.k_norm.weight", at.k_norm)
            groups = [("self_attn.", at.qkv_proj), ("self_attn.", at.o_proj)]
            if isinstance(layer.mlp, MLP):
                groups += [("mlp.", layer.mlp.gate_up_proj), ("mlp.", layer.mlp.down_proj)]
            else:
                used |= layer.mlp.load_hf_state_dict(sd, p + "mlp.", strict)
            for pre, fl in groups:
                o = 0
                for nm, sz in zip(fl.seg_names, fl.seg_sizes):
                    take(p + pre + nm + ".weight", fl.weight[o:o + sz])
                    if fl.bias is not None:
                        take(p + pre + nm + ".bias", fl.bias[o:o + sz])
                    o += sz
        return [k for k in sd if k not in used]

    def num_parameters(self, trainable_only: bool = False) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad or not trainable_only)
