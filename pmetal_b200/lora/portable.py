"""LoRA for the portable architecture implementations (``models/architectures``): Gemma, Phi, Cohere, Granite,
DeepSeek, GPT-OSS, Llama 4, Mixtral, Qwen3-Next, Nemotron-H and the encoders.

The hand-written kernels fuse LoRA into the projections of the fast decoder (``lora/adapter.py``); every other family
gets adapters as plain modules wrapped around its ``nn.Linear`` projections: ``y = W x + s * B (A x)`` with ``A`` drawn
from U(+-sqrt(3 / in)) (rsLoRA: +-sqrt(1 / r)), ``B = 0`` and ``s = alpha / r`` (``alpha / sqrt(r)``), DoRA optionally on
top (column-norm magnitude vector). Adapter files use the same key format as the fast path and the reference
(``layers.N.self_attn.q_proj.lora_a`` [r, in] / ``.lora_b`` [out, r], no ``model.`` prefix; crates/pmetal-lora/src/
lora_helpers.rs:33-250, crates/pmetal-lora/src/dynamic.rs:125-600 dispatches one wrapper type per architecture), so an
adapter can be fused into the base weights by ``pmetal fuse`` whatever produced it."""
from __future__ import annotations

import math
import os
from typing import Dict, Iterable, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..core.config import LoraConfig
from ..utils import safetensors_io as st

WEIGHTS_NAME = "lora_weights.safetensors"


class LoraLinear(nn.Module):
    def __init__(self, base: nn.Linear, r: int, scale: float, rslora: bool = False, dora: bool = False,
                 generator: Optional[torch.Generator] = None):
        super().__init__()
        self.base, self.r, self.scale = base, r, scale
        bound = math.sqrt(1.0 / r) if rslora else math.sqrt(3.0 / base.in_features)
        a = (torch.rand(r, base.in_features, generator=generator) * 2 - 1) * bound
        self.lora_a = nn.Parameter(a.to(base.weight.device))
        self.lora_b = nn.Parameter(torch.zeros(base.out_features, r, device=base.weight.device))
        self.magnitude = None
        if dora:                                # per-output-row norm of the adapted weight, initialised from the base
            self.magnitude = nn.Parameter(base.weight.detach().float().norm(dim=1).to(base.weight.device))
        for p in base.parameters():
            p.requires_grad_(False)

    @property
    def weight(self):
        return self.base.weight

    def delta(self) -> torch.Tensor:
        return self.scale * (self.lora_b.float() @ self.lora_a.float())

    def forward(self, x):
        if self.magnitude is None:
            lo = F.linear(F.linear(x.to(self.lora_a.dtype), self.lora_a), self.lora_b) * self.scale
            return self.base(x) + lo.to(x.dtype)
        w = self.base.weight.float() + self.delta()
        w = w * (self.magnitude.float() / w.norm(dim=1).clamp(min=1e-8))[:, None]
        return F.linear(x, w.to(x.dtype), self.base.bias)

    @torch.no_grad()
    def merged_weight(self) -> torch.Tensor:
        w = self.base.weight.double() + self.delta().double()
        if self.magnitude is not None:
            w = w * (self.magnitude.double() / w.norm(dim=1).clamp(min=1e-8))[:, None]
        return w.to(self.base.weight.dtype)


class QuantLinear(nn.Module):
    """A frozen projection whose weight is stored as 4-bit (NF4 / FP4) or int8 blocks and expanded into a transient
    matrix of the activation's type at every use: the QLoRA base for the config-driven architectures
    (crates/pmetal-lora/src/qlora.rs:33-480). It offers what ``LoraLinear`` asks of its base: ``weight`` (dequantised on
    access), ``bias``, ``in_features`` / ``out_features`` and a forward."""

    def __init__(self, linear: nn.Linear, scheme: str = "nf4", block_size: int = 64, double_quant: bool = False):
        super().__init__()
        from .nf4 import quantize
        self.in_features, self.out_features = linear.in_features, linear.out_features
        self.dtype = linear.weight.dtype
        q = quantize(linear.weight.detach(), scheme, block_size, double_quant)
        self.qweight = q.to(linear.weight.device) if q.data.device != linear.weight.device else q
        self.bias = None if linear.bias is None else nn.Parameter(linear.bias.detach().clone(), requires_grad=False)

    @property
    def weight(self) -> torch.Tensor:
        from .qlora import dequantize_weight
        return dequantize_weight(self.qweight, self.dtype)

    def forward(self, x):
        return F.linear(x, self.weight.to(x.dtype), self.bias)

    def _apply(self, fn, recurse=True):            # .to(device) / .cuda() move the packed blocks too
        super()._apply(fn, recurse)
        probe = fn(torch.empty(0, device=self.qweight.data.device))
        if probe.device != self.qweight.data.device:
            self.qweight = self.qweight.to(probe.device)
        return self


@torch.no_grad()
def quantize_base_portable(model: nn.Module, scheme: str = "nf4", block_size: int = 64, double_quant: bool = False,
                           skip: Iterable[str] = ("lm_head", "embed_tokens", "router", "gate")) -> int:
    """Replace every ``nn.Linear`` of the decoder blocks by a :class:`QuantLinear`; read-out, embeddings and routers keep
    their precision. Call before ``apply_lora_portable``. Returns the bytes saved."""
    skip = set(skip)
    saved = 0
    for full, mod in list(model.named_modules()):
        for name, child in list(mod.named_children()):
            if type(child).__name__ in ("Linear",) and isinstance(child, nn.Linear) and name not in skip:
                q = QuantLinear(child, scheme, block_size, double_quant)
                saved += child.weight.numel() * child.weight.element_size() - q.qweight.nbytes()
                setattr(mod, name, q)
    return saved


def _targets(model: nn.Module, names: Iterable[str]) -> List[Tuple[nn.Module, str, str]]:
    want = set(names)
    out = []
    for full, mod in model.named_modules():
        for child_name, child in mod.named_children():
            if isinstance(child, (nn.Linear, QuantLinear)) and child_name in want:
                out.append((mod, child_name, f"{full}.{child_name}" if full else child_name))
    return out


def apply_lora_portable(model: nn.Module, cfg: LoraConfig, seed: int = 42) -> nn.Module:
    """Wrap every ``nn.Linear`` whose attribute name is in ``cfg.target_modules`` and freeze all other parameters."""
    g = torch.Generator().manual_seed(seed)
    for p in model.parameters():
        p.requires_grad_(False)
    hits = _targets(model, cfg.target_modules)
    if not hits:
        raise ValueError(f"no projection named one of {sorted(cfg.target_modules)} in {type(model).__name__}")
    for parent, name, _ in hits:
        setattr(parent, name, LoraLinear(getattr(parent, name), cfg.r, cfg.scaling(), cfg.use_rslora,
                                         getattr(cfg, "use_dora", False), g))
    return model


def _key(path: str) -> str:
    for prefix in ("model.language_model.", "model.", "backbone."):
        if path.startswith(prefix):
            return path[len(prefix):]
    return path


def lora_modules(model: nn.Module) -> Dict[str, LoraLinear]:
    return {_key(n): m for n, m in model.named_modules() if isinstance(m, LoraLinear)}


def lora_state_dict(model: nn.Module) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for key, m in lora_modules(model).items():
        out[key + ".lora_a"] = m.lora_a.detach().float().cpu().contiguous()
        out[key + ".lora_b"] = m.lora_b.detach().float().cpu().contiguous()
        if m.magnitude is not None:
            out[key + ".magnitude"] = m.magnitude.detach().float().cpu().reshape(-1, 1).contiguous()
    return out


def save_adapter_portable(model: nn.Module, out_dir: str, cfg: LoraConfig, base_model: Optional[str] = None) -> str:
    from .adapter import save_adapter_config
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, WEIGHTS_NAME)
    st.save_file(lora_state_dict(model), path, metadata={"format": "mlx"})
    save_adapter_config(out_dir, cfg, base_model)
    return path


def load_adapter_portable(model: nn.Module, path: str) -> int:
    """Copy adapter tensors into the wrapped projections; unknown keys are ignored. Returns the number loaded."""
    from .adapter import resolve_adapter_file
    sd = st.load_file(resolve_adapter_file(path))
    n = 0
    with torch.no_grad():
        for key, m in lora_modules(model).items():
            a, b = sd.get(key + ".lora_a"), sd.get(key + ".lora_b")
            if a is None or b is None or a.shape != m.lora_a.shape or b.shape != m.lora_b.shape:
                continue
            m.lora_a.copy_(a)
            m.lora_b.copy_(b)
            mag = sd.get(key + ".magnitude")
            if mag is not None and m.magnitude is not None:
                m.magnitude.copy_(mag.reshape(-1))
            n += 1
    return n


def merge_lora_portable(model: nn.Module) -> nn.Module:
    """Fold every adapter into its base weight and put the plain ``nn.Linear`` back."""
    for full, mod in list(model.named_modules()):
        for name, child in list(mod.named_children()):
            if isinstance(child, LoraLinear):
                w = child.merged_weight()
                base = child.base
                if isinstance(base, QuantLinear):          # a packed base comes back as a plain matrix of its original type
                    lin = nn.Linear(base.in_features, base.out_features, bias=base.bias is not None, device=w.device, dtype=w.dtype)
                    if base.bias is not None:
                        lin.bias.data.copy_(base.bias)
                    lin.requires_grad_(False)
                    base = lin
                base.weight.data.copy_(w)
                setattr(mod, name, base)
    return model


# ------------------------------------------------------------------------------------------------ training
def causal_lm_loss(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Mean next-token cross entropy: position t predicts labels[t + 1]."""
    return F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(), labels[:, 1:].reshape(-1),
                           ignore_index=ignore_index)


class PortableLoraTrainer:
    """Padded-batch supervised fine-tuning of adapters on a portable model: ``torch.optim.AdamW`` (bias-corrected,
    decoupled decay), global-norm clipping, warm-up + cosine schedule, optional LoRA+ learning-rate ratio for ``B``."""

    def __init__(self, model: nn.Module, learning_rate: float = 2e-4, weight_decay: float = 0.01, max_grad_norm: float = 1.0,
                 warmup_steps: int = 0, total_steps: int = 1000, schedule: str = "cosine", loraplus_ratio: Optional[float] = None):
        from ..core.scheduler import LearningRateScheduler
        self.model = model
        params = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        if not params:
            raise ValueError("the model has no trainable parameters (apply_lora_portable first)")
        ratio = loraplus_ratio or 1.0
        groups = [{"params": [p for n, p in params if "lora_b" not in n], "lr_mult": 1.0},
                  {"params": [p for n, p in params if "lora_b" in n], "lr_mult": ratio}]
        self.groups = [g for g in groups if g["params"]]
        self.opt = torch.optim.AdamW([{"params": g["params"]} for g in self.groups], lr=learning_rate, betas=(0.9, 0.999),
                                     eps=1e-8, weight_decay=weight_decay)
        self.sched = LearningRateScheduler(learning_rate, total_steps, warmup_steps, schedule)
        self.max_grad_norm, self.step_count = max_grad_norm, 0

    def micro_step(self, input_ids: torch.Tensor, labels: torch.Tensor, scale: float = 1.0,
                   positions: Optional[torch.Tensor] = None, doc_ids: Optional[torch.Tensor] = None) -> float:
        """Forward + backward of one micro-batch; ``scale`` (1 / accumulation steps) multiplies its loss so that the
        accumulated gradient is the mean over the micro-batches. Gradients add up until ``optimizer_step``.
        ``positions`` / ``doc_ids`` [B, T] describe packed rows (several documents per row)."""
        loss = self.loss(input_ids, labels, positions, doc_ids)
        (loss * scale if scale != 1.0 else loss).backward()
        return float(loss.detach())

    def loss(self, input_ids: torch.Tensor, labels: torch.Tensor, positions: Optional[torch.Tensor] = None,
             doc_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Mean next-token cross entropy. Models that expose their read-out matrix (``loss_head``) get the chunked
        linear + cross-entropy (logit scale and soft cap inside it), so the [batch, tokens, vocabulary] logits are never
        formed; the others go through their own ``forward``. Packed rows pass their per-document positions and document
        ids; their labels are expected to be masked at every document start."""
        packed = {} if doc_ids is None else {"positions": positions, "doc_ids": doc_ids}
        spec = getattr(self.model, "loss_head", None)
        spec = spec() if callable(spec) else None
        if spec is None or input_ids.dim() != 2:
            return causal_lm_loss(self.model(input_ids, **packed), labels)
        from ..ops import functional as ops
        w, factor, cap = spec
        h = self.model.forward_hidden(input_ids, **packed)
        hs = h[:, :-1].reshape(-1, h.shape[-1])
        s, n = ops.linear_cross_entropy(hs, w, labels[:, 1:].reshape(-1), softcap=cap, logit_scale=factor)
        return s / n.clamp(min=1).to(s.dtype)

    def optimizer_step(self) -> dict:
        lr = self.sched.get_lr(self.step_count)
        for g, meta in zip(self.opt.param_groups, self.groups):
            g["lr"] = lr * meta["lr_mult"]
        gn = torch.nn.utils.clip_grad_norm_([p for g in self.groups for p in g["params"]], self.max_grad_norm or float("inf"))
        self.opt.step()
        self.opt.zero_grad(set_to_none=True)
        self.step_count += 1
        return {"grad_norm": float(gn), "lr": lr}

    def step(self, input_ids: torch.Tensor, labels: torch.Tensor) -> dict:
        """One optimiser step on one batch (no accumulation)."""
        self.opt.zero_grad(set_to_none=True)
        loss = self.micro_step(input_ids, labels)
        return {"loss": loss, **self.optimizer_step()}

    # -- resume: step counter (drives the schedule) and the optimiser moments
    def state_dict(self) -> dict:
        return {"step": self.step_count, "optimizer": self.opt.state_dict()}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd["step"])
        self.opt.load_state_dict(sd["optimizer"])


# ------------------------------------------------------------------------------------------------ Q-BLoRA
class QBLoraLinear(nn.Module):
    """Balanced adapter for quantised bases (Q-BLoRA; crates/pmetal-lora/src/qblora.rs:63-480):

        y = W x + s * (((x P_in) A^T) B^T) P_out

    The adapter sees a simplified input (``P_in`` [in, d_in]) and writes through a simplified output (``P_out``
    [d_out, out]); in exchange its rank is ``rank_multiplier`` times the usual one. Projections are learnable or fixed
    random maps scaled to preserve norms; ``B`` starts at zero, so the adapted layer starts equal to the base layer.
    ``gradient_scale`` multiplies the adapter branch's gradient without changing its forward value."""

    def __init__(self, base: nn.Module, in_features: int, out_features: int, r: int, scale: float,
                 input_proj_dim: Optional[int] = None, output_proj_dim: Optional[int] = None, rank_multiplier: float = 2.0,
                 learnable_projections: bool = True, gradient_scale: float = 1.0, generator: Optional[torch.Generator] = None):
        super().__init__()
        self.base, self.scale, self.gradient_scale = base, scale, gradient_scale
        self.r = max(int(round(r * rank_multiplier)), 1)
        d_in, d_out = input_proj_dim or in_features, output_proj_dim or out_features
        g = generator

        def rnd(*shape, std):
            return torch.randn(*shape, generator=g) * std
        self.lora_a = nn.Parameter((torch.rand(self.r, d_in, generator=g) * 2 - 1) * math.sqrt(3.0 / d_in))
        self.lora_b = nn.Parameter(torch.zeros(d_out, self.r))
        self.p_in = self.p_out = None
        if input_proj_dim:
            p = rnd(in_features, d_in, std=d_in ** -0.5)
            self.p_in = nn.Parameter(p) if learnable_projections else None
            if not learnable_projections:
                self.register_buffer("p_in_fixed", p)
        if output_proj_dim:
            p = rnd(d_out, out_features, std=d_out ** -0.5)
            self.p_out = nn.Parameter(p) if learnable_projections else None
            if not learnable_projections:
                self.register_buffer("p_out_fixed", p)
        for q in base.parameters():
            q.requires_grad_(False)

    def adapter(self, x: torch.Tensor) -> torch.Tensor:
        p_in = self.p_in if self.p_in is not None else getattr(self, "p_in_fixed", None)
        p_out = self.p_out if self.p_out is not None else getattr(self, "p_out_fixed", None)
        h = x.to(self.lora_a.dtype)
        if p_in is not None:
            h = h @ p_in
        h = F.linear(F.linear(h, self.lora_a), self.lora_b)
        if p_out is not None:
            h = h @ p_out
        return h * self.scale

    def forward(self, x):
        lo = self.adapter(x)
        if self.gradient_scale != 1.0:                         # same value, scaled gradient
            lo = lo.detach() + self.gradient_scale * (lo - lo.detach())
        return self.base(x) + lo.to(x.dtype)

    def trainable_parameters(self) -> List[nn.Parameter]:
        return [p for p in (self.lora_a, self.lora_b, self.p_in, self.p_out) if p is not None]
