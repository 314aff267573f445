"""AdamW over one flat parameter buffer.

Update rule and parameter classes follow the reference
(crates/pmetal-bridge/src/optimizer.rs:215-356): bias-corrected Adam step, then
decoupled decay applied to the already-updated parameter; parameters whose name
contains ``bias|norm|scale`` get no decay, ``embed|lm_head`` use the embedding
learning rate, ``lora_b`` uses ``lr · loraplus_ratio``.

All trainable parameters are re-homed as views into one fp32 buffer (gradients into
a second one), so that one kernel launch performs global-norm clipping and the
update for every tensor, writes the bf16 shadow copy the GEMMs read, and — in
data-parallel runs — can be fused with the gradient reduction
(``pmetal_b200.parallel.fused_dp``). Per-tensor learning-rate multiplier and decay
live in a small table indexed by 1024-element chunk, which keeps LoRA+ and
embedding learning rates available on the fused path (the reference's fused Metal
optimizer cannot do that, run_metal_fused.rs:33-40).
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Tuple

import torch

from ..ops import reference as ref

CHUNK = 1024


def classify_param(name: str) -> str:
    if "bias" in name or "norm" in name or "scale" in name:
        return "no_decay"
    if "embed" in name or "lm_head" in name:
        return "embedding"
    if "lora_b" in name:
        return "lora_b"
    return "regular"


class FlatAdamW:
    def __init__(self, named_params: Iterable[Tuple[str, torch.nn.Parameter]], lr: float = 2e-4,
                 betas: Tuple[float, float] = (0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 embedding_lr: Optional[float] = 5e-5, loraplus_ratio: Optional[float] = None,
                 max_grad_norm: float = 0.0, shadow_dtype: Optional[torch.dtype] = None, bias_correction: bool = True):
        """``bias_correction=False`` uses the running moments as they are (the plain variant of the reference's fused
        update, fused_training.metal: ``fused_adamw_update`` next to ``fused_adamw_update_bias_corrected``)."""
        self.bias_correction = bias_correction
        self.named = [(n, p) for n, p in named_params if p.requires_grad]
        if not self.named:
            raise ValueError("no trainable parameters")
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.embedding_lr, self.loraplus_ratio, self.max_grad_norm = embedding_lr, loraplus_ratio, max_grad_norm
        self.step_count = 0
        dev = self.named[0][1].device
        self.device = dev
        offs, total = [], 0
        for _, p in self.named:
            offs.append(total)
            total += -(-p.numel() // CHUNK) * CHUNK
        self.offsets, self.total = offs, total
        self.flat_p = torch.zeros(total, dtype=torch.float32, device=dev)
        self.flat_g = torch.zeros(total, dtype=torch.float32, device=dev)
        self.flat_m = torch.zeros(total, dtype=torch.float32, device=dev)
        self.flat_v = torch.zeros(total, dtype=torch.float32, device=dev)
        self.flat_shadow = torch.zeros(total, dtype=shadow_dtype, device=dev) if shadow_dtype else None
        lr_mult = torch.ones(total // CHUNK, dtype=torch.float32)
        wd_tab = torch.zeros(total // CHUNK, dtype=torch.float32)
        self.classes: Dict[str, str] = {}
        self.shadows: Dict[str, torch.Tensor] = {}
        for (n, p), o in zip(self.named, offs):
            cls = classify_param(n)
            self.classes[n] = cls
            mult, wd = 1.0, weight_decay
            if cls == "no_decay":
                wd = 0.0
            elif cls == "embedding" and embedding_lr is not None:
                mult = embedding_lr / lr if lr > 0 else 1.0
            elif cls == "lora_b" and loraplus_ratio:
                mult = loraplus_ratio
            c0, c1 = o // CHUNK, (o + p.numel() + CHUNK - 1) // CHUNK
            lr_mult[c0:c1], wd_tab[c0:c1] = mult, wd
            with torch.no_grad():
                self.flat_p[o:o + p.numel()].copy_(p.detach().float().reshape(-1))
                p.data = self.flat_p[o:o + p.numel()].view(p.shape)
                p.grad = self.flat_g[o:o + p.numel()].view(p.shape)
                if self.flat_shadow is not None:
                    sh = self.flat_shadow[o:o + p.numel()].view(p.shape)
                    sh.copy_(p.data)
                    self.shadows[n] = sh
        self.lr_mult = lr_mult.to(dev)
        self.wd_tab = wd_tab.to(dev)
        self.grad_norm = torch.zeros(1, dtype=torch.float32, device=dev)
        # [lr, 1-beta1^t, 1-beta2^t] on the device; used instead of scalars while replaying a CUDA graph
        self._hp = torch.zeros(4, dtype=torch.float32, device=dev) if dev.type == "cuda" else None
        self._hp_host = torch.zeros(4, dtype=torch.float32).pin_memory() if dev.type == "cuda" else None
        self.device_hparams = False

    def rehome(self, flat_p: torch.Tensor, flat_g: torch.Tensor, flat_shadow: Optional[torch.Tensor]) -> None:
        """Adopt externally allocated flat buffers (e.g. symmetric memory); contents must already be copied."""
        self.flat_p, self.flat_g = flat_p, flat_g
        if flat_shadow is not None:
            self.flat_shadow = flat_shadow
        for (n, p), o in zip(self.named, self.offsets):
            p.data = self.flat_p[o:o + p.numel()].view(p.shape)
            p.grad = self.flat_g[o:o + p.numel()].view(p.shape)
            if self.flat_shadow is not None:
                self.shadows[n] = self.flat_shadow[o:o + p.numel()].view(p.shape)

    # ---------------------------------------------------------------- helpers
    def zero_grad(self) -> None:
        self.flat_g.zero_()
        for (_, p), o in zip(self.named, self.offsets):      # re-attach in case autograd replaced .grad
            if p.grad is None or p.grad.data_ptr() != self.flat_g.data_ptr() + 4 * o:
                p.grad = self.flat_g[o:o + p.numel()].view(p.shape)

    def set_lr(self, lr: float) -> None:
        self.lr = lr

    def _use_native(self) -> bool:
        if self.device.type != "cuda":
            return False
        from ..ops import native
        return native.available()

    def compute_grad_norm(self) -> torch.Tensor:
        if self._use_native():
            from ..ops import native
            native.sumsq(self.flat_g, self.grad_norm)
            return self.grad_norm.sqrt()
        self.grad_norm = (self.flat_g.double() ** 2).sum().sqrt().float().reshape(1)
        return self.grad_norm

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0) -> torch.Tensor:
        """One update. ``grad_scale`` multiplies every gradient first (e.g. 1/accumulation).
        Returns the pre-clip global gradient norm (device tensor, no host sync)."""
        self.step_count += 1
        b1, b2 = self.betas
        if self._use_native():
            from ..ops import native
            native.sumsq(self.flat_g, self.grad_norm)
            native.adamw_flat(self.flat_p, self.flat_g, self.flat_m, self.flat_v, self.flat_shadow, self.lr_mult,
                              self.wd_tab, self.grad_norm, self.lr, b1, b2, self.eps,
                              self.step_count if self.bias_correction else 0, grad_scale,
                              self.max_grad_norm, self._hp if self.device_hparams else None)
            return self.grad_norm.sqrt() * grad_scale
        if grad_scale != 1.0:
            self.flat_g.mul_(grad_scale)
        norm = (self.flat_g.double() ** 2).sum().sqrt().float()
        if self.max_grad_norm and self.max_grad_norm > 0:
            coef = torch.clamp(self.max_grad_norm / (norm + 1e-6), max=1.0)
            self.flat_g.mul_(coef)
        for (n, p), o in zip(self.named, self.offsets):
            k = p.numel()
            c = o // CHUNK
            ref.adamw_step(self.flat_p[o:o + k], self.flat_g[o:o + k], self.flat_m[o:o + k], self.flat_v[o:o + k],
                           self.step_count if self.bias_correction else 0, self.lr * float(self.lr_mult[c]), b1, b2,
                           self.eps, float(self.wd_tab[c]))
        if self.flat_shadow is not None:
            self.flat_shadow.copy_(self.flat_p)
        return norm.reshape(1)

    def push_hparams(self, step: int) -> None:
        """Stage lr and the bias corrections of ``step`` on the device (call before replaying a captured step)."""
        b1, b2 = self.betas
        if not self.bias_correction:
            step = 0
        self._hp_host[0] = self.lr
        self._hp_host[1], self._hp_host[2] = (1 - b1 ** step, 1 - b2 ** step) if step > 0 else (1.0, 1.0)
        self._hp.copy_(self._hp_host, non_blocking=True)

    # ---------------------------------------------------------------- state
    def state_dict(self) -> dict:
        return {"step": self.step_count, "m": self.flat_m.cpu(), "v": self.flat_v.cpu(),
                "names": [n for n, _ in self.named], "offsets": list(self.offsets)}

    def load_state_dict(self, sd: dict) -> None:
        if list(sd["names"]) != [n for n, _ in self.named]:
            raise ValueError("optimizer state does not match the parameter list")
        self.step_count = int(sd["step"])
        self.flat_m.copy_(sd["m"])
        self.flat_v.copy_(sd["v"])

    def sync_shadow(self) -> None:
        if self.flat_shadow is not None:
            self.flat_shadow.copy_(self.flat_p)


def attach_shadows(model, opt: FlatAdamW) -> None:
    """Point every fused linear at the bf16 shadow of its LoRA factors so forward never casts."""
    byname = dict(model.named_parameters())
    ids = {id(p): n for n, p in byname.items()}
    for _, _, fl in model.fused_linears():
        if fl.lora_a is not None:
            fl.lora_a_c = opt.shadows.get(ids[id(fl.lora_a)])
            fl.lora_b_c = opt.shadows.get(ids[id(fl.lora_b)])
    # full-parameter training: every fp32 master that trains carries its bf16 shadow, which the kernels read
    # (ops.functional.live / dense_linear); adapter factors keep their own route above
    for n, p in byname.items():
        if "lora_" in n or not p.requires_grad or p.dtype != torch.float32:
            continue
        sh = opt.shadows.get(n)
        if sh is not None:
            p.shadow = sh
