"""Optimiser variants beside the flat fused AdamW: 8-bit Adam, schedule-free AdamW, parameter groups.

* ``Adam8bit`` (crates/pmetal-trainer/src/adam8bit.rs): first and second moments stored as int8 / uint8 with one fp32 absmax
  scale per block of 2048 elements (dynamic block-wise quantisation), dequantised block by block inside the step.
* ``ScheduleFreeAdamW`` (crates/pmetal-trainer/src/schedule_free.rs): the schedule-free method of Defazio et al. — the
  gradient is evaluated at y = (1 - beta1) z + beta1 x, z takes the Adam step, x is the running average of z; ``eval()`` /
  ``train()`` switch the parameters between x and y.
* ``build_param_groups`` (crates/pmetal-trainer/src/param_groups.rs): no-decay for bias / norm / scale, separate LR for
  embeddings and for LoRA B (LoRA+)."""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Tuple

import torch

BLOCK = 2048


def _quant_blockwise(x: torch.Tensor, signed: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    flat = x.reshape(-1)
    pad = (-flat.numel()) % BLOCK
    if pad:
        flat = torch.cat([flat, flat.new_zeros(pad)])
    blocks = flat.view(-1, BLOCK)
    amax = blocks.abs().amax(1).clamp(min=1e-12)
    if signed:
        q = torch.round(blocks / amax[:, None] * 127).clamp(-127, 127).to(torch.int8)
    else:
        q = torch.round(torch.sqrt(blocks / amax[:, None]) * 255).clamp(0, 255).to(torch.uint8)   # sqrt companding for v >= 0
    return q, amax


def _dequant_blockwise(q: torch.Tensor, amax: torch.Tensor, n: int, signed: bool) -> torch.Tensor:
    if signed:
        x = q.float() / 127 * amax[:, None]
    else:
        x = (q.float() / 255) ** 2 * amax[:, None]
    return x.reshape(-1)[:n]


class Adam8bit(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, min_8bit_size: int = 4096):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.min_8bit_size = min_8bit_size

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                n = p.numel()
                small = n < self.min_8bit_size
                if not st:
                    st["step"] = 0
                    if small:
                        st["m"], st["v"] = torch.zeros_like(p, dtype=torch.float32), torch.zeros_like(p, dtype=torch.float32)
                    else:
                        st["mq"], st["ms"] = _quant_blockwise(torch.zeros(n, device=p.device), True)
                        st["vq"], st["vs"] = _quant_blockwise(torch.zeros(n, device=p.device), False)
                st["step"] += 1
                grad = p.grad.float().reshape(-1)
                m = st["m"].reshape(-1) if small else _dequant_blockwise(st["mq"], st["ms"], n, True)
                v = st["v"].reshape(-1) if small else _dequant_blockwise(st["vq"], st["vs"], n, False)
                m = b1 * m + (1 - b1) * grad
                v = b2 * v + (1 - b2) * grad * grad
                mh = m / (1 - b1 ** st["step"])
                vh = v / (1 - b2 ** st["step"])
                upd = mh / (vh.sqrt() + g["eps"])
                pf = p.float().reshape(-1) - g["lr"] * upd
                if g["weight_decay"]:
                    pf = pf - g["lr"] * g["weight_decay"] * pf
                p.copy_(pf.view_as(p).to(p.dtype))
                if small:
                    st["m"], st["v"] = m.view_as(p), v.view_as(p)
                else:
                    st["mq"], st["ms"] = _quant_blockwise(m, True)
                    st["vq"], st["vs"] = _quant_blockwise(v, False)

    def state_bytes(self) -> int:
        tot = 0
        for st in self.state.values():
            for k, t in st.items():
                if isinstance(t, torch.Tensor):
                    tot += t.numel() * t.element_size()
        return tot


class ScheduleFreeAdamW(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, warmup_steps: int = 0, r: float = 0.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, warmup_steps=warmup_steps,
                                      r=r, k=0, lr_sum=0.0, train_mode=True))

    @torch.no_grad()
    def _swap(self, to_train: bool):
        for g in self.param_groups:
            if g["train_mode"] == to_train:
                continue
            b1 = g["betas"][0]
            for p in g["params"]:
                st = self.state.get(p)
                if st and "z" in st:
                    # y = (1-b1) z + b1 x  <->  x = (y - (1-b1) z) / b1
                    if to_train:
                        p.lerp_(st["z"].to(p.dtype), 1 - b1)
                    else:
                        p.copy_(((p.float() - (1 - b1) * st["z"]) / b1).to(p.dtype))
            g["train_mode"] = to_train

    def train(self):
        self._swap(True)

    def eval(self):
        self._swap(False)

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            g["k"] += 1
            k = g["k"]
            sched = min(1.0, k / g["warmup_steps"]) if g["warmup_steps"] > 0 else 1.0
            lr = g["lr"] * sched * (1 - b2 ** k) ** 0.5
            w = (k ** g["r"]) * (lr ** 2)
            g["lr_sum"] += w
            ck = w / g["lr_sum"] if g["lr_sum"] > 0 else 0.0
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["z"] = p.detach().float().clone()
                    st["v"] = torch.zeros_like(st["z"])
                grad = p.grad.float()
                st["v"].mul_(b2).addcmul_(grad, grad, value=1 - b2)
                upd = grad / (st["v"].sqrt() + g["eps"])
                y = p.float()
                if g["weight_decay"]:
                    upd = upd + g["weight_decay"] * y
                # x_{k+1} = (1-ck) x_k + ck z_{k+1}; expressed on y so that only y and z are stored
                x = (y - (1 - b1) * st["z"]) / b1
                st["z"].sub_(lr * upd)
                x = (1 - ck) * x + ck * st["z"]
                p.copy_(((1 - b1) * st["z"] + b1 * x).to(p.dtype))


def build_param_groups(named_params: Iterable[Tuple[str, torch.nn.Parameter]], lr: float, weight_decay: float = 0.01,
                       embedding_lr: Optional[float] = 5e-5, loraplus_ratio: Optional[float] = None) -> List[Dict]:
    from .optimizer import classify_param
    groups: Dict[str, Dict] = {}
    for n, p in named_params:
        if not p.requires_grad:
            continue
        cls = classify_param(n)
        g_lr, wd = lr, weight_decay
        if cls == "no_decay":
            wd = 0.0
        elif cls == "embedding" and embedding_lr is not None:
            g_lr = embedding_lr
        elif cls == "lora_b" and loraplus_ratio:
            g_lr = lr * loraplus_ratio
        groups.setdefault(cls, {"params": [], "lr": g_lr, "weight_decay": wd, "name": cls})["params"].append(p)
    return list(groups.values())
