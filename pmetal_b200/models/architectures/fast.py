"""Native-kernel routes for the config-driven architectures: the building blocks of ``generic.py`` and its siblings are
ordinary ``torch.nn`` modules (they are checked against Hugging Face on CPU in fp32); on a GPU in bf16 their hot operators
are sent to the same sm_100a kernels as the fast decoder:

* ``Linear``      frozen bf16 projections run on the tcgen05 GEMM forward and for the input gradient (split-K inside the
                  kernel for a handful of rows), bias added on top; trainable or fp32 weights keep ``F.linear``;
* ``rms_norm``    plain RMS norms over the last dimension run on the fused norm kernel;
* ``glu``         gated activations act(gate) * up (SiLU, tanh-GELU, GELU) run as one kernel forward and one backward,
                  reading gate and up in place when they are the two halves of a fused projection;
* ``causal_attention``  full-sequence causal (optionally sliding-window) self-attention without soft-capping, sinks or an
                  explicit mask runs on the varlen flash-attention kernels, every batch row as one document, head sizes
                  below 128 zero-padded.

Everything else (soft-capped logits, attention sinks, chunked masks, cached decode steps, layer norms) stays on the
PyTorch operators. The reference has stand-alone native engines per family
(crates/pmetal-bridge/src/{qwen3,deepseek,gpt_oss,llama4}_native/, gemma4_native.rs); here one set of kernels serves
every family through these entry points."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


import os

# comma-separated routes that are switched on: linear, norm, attention, glu (all by default)
ROUTES = set(os.environ.get("PMETAL_PORTABLE_FAST", "linear,norm,attention,glu").split(","))
GLU_NAMES = {"silu": "silu", "swish": "silu", "gelu_tanh": "gelu_tanh", "gelu_pytorch_tanh": "gelu_tanh", "gelu_new": "gelu_tanh",
             "gelu": "gelu"}


def _native(x: torch.Tensor) -> bool:
    if not x.is_cuda or x.dtype != torch.bfloat16:
        return False
    from ...ops import functional as ops
    return ops.use_native(x)


class Linear(nn.Linear):
    """``nn.Linear`` whose forward takes the tensor-core GEMM when the weight is a frozen bf16 matrix."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = self.weight
        if ("linear" in ROUTES and w.dtype == torch.bfloat16 and not w.requires_grad and self.in_features % 8 == 0 and self.out_features % 8 == 0
                and x.numel() > 0 and _native(x)):
            from ...ops import functional as ops
            x2 = x.reshape(-1, self.in_features)
            if x2.stride(-1) != 1 or (x2.stride(0) % 8):
                x2 = x2.contiguous()
            y = ops.lora_linear(x2, w, None, None, None, (self.out_features,), 0, 0.0, None)
            if self.bias is not None:
                y = y + self.bias
            return y.view(*x.shape[:-1], self.out_features)
        return F.linear(x, w, self.bias)


def glu(gate: torch.Tensor, up: torch.Tensor, act_name: str, act_fn) -> torch.Tensor:
    """act(gate) * up; the fused kernel pair when the route is on and the activation is one it knows."""
    name = GLU_NAMES.get(act_name)
    if "glu" in ROUTES and name is not None and _native(gate) and up.dtype == gate.dtype:
        from ...ops import functional as ops
        return ops.glu(gate, up, name)
    return act_fn(gate) * up


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> Optional[torch.Tensor]:
    """weight * x / rms(x) over the last dimension on the fused kernel, or None when the shapes / types do not fit."""
    if "norm" not in ROUTES or weight.dim() != 1 or x.shape[-1] != weight.shape[0] or x.shape[-1] % 8 or weight.dtype != torch.bfloat16 \
            or not _native(x):
        return None
    from ...ops import functional as ops
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    return ops.rms_norm(x2, weight, eps).view(x.shape)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int = 0,
                     doc_ids: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """q [B, h, T, d], k / v [B, hkv, T, d] (same T: no cache) -> [B, h, T, d] with a causal (sliding-window) mask, on the
    varlen kernels; None when the case is not covered. ``doc_ids`` [B, T] (non-decreasing along a row) cuts every row
    into documents that do not see each other."""
    B, h, T, d = q.shape
    if "attention" not in ROUTES or k.shape[2] != T or v.shape[-1] != d or d > 128 or d % 8 or h % k.shape[1] or not _native(q):
        return None
    from ...ops import functional as ops
    hkv = k.shape[1]
    qf = q.transpose(1, 2).reshape(B * T, h, d)
    kf = k.transpose(1, 2).reshape(B * T, hkv, d)
    vf = v.transpose(1, 2).reshape(B * T, hkv, d)
    if d < 128:
        pad = (0, 128 - d)
        qf, kf, vf = F.pad(qf, pad), F.pad(kf, pad), F.pad(vf, pad)
    qf, kf, vf = qf.contiguous(), kf.contiguous(), vf.contiguous()
    if doc_ids is None:
        seq_start = (torch.arange(B, device=q.device, dtype=torch.int32) * T).repeat_interleave(T)
    else:
        # flat index of the first token of each token's document: a new document starts where the id changes or a row begins
        flat = doc_ids.reshape(-1)
        idx = torch.arange(B * T, device=q.device)
        new = torch.ones(B * T, dtype=torch.bool, device=q.device)
        new[1:] = (flat[1:] != flat[:-1]) | (idx[1:] % T == 0)
        seq_start = torch.cummax(torch.where(new, idx, torch.zeros_like(idx)), 0).values.to(torch.int32)
    o = ops._AttnCoreFn.apply(qf, kf, vf, seq_start, scale, int(window))
    return o[..., :d].reshape(B, T, h, d).transpose(1, 2)
