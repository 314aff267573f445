"""Mixture-of-experts feed-forward block (Qwen3-MoE).

Routing follows crates/pmetal-models/src/moe_routing.rs:36-108 and
architectures/qwen3_moe.rs:519-540: softmax over all experts in fp32, top-k, and
optional renormalisation of the k weights (``norm_topk_prob``, eps 1e-8). Experts are
stored stacked, ``gate_up`` [E, 2I, H] and ``down`` [E, H, I]; tokens are sorted by
expert and each expert's contiguous slab goes through a grouped GEMM.
"""
from __future__ import annotations

from typing import Dict, Optional, Set, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .config import ModelArgs


def route_topk(router_logits: torch.Tensor, k: int, norm_topk_prob: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    probs = torch.softmax(router_logits.float(), dim=-1)
    w, idx = torch.topk(probs, k, dim=-1)
    if norm_topk_prob:
        w = w / (w.sum(-1, keepdim=True) + 1e-8)
    return w, idx


def sort_by_expert(idx: torch.Tensor, num_experts: int):
    """Flatten [T,k] assignments; returns (order, counts, offsets) with tokens grouped by expert."""
    flat = idx.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts)
    offsets = torch.zeros(num_experts + 1, dtype=torch.int64, device=idx.device)
    offsets[1:] = torch.cumsum(counts, 0)
    return order, counts, offsets


class SparseMoeBlock(nn.Module):
    def __init__(self, cfg: ModelArgs, dtype, device):
        super().__init__()
        self.cfg = cfg
        E, H, I = cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size
        self.router = nn.Parameter(torch.empty(E, H, dtype=dtype, device=device))
        self.gate_up = nn.Parameter(torch.empty(E, 2 * I, H, dtype=dtype, device=device))
        self.down = nn.Parameter(torch.empty(E, H, I, dtype=dtype, device=device))
        self.ep_group = None       # set by parallel.ep.shard_experts
        self.local_experts: Optional[Tuple[int, int]] = None

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        cfg = self.cfg
        if getattr(self, "tp_reduce", None) is not None and self.local_experts is not None:
            from ..parallel.tp_model import moe_local_forward
            return moe_local_forward(self, x, residual)      # replicated tokens, this rank's experts, summed over ranks
        logits = F.linear(x, self.router)
        eng = getattr(self, "ep_engine", None)
        if eng is not None and x.is_cuda and not torch.is_grad_enabled() and x.shape[0] * eng.k <= eng.max_rows:
            # fused routing + (expert-parallel) dispatch + grouped GEMMs + combine (parallel/ep.py)
            if residual is not None and x.dtype == torch.bfloat16:
                return eng.forward(x, logits, residual)          # residual add fused into the combine kernel
            out = eng.forward(x.to(torch.bfloat16), logits).to(x.dtype)
            return out if residual is None else out + residual
        w, idx = route_topk(logits, cfg.num_experts_per_tok, cfg.norm_topk_prob)
        if getattr(self, "offload", None) is not None:
            from .expert_store import offloaded_experts_forward
            out = offloaded_experts_forward(self, x, w, idx)     # experts read from a packed directory on demand
        elif self.ep_group is not None and getattr(self, "ep_train", False):
            from ..parallel.ep_train import ep_moe_train_forward
            out = ep_moe_train_forward(self, x, w, idx)          # sharded expert parameters, differentiable exchange
        elif self.ep_group is not None:
            from ..parallel.ep import ep_moe_forward_nccl
            out = ep_moe_forward_nccl(self, x, w, idx)
        else:
            out = self.experts_forward(x, w, idx)
        return out if residual is None else out + residual

    def experts_forward(self, x: torch.Tensor, w: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        from ..ops import functional as ops
        return ops.moe_experts(x, w, idx, self.gate_up, self.down)

    def hf_state_dict(self) -> Dict[str, torch.Tensor]:
        if getattr(self, "offload", None) is not None:
            raise RuntimeError("the experts of this block live in a packed directory and cannot be exported from here")
        I = self.cfg.moe_intermediate_size
        sd = {"gate.weight": self.router.detach()}
        for e in range(self.cfg.num_experts):
            sd[f"experts.{e}.gate_proj.weight"] = self.gate_up.detach()[e, :I]
            sd[f"experts.{e}.up_proj.weight"] = self.gate_up.detach()[e, I:]
            sd[f"experts.{e}.down_proj.weight"] = self.down.detach()[e]
        return sd

    @torch.no_grad()
    def load_hf_state_dict(self, sd, prefix: str, strict: bool = True) -> Set[str]:
        used = set()
        I = self.cfg.moe_intermediate_size

        def take(name, dst):
            if name in sd:
                dst.copy_(sd[name].to(dst.dtype))
                used.add(name)
            elif strict:
                raise KeyError(name)
        take(prefix + "gate.weight", self.router)
        if prefix + "switch_mlp.gate_proj.weight" in sd:       # stacked layout used by the reference loader
            self.gate_up[:, :I].copy_(sd[prefix + "switch_mlp.gate_proj.weight"])
            self.gate_up[:, I:].copy_(sd[prefix + "switch_mlp.up_proj.weight"])
            self.down.copy_(sd[prefix + "switch_mlp.down_proj.weight"])
            used |= {prefix + f"switch_mlp.{n}_proj.weight" for n in ("gate", "up", "down")}
            return used
        for e in range(self.cfg.num_experts):
            take(prefix + f"experts.{e}.gate_proj.weight", self.gate_up[e, :I])
            take(prefix + f"experts.{e}.up_proj.weight", self.gate_up[e, I:])
            take(prefix + f"experts.{e}.down_proj.weight", self.down[e])
        return used
