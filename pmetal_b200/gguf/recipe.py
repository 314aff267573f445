"""Per-tensor GGUF type selection.

``tensor_type`` is the llama.cpp-style recipe of the reference (crates/pmetal/src/commands/quantize.rs:955-1137):
norms / routers / positional tables stay dense, ``output`` and ``token_embd`` get Q6_K under the K methods, and
attn_v / ffn_down / attn_output / attn_qkv are bumped by method and layer position. ``DynamicQuantizer`` is the
``dynamic`` method (crates/pmetal-gguf/src/dynamic.rs:31-59,240-372,420-560): critical tensors to the fallback type,
importance-ranked tensors to the high type, optional error-calibrated search and a bits-per-weight target."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .types import BLOCK_GEOMETRY, QUANT_METHODS, GgmlType, bits_per_weight

_DENSE_MARKERS = ("_norm.weight", "norm.weight", "ffn_gate_inp.weight", "router", "altup", "laurel",
                  "per_layer_model_proj", "pos_embd", "token_types", "ssm_conv1d", "shortconv.conv.weight",
                  "attn_rel_b.weight", ".position_embd", ".rel_pos", ".patch_embd", ".patch_merger")
_K_METHODS = {"dynamic", "q2_k", "q3_k_m", "q3_k_s", "q3_k_l", "q4_k_m", "q4_k_s", "q5_k_m", "q5_k_s", "q6_k"}
_NO_EMBED_QUANT = {"q1_0", "tq1_0", "tq2_0", "mxfp4", "nvfp4"}


def is_quantizable(name: str, shape: Sequence[int]) -> bool:
    if len(shape) not in (2, 3) or not name.endswith(".weight"):
        return False
    low = name.lower()
    return not any(m in low for m in _DENSE_MARKERS)


def layer_of(name: str) -> Optional[int]:
    if not name.startswith("blk."):
        return None
    part = name[4:].split(".", 1)[0]
    return int(part) if part.isdigit() else None


def use_more_bits(layer: int, n_layers: int) -> bool:
    if n_layers == 0:
        return False
    return layer < n_layers // 8 or layer >= 7 * n_layers // 8 or max(layer - n_layers // 8, 0) % 3 == 2


def tensor_type(method: str, name: str, shape: Sequence[int], config: Optional[dict] = None,
                proposed: Optional[GgmlType] = None) -> GgmlType:
    method = method.lower()
    base = QUANT_METHODS[method][0]
    if method in ("f32", "f16", "bf16"):
        return base
    if not is_quantizable(name, shape):
        return GgmlType.F16
    T = GgmlType
    dtype = proposed if (method == "dynamic" and proposed is not None) else base
    cfg = config or {}
    n_layers = int(cfg.get("num_hidden_layers", 0) or 0)
    n_heads = int(cfg.get("num_attention_heads", 0) or 0)
    n_kv = int(cfg.get("num_key_value_heads", max(n_heads, 1)) or max(n_heads, 1))
    n_gqa = n_heads // n_kv if n_kv else 1
    layer = layer_of(name) or 0
    if name in ("output.weight", "token_embd.weight"):
        if method in _NO_EMBED_QUANT:
            return T.F16
        if dtype == T.Q8_0:
            return T.Q8_0
        return T.Q6K if method in _K_METHODS else dtype
    more = use_more_bits(layer, n_layers)
    if "attn_v.weight" in name:
        dtype = {"q2_k": T.Q4K if n_gqa >= 4 else T.Q3K, "q3_k_m": T.Q5K if layer < 2 else T.Q4K, "q3_k_l": T.Q5K,
                 "q4_k_m": T.Q6K if more else dtype, "q5_k_m": T.Q6K if more else dtype,
                 "q4_k_s": T.Q5K if layer < 4 else dtype}.get(method, dtype)
    elif "ffn_down.weight" in name or "ffn_down_exps.weight" in name:
        dtype = {"q2_k": T.Q3K,
                 "q3_k_m": T.Q5K if layer < n_layers // 16 else (T.Q4K if more else T.Q3K), "q3_k_l": T.Q5K,
                 "q4_k_m": T.Q6K if more else dtype, "q5_k_m": T.Q6K if more else dtype,
                 "q4_k_s": T.Q5K if layer < n_layers // 8 else dtype}.get(method, dtype)
    elif "attn_output.weight" in name:
        dtype = {"q2_k": T.Q3K, "q3_k_m": T.Q4K, "q3_k_l": T.Q5K}.get(method, dtype)
    elif "attn_qkv.weight" in name:
        dtype = {"q3_k_m": T.Q4K, "q3_k_l": T.Q4K, "q4_k_m": T.Q5K, "q5_k_m": T.Q6K}.get(method, dtype)
    return dtype


def fit_to_shape(dtype: GgmlType, shape: Sequence[int]) -> GgmlType:
    """Rows must hold whole blocks; otherwise step down to a 32-element format, then to F16."""
    row = int(shape[-1])
    if row % BLOCK_GEOMETRY[dtype][0] == 0:
        return dtype
    if row % 32 == 0 and BLOCK_GEOMETRY[dtype][0] == 256:
        return GgmlType.Q8_0 if bits_per_weight(dtype) > 5 else (GgmlType.Q5_0 if bits_per_weight(dtype) > 4.6 else GgmlType.Q4_0)
    return GgmlType.F16


_CRITICAL = ("lm_head", "output", "token_embd", "embed_tokens", "wte", "final_norm", "ln_f")


@dataclass
class DynamicConfig:
    base_type: GgmlType = GgmlType.Q4K
    high_type: GgmlType = GgmlType.Q6K
    fallback_type: GgmlType = GgmlType.Q6K
    importance_percentile: float = 0.20
    protect_attention: bool = False
    protect_first_layers: int = 0
    kl_calibrate: bool = False
    error_budget: float = 0.01
    target_bpw: Optional[float] = None
    candidates: Tuple[GgmlType, ...] = (GgmlType.Q8K, GgmlType.Q6K, GgmlType.Q5K, GgmlType.Q4K, GgmlType.Q3K, GgmlType.Q2K)


@dataclass
class DynamicQuantizer:
    config: DynamicConfig = field(default_factory=DynamicConfig)
    imatrix: Optional["IMatrix"] = None      # noqa: F821
    _cutoff: Optional[float] = None

    def _is_critical(self, name: str) -> bool:
        low = name.lower()
        return any(c in low for c in _CRITICAL)

    def _importance_cutoff(self) -> float:
        if self._cutoff is None:
            vals = sorted((self.imatrix.importance(n) for n in self.imatrix.data), reverse=True)
            k = max(int(len(vals) * self.config.importance_percentile), 1)
            self._cutoff = vals[min(k, len(vals)) - 1] if vals else float("inf")
        return self._cutoff

    def propose(self, name: str, imatrix_key: Optional[str] = None) -> GgmlType:
        c = self.config
        if self._is_critical(name):
            return c.fallback_type
        if c.protect_attention and "attn" in name:
            return c.high_type
        layer = layer_of(name)
        if layer is not None and layer < c.protect_first_layers:
            return c.high_type
        if self.imatrix is not None and self.imatrix.data:
            key = imatrix_key or name
            if key in self.imatrix.data and self.imatrix.importance(key) >= self._importance_cutoff():
                return c.high_type
        return c.base_type

    @staticmethod
    def score(x: np.ndarray, y: np.ndarray) -> float:
        """NRMSE + cosine distance between a tensor and its quantise/dequantise round trip."""
        x = x.reshape(-1).astype(np.float64)
        y = y.reshape(-1).astype(np.float64)
        nx = np.linalg.norm(x)
        if nx == 0:
            return 0.0
        nrmse = np.linalg.norm(x - y) / nx
        ny = np.linalg.norm(y)
        cos = 1.0 - float(x @ y) / (nx * ny) if ny > 0 else 1.0
        return float(nrmse + cos)

    def calibrate(self, name: str, x: np.ndarray) -> GgmlType:
        """Cheapest candidate whose round-trip score stays within the error budget (most bits first)."""
        from . import native
        if self._is_critical(name):
            return self.config.fallback_type
        best = self.config.candidates[0]
        sample = x.reshape(-1)
        sample = sample[: (min(sample.size, 1 << 20) // 256) * 256]
        if sample.size == 0:
            return self.config.base_type
        for t in self.config.candidates:
            y = native.dequantize(native.quantize(sample, t), t, sample.size)
            if self.score(sample, y) <= self.config.error_budget:
                best = t
            else:
                break
        return best

    def fit_target_bpw(self, plan: Dict[str, Tuple[GgmlType, int, float]]) -> Dict[str, GgmlType]:
        """Greedy downgrade to reach ``target_bpw``. ``plan``: name -> (type, n_elements, importance)."""
        out = {n: t for n, (t, _, _) in plan.items()}
        if self.config.target_bpw is None:
            return out
        order: List[GgmlType] = [GgmlType.Q8K, GgmlType.Q6K, GgmlType.Q5K, GgmlType.Q4K, GgmlType.Q3K, GgmlType.Q2K]
        total = sum(n for _, n, _ in plan.values())

        def bpw():
            return sum(bits_per_weight(out[n]) * plan[n][1] for n in plan) / max(total, 1)
        names = sorted((n for n in plan if not self._is_critical(n) and out[n] in order), key=lambda n: plan[n][2])
        progressed = True
        while bpw() > self.config.target_bpw and progressed:
            progressed = False
            for n in names:
                i = order.index(out[n])
                if i + 1 < len(order):
                    out[n] = order[i + 1]
                    progressed = True
                    if bpw() <= self.config.target_bpw:
                        break
        return out
