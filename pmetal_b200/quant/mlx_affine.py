"""Affine group quantisation in the MLX checkpoint layout, with per-tensor bit allocation driven by reconstruction
quality (crates/pmetal-bridge/src/mlx_quant.rs:56-700; quantised matmul: crates/pmetal-mlx/src/kernels/quantized_matmul.rs).

Format: along the last axis every ``group_size`` weights share ``scale`` and ``bias`` (fp16): w ~ scale * q + bias with
q in [0, 2^bits - 1]. The edge (the end of the group's range with the larger magnitude) is represented exactly:
scale = +-(max - min) / (2^bits - 1) with the sign chosen so that the edge is q = 0's neighbour, then scale is
re-derived from round(edge / scale) so that zero stays representable. Codes are packed LSB-first into uint32 words
(``weight``), next to ``scales`` and ``biases`` tensors, and ``config.json`` gains a ``quantization`` section with the
default and the per-tensor overrides.

Pipeline: (1) score every matrix at every candidate bit width by NRMSE + (1 - cosine) of the round trip; (2) pin critical
tensors (norms, embeddings, head, router gates, expert stacks, recurrence parameters) to >= 8 bits, start the rest at
the lowest width and upgrade the worst-scoring tensor first until the bits-per-weight budget is used; (3) quantise and
write the shards."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

CANDIDATE_BITS = (2, 3, 4, 6, 8)


def quantize_affine(w: torch.Tensor, bits: int = 4, group_size: int = 64) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """w [..., K] (K % group_size == 0) -> (packed uint32 [..., K * bits / 32], scales fp16 [..., K / g], biases fp16)."""
    if w.shape[-1] % group_size:
        raise ValueError(f"last dimension {w.shape[-1]} is not a multiple of the group size {group_size}")
    if (w.shape[-1] * bits) % 32:
        raise ValueError("packed row length must be a whole number of 32-bit words")
    n_bins = float((1 << bits) - 1)
    g = w.float().reshape(*w.shape[:-1], -1, group_size)
    w_max, w_min = g.amax(-1, keepdim=True), g.amin(-1, keepdim=True)
    lower_edge = w_min.abs() > w_max.abs()
    scales = torch.where(lower_edge, w_max - w_min, w_min - w_max) / n_bins
    scales = torch.where(scales.abs() < 1e-7, torch.full_like(scales, 1e-7), scales)
    edge = torch.where(lower_edge, w_min, w_max)
    q0 = torch.round(edge / scales)
    scales = torch.where(q0 != 0, edge / torch.where(q0 != 0, q0, torch.ones_like(q0)), scales)
    biases = torch.where(q0 == 0, torch.zeros_like(edge), edge)
    scales, biases = scales.half(), biases.half()                       # what is stored is what is used
    q = torch.clamp(torch.round((g - biases.float()) / scales.float()), 0, n_bins).to(torch.int64)
    q = q.reshape(*w.shape[:-1], -1)
    return pack_bits(q, bits), scales.squeeze(-1), biases.squeeze(-1)


def pack_bits(q: torch.Tensor, bits: int) -> torch.Tensor:
    """LSB-first bit stream of ``bits``-wide codes along the last axis, as uint32 words (stored in an int32 tensor)."""
    K = q.shape[-1]
    pos = torch.arange(K, device=q.device) * bits
    words = (K * bits) // 32
    out = torch.zeros(*q.shape[:-1], words, dtype=torch.int64, device=q.device)
    lo_word, lo_shift = pos // 32, pos % 32
    out.scatter_add_(-1, lo_word.expand_as(q), (q << lo_shift) & 0xFFFFFFFF)
    spill = lo_shift + bits > 32                                       # codes that straddle a word boundary (3 / 6 bit)
    if bool(spill.any()):
        idx = spill.nonzero().squeeze(-1)
        hi = q[..., idx] >> (32 - lo_shift[idx])
        out.scatter_add_(-1, (lo_word[idx] + 1).expand_as(hi), hi)
    out = out & 0xFFFFFFFF
    return torch.where(out >= (1 << 31), out - (1 << 32), out).to(torch.int32)


def unpack_bits(packed: torch.Tensor, bits: int, K: int) -> torch.Tensor:
    w = packed.to(torch.int64) & 0xFFFFFFFF
    pos = torch.arange(K, device=packed.device) * bits
    lo_word, lo_shift = pos // 32, pos % 32
    lo = w[..., lo_word] >> lo_shift
    hi_word = torch.clamp(lo_word + 1, max=w.shape[-1] - 1)
    hi = torch.where(lo_shift + bits > 32, w[..., hi_word] << (32 - lo_shift), torch.zeros_like(lo))
    return (lo | hi) & ((1 << bits) - 1)


def dequantize_affine(packed: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, bits: int, group_size: int,
                      dtype=torch.float32) -> torch.Tensor:
    K = scales.shape[-1] * group_size
    q = unpack_bits(packed, bits, K).float().reshape(*scales.shape, group_size)
    return (q * scales.float()[..., None] + biases.float()[..., None]).reshape(*scales.shape[:-1], K).to(dtype)


def quantized_matmul(x: torch.Tensor, packed, scales, biases, bits: int, group_size: int) -> torch.Tensor:
    """x [..., K] @ dequant(W [N, K])^T: the weight is expanded in tiles of rows so that the full matrix never exists."""
    N = scales.shape[0]
    outs = []
    for a in range(0, N, 4096):
        w = dequantize_affine(packed[a:a + 4096], scales[a:a + 4096], biases[a:a + 4096], bits, group_size, x.dtype)
        outs.append(x @ w.t())
    return torch.cat(outs, -1)


def gather_qmm(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, indices: torch.Tensor,
               bits: int, group_size: int) -> torch.Tensor:
    """Quantised gather-matmul for mixture-of-experts layers: row ``i`` of ``x`` [R, K] is multiplied by the quantised
    matrix of expert ``indices[i]`` out of a stack ``packed`` [E, N, K * bits / 32] (``scales`` / ``biases`` [E, N, K /
    group]); returns [R, N]. Rows are grouped by expert so that each expert's matrix is expanded once and only while it
    is used (bridge_inference.cpp ``gather_qmm``, crates/pmetal-bridge/cpp/bridge_inference.cpp)."""
    R = x.shape[0]
    N = scales.shape[1]
    out = x.new_empty(R, N)
    order = torch.argsort(indices, stable=True)
    counts = torch.bincount(indices, minlength=packed.shape[0]).tolist()
    pos = 0
    for e, n in enumerate(counts):
        if n == 0:
            continue
        rows = order[pos:pos + n]
        out[rows] = quantized_matmul(x[rows], packed[e], scales[e], biases[e], bits, group_size)
        pos += n
    return out


# ------------------------------------------------------------------------------------------------ allocation
def is_critical_tensor(name: str) -> bool:
    n = name.lower()
    if n in ("model.norm.weight", "model.embed_tokens.weight", "lm_head.weight"):
        return True
    if "layernorm" in n or "ln_" in n or ".norm." in n or n.endswith((".norm", "norm.weight", "norm.bias")):
        return True
    if n.endswith(".gate.weight") or ".experts." in n:
        return True
    return "a_log" in n or "dt_bias" in n or "conv1d" in n


def reconstruction_score(w: torch.Tensor, bits: int, group_size: int) -> float:
    p, s, b = quantize_affine(w, bits, group_size)
    r = dequantize_affine(p, s, b, bits, group_size)
    wf = w.float()
    nrmse = float((r - wf).norm() / wf.norm().clamp(min=1e-12))
    cos = float(torch.nn.functional.cosine_similarity(r.flatten(), wf.flatten(), dim=0))
    return nrmse + (1.0 - cos)


def quantizable(name: str, w: torch.Tensor, group_size: int) -> bool:
    return w.dim() == 2 and w.shape[-1] % group_size == 0 and w.shape[-1] >= group_size and name.endswith(".weight")


def evaluate_tensor_quality(tensors: Dict[str, torch.Tensor], group_size: int = 64,
                            candidates: Sequence[int] = CANDIDATE_BITS) -> List[Tuple[str, int, List[Tuple[int, float]]]]:
    """[(name, parameter count, [(bits, score)] ascending in bits)]; non-matrices get an empty list (kept as they are)."""
    out = []
    for name, w in tensors.items():
        scores = []
        if quantizable(name, w, group_size):
            scores = [(b, reconstruction_score(w, b, group_size)) for b in candidates if (w.shape[-1] * b) % 32 == 0]
        out.append((name, w.numel(), scores))
    return out


@dataclass
class TensorQuant:
    name: str
    bits: int
    group_size: int
    param_count: int
    quality_score: float


def _bits_per_weight(bits: int, group_size: int) -> float:
    return bits + 32.0 / group_size                      # codes + fp16 scale and bias per group


def allocate_bits_for_bpw(tensor_scores, target_bpw: float, group_size: int = 64,
                          critical_patterns: Sequence[str] = ()) -> List[TensorQuant]:
    step = [0] * len(tensor_scores)
    forced = [False] * len(tensor_scores)
    for i, (name, _, scores) in enumerate(tensor_scores):
        if not scores:
            continue
        if is_critical_tensor(name) or any(p in name for p in critical_patterns):
            forced[i] = True
            step[i] = next((k for k, (b, _) in enumerate(scores) if b >= 8), len(scores) - 1)

    def bpw() -> float:
        bits = params = 0.0
        for i, (_, n, scores) in enumerate(tensor_scores):
            params += n
            bits += n * (_bits_per_weight(scores[step[i]][0], group_size) if scores else 16.0)
        return bits / max(params, 1.0)
    while bpw() < target_bpw:
        cands = [i for i, (_, _, sc) in enumerate(tensor_scores) if sc and not forced[i] and step[i] + 1 < len(sc)]
        if not cands:
            break
        worst = max(cands, key=lambda i: tensor_scores[i][2][step[i]][1])
        step[worst] += 1
        if bpw() > target_bpw + 1e-9 and len(cands) > 1:           # the upgrade overshot: undo it and stop
            step[worst] -= 1
            break
    return [TensorQuant(name, sc[step[i]][0], group_size, n, sc[step[i]][1])
            for i, (name, n, sc) in enumerate(tensor_scores) if sc]


# ------------------------------------------------------------------------------------------------ model level
def quantize_state_dict(tensors: Dict[str, torch.Tensor], plan: Sequence[TensorQuant]) -> Dict[str, torch.Tensor]:
    """``name.weight`` -> packed ``name.weight`` (uint32 as int32) + ``name.scales`` + ``name.biases``; the rest unchanged."""
    by_name = {t.name: t for t in plan}
    out: Dict[str, torch.Tensor] = {}
    for name, w in tensors.items():
        t = by_name.get(name)
        if t is None:
            out[name] = w
            continue
        p, s, b = quantize_affine(w, t.bits, t.group_size)
        stem = name[: -len(".weight")]
        out[name], out[stem + ".scales"], out[stem + ".biases"] = p, s, b
    return out


def quantization_config(plan: Sequence[TensorQuant], default_bits: int, group_size: int) -> dict:
    cfg = {"group_size": group_size, "bits": default_bits}
    for t in plan:
        if t.bits != default_bits:
            cfg[t.name[: -len(".weight")]] = {"group_size": t.group_size, "bits": t.bits}
    return cfg


def quantize_model(model_dir: str, out_dir: str, target_bpw: float = 4.5, group_size: int = 64,
                   candidates: Sequence[int] = CANDIDATE_BITS) -> dict:
    """Quantise a Hugging Face checkpoint directory into ``out_dir`` (model.safetensors + config.json). Returns a report."""
    from ..models.loader import read_state_dict
    from ..utils.safetensors_io import save_file
    sd = read_state_dict(model_dir)
    scores = evaluate_tensor_quality(sd, group_size, candidates)
    plan = allocate_bits_for_bpw(scores, target_bpw, group_size)
    os.makedirs(out_dir, exist_ok=True)
    save_file({k: v.contiguous() for k, v in quantize_state_dict(sd, plan).items()}, os.path.join(out_dir, "model.safetensors"),
              metadata={"format": "mlx"})
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as fh:
        cfg = json.load(fh)
    counts: Dict[int, int] = {}
    for t in plan:
        counts[t.bits] = counts.get(t.bits, 0) + 1
    default_bits = max(counts, key=counts.get) if counts else 4
    cfg["quantization"] = cfg["quantization_config"] = quantization_config(plan, default_bits, group_size)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(cfg, fh, indent=2)
    total = sum(v.numel() for v in sd.values())
    qbits = sum(t.param_count * _bits_per_weight(t.bits, group_size) for t in plan)
    rest = (total - sum(t.param_count for t in plan)) * 16.0
    return {"tensors": len(plan), "bits_histogram": counts, "effective_bpw": round((qbits + rest) / max(total, 1), 3),
            "output": out_dir}


def load_quantized_state_dict(sd: Dict[str, torch.Tensor], quantization: dict, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Expand an MLX-quantised state dict back to dense tensors (``.scales`` / ``.biases`` entries are consumed)."""
    out = {}
    for name, v in sd.items():
        if name.endswith((".scales", ".biases")):
            continue
        stem = name[: -len(".weight")] if name.endswith(".weight") else None
        if stem is not None and stem + ".scales" in sd:
            q = quantization.get(stem) or quantization
            out[name] = dequantize_affine(v, sd[stem + ".scales"], sd[stem + ".biases"], int(q["bits"]), int(q["group_size"]), dtype)
        else:
            out[name] = v
    return out
