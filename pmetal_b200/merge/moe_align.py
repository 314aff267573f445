"""Expert alignment for merging mixture-of-experts checkpoints.

Tensor-by-name merging pairs expert *i* of one checkpoint with expert *i* of the other. Two fine-tunes that specialised
their experts in different orders make that pairing meaningless. Per MoE layer and per non-reference model this module
fingerprints every expert (flattened, L2-normalised gate projection), builds the cosine-similarity matrix against the
reference model's experts and solves the maximum-weight assignment (Hungarian algorithm, O(N^3), N <= a few hundred);
the resulting permutation is applied to the expert tensors *and* to the router rows, so each model computes exactly the
same function as before while its experts line up with the reference
(crates/pmetal-merge/src/moe_align.rs:1-330 renames ``experts.{i}`` -> ``experts.{pi(i)}`` in the tensor loader).

Both expert layouts are handled: one tensor per expert (``...experts.{i}.gate_proj.weight``) and stacked banks
(``...experts.gate_up_proj`` of shape [E, ...])."""
from __future__ import annotations

import re
from typing import Dict, List, Optional, Sequence

import torch

_PER_EXPERT = re.compile(r"^(.*\.layers\.(\d+)\..*?experts)\.(\d+)\.(.+)$")
_STACKED = re.compile(r"^(.*\.layers\.(\d+)\..*?experts)\.(gate_up_proj|gate_proj|up_proj|down_proj|w1|w2|w3)(\.weight)?$")
_ROUTER = re.compile(r"^(.*\.layers\.(\d+)\.(?:mlp|block_sparse_moe|feed_forward))\.(gate|router|gate\.wg|router\.proj|router\.layer)"
                     r"\.(weight|bias|e_score_correction_bias)$")
_FINGERPRINT_PARTS = ("gate_proj.weight", "w1.weight", "gate_up_proj", "up_proj.weight", "w3.weight")


def hungarian_max(weights: torch.Tensor) -> List[int]:
    """Assignment ``row -> column`` maximising the total weight of a square matrix (Kuhn-Munkres with potentials)."""
    n = weights.shape[0]
    cost = (-weights.double()).tolist()
    INF = float("inf")
    u, v, p, way = [0.0] * (n + 1), [0.0] * (n + 1), [0] * (n + 1), [0] * (n + 1)
    for i in range(1, n + 1):
        p[0] = i
        j0 = 0
        minv = [INF] * (n + 1)
        used = [False] * (n + 1)
        while True:
            used[j0] = True
            i0, delta, j1 = p[j0], INF, 0
            for j in range(1, n + 1):
                if not used[j]:
                    cur = cost[i0 - 1][j - 1] - u[i0] - v[j]
                    if cur < minv[j]:
                        minv[j], way[j] = cur, j0
                    if minv[j] < delta:
                        delta, j1 = minv[j], j
            for j in range(n + 1):
                if used[j]:
                    u[p[j]] += delta
                    v[j] -= delta
                else:
                    minv[j] -= delta
            j0 = j1
            if p[j0] == 0:
                break
        while True:
            j1 = way[j0]
            p[j0] = p[j1]
            j0 = j1
            if j0 == 0:
                break
    out = [0] * n
    for j in range(1, n + 1):
        out[p[j] - 1] = j - 1
    return out


def expert_layers(names: Sequence[str]) -> Dict[int, dict]:
    """layer -> {"prefix", "layout": "per_expert" | "stacked", "experts": E or None} for every MoE layer in ``names``."""
    out: Dict[int, dict] = {}
    for n in names:
        m = _PER_EXPERT.match(n)
        if m:
            d = out.setdefault(int(m.group(2)), {"prefix": m.group(1), "layout": "per_expert", "experts": 0})
            d["experts"] = max(d["experts"], int(m.group(3)) + 1)
            continue
        m = _STACKED.match(n)
        if m:
            out.setdefault(int(m.group(2)), {"prefix": m.group(1), "layout": "stacked", "experts": None})
    return out


def _fingerprints(ck, info: dict) -> Optional[torch.Tensor]:
    """[E, D] L2-normalised fingerprints of one layer's experts, or None when no known projection is present."""
    pre = info["prefix"]
    if info["layout"] == "stacked":
        for part in _FINGERPRINT_PARTS:
            for name in (f"{pre}.{part}", f"{pre}.{part}.weight"):
                if name in ck.index:
                    t = ck.get(name).float()
                    return torch.nn.functional.normalize(t.reshape(t.shape[0], -1), dim=-1)
        return None
    rows = []
    for e in range(info["experts"]):
        name = next((f"{pre}.{e}.{part}" for part in _FINGERPRINT_PARTS if f"{pre}.{e}.{part}" in ck.index), None)
        if name is None:
            return None
        rows.append(ck.get(name).float().reshape(-1))
    return torch.nn.functional.normalize(torch.stack(rows), dim=-1)


class MoeAlignment:
    """``perm[model][layer][i]`` = index of the expert of ``model`` that plays the role of the reference's expert ``i``."""

    def __init__(self, perms: List[Dict[int, List[int]]], layers: Dict[int, dict]):
        self.perms, self.layers = perms, layers

    def is_identity(self) -> bool:
        return all(p == list(range(len(p))) for m in self.perms for p in m.values())

    def fetch(self, ck, model_idx: int, name: str) -> torch.Tensor:
        """Tensor ``name`` of model ``model_idx`` as the reference indexes it (experts and router rows permuted)."""
        perms = self.perms[model_idx]
        m = _PER_EXPERT.match(name)
        if m and int(m.group(2)) in perms:
            src = perms[int(m.group(2))][int(m.group(3))]
            return ck.get(f"{m.group(1)}.{src}.{m.group(4)}")
        m = _STACKED.match(name) or _ROUTER.match(name)
        if m and int(m.group(2)) in perms:
            t = ck.get(name)
            p = perms[int(m.group(2))]
            if t.dim() >= 1 and t.shape[0] == len(p):
                return t.index_select(0, torch.tensor(p))
        return ck.get(name)


def align_experts(checkpoints: Sequence, reference: int = 0) -> Optional[MoeAlignment]:
    """Permutations of every model against ``checkpoints[reference]``; None when the models have no routed experts."""
    layers = expert_layers(checkpoints[reference].keys())
    if not layers:
        return None
    ref_fp = {l: _fingerprints(checkpoints[reference], info) for l, info in layers.items()}
    perms: List[Dict[int, List[int]]] = []
    for mi, ck in enumerate(checkpoints):
        per_layer: Dict[int, List[int]] = {}
        for l, info in layers.items():
            a = ref_fp[l]
            if a is None:
                continue
            if mi == reference:
                per_layer[l] = list(range(a.shape[0]))
                continue
            b = _fingerprints(ck, info)
            if b is None or b.shape != a.shape:
                raise ValueError(f"layer {l}: the models' expert banks differ in size or layout")
            per_layer[l] = hungarian_max(a @ b.t())
        perms.append(per_layer)
    return MoeAlignment(perms, layers)
