"""Parallelism plans: tensor-parallel sharding directives, expert placement and capacity, ZeRO ownership,
pipeline schedules, pipeline layer assignment. Pure host-side planning (no device work).

Restated from the reference's planning code:
* TP (tensor_parallel/{sharding,plan}.rs): Megatron column/row split — q/k/v/gate/up are ``all_to_sharded``
  on the output axis, o/down are ``sharded_to_all`` on the input axis, norms/embeddings replicated, MoE
  experts ``expert_sharded``; uneven splits give the remainder to the first ranks.
* EP (expert_shard.rs:54-110, expert_parallel/{placement,capacity}.rs): contiguous expert ranges with the
  remainder on the first ranks; capacity = ceil(tokens * k / experts * factor) with factor 1.25; Switch
  load-balancing auxiliary loss E * sum_e f_e * P_e.
* ZeRO-1/2 (zero/state_partition.rs:7-130): parameters sorted by name, owner = index mod world.
* PP (pipeline_training/schedule_1f1b.rs:19-140, schedule_zbv.rs:24-200): 1F1B action lists with bubble
  (P-1)/(M+P-1); zero-bubble variant splits backward into input-gradient (B) and weight-gradient (W) and
  fills the cooldown with deferred W.
* layer assignment (layer_assignment.rs:17-140, solver.rs:14-170): contiguous layer ranges proportional to
  device memory, or the bandwidth-aware exhaustive split that minimises the slowest stage.
"""
from __future__ import annotations

import itertools
import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple


# --------------------------------------------------------------------------- tensor parallel
@dataclass(frozen=True)
class ShardingDirective:
    kind: str          # all_to_sharded | sharded_to_all | replicated | expert_sharded
    axis: int = 0
    total: int = 0


def shard_bounds(size: int, rank: int, world: int) -> Tuple[int, int]:
    base, rem = divmod(size, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def shard_weight(w, directive: ShardingDirective, rank: int, world: int):
    if directive.kind == "replicated":
        return w
    if directive.kind == "expert_sharded":
        lo, n = expert_range(directive.total or w.shape[0], rank, world)
        return w[lo:lo + n]
    lo, hi = shard_bounds(w.shape[directive.axis], rank, world)
    return w.narrow(directive.axis, lo, hi - lo)


_COL = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj", "qkv_proj", "gate_up_proj", "in_proj", "w1", "w3")
_ROW = ("o_proj", "down_proj", "out_proj", "w2")


def build_tp_plan(arch: str, config: dict, world: int) -> Dict[str, ShardingDirective]:
    """Name-pattern -> directive for a decoder of family ``arch`` (llama, mistral, qwen2, qwen3, qwen3_moe, ...)."""
    heads = config.get("num_attention_heads", 0)
    kv = config.get("num_key_value_heads", heads)
    if heads and heads % world:
        raise ValueError(f"{heads} attention heads do not divide over {world} ranks")
    plan: Dict[str, ShardingDirective] = {}
    for n in _COL:
        plan[n] = ShardingDirective("all_to_sharded", 0)
    for n in _ROW:
        plan[n] = ShardingDirective("sharded_to_all", 1)
    if kv and kv % world:
        # fewer kv heads than ranks: k/v are replicated (each rank keeps the heads its q heads need)
        plan["k_proj"] = plan["v_proj"] = ShardingDirective("replicated")
    for n in ("embed_tokens", "norm", "layernorm", "q_norm", "k_norm", "router", "gate.weight"):
        plan[n] = ShardingDirective("replicated")
    plan["lm_head"] = ShardingDirective("all_to_sharded", 0)
    if arch in ("qwen3_moe", "deepseek", "llama4", "gpt_oss") or config.get("num_experts"):
        plan["experts"] = ShardingDirective("expert_sharded", 0, config.get("num_experts", 0))
    return plan


# --------------------------------------------------------------------------- per-architecture tensor plans
# Block planners: suffix -> directive tables for one block of a layer; ``build_plan`` walks the layers of a checkpoint
# and applies the table that fits each block (crates/pmetal-distributed/src/tensor_parallel/plan.rs:50-748). Weights
# are named as in Hugging Face checkpoints; "col" splits output rows (axis 0) and expects a replicated input, "row"
# splits input columns (axis 1) and produces partial sums that are reduced.
_COLW, _ROWW, _REP = ShardingDirective("all_to_sharded", 0), ShardingDirective("sharded_to_all", 1), ShardingDirective("replicated")


def _apply(prefix: str, table: Dict[str, ShardingDirective]) -> Dict[str, ShardingDirective]:
    return {f"{prefix}.{k}": v for k, v in table.items()}


def plan_attention(prefix: str) -> Dict[str, ShardingDirective]:
    """Multi-head / grouped-query attention: q, k, v by head (weights and biases), o by input columns; the o bias is
    added once after the reduction, so it stays whole."""
    t = {f"{p}_proj.{k}": _COLW for p in "qkv" for k in ("weight", "bias")}
    t.update({"o_proj.weight": _ROWW, "o_proj.bias": _REP, "q_norm.weight": _REP, "k_norm.weight": _REP})
    return _apply(prefix, t)


def plan_mla(prefix: str, q_lora_rank: Optional[int]) -> Dict[str, ShardingDirective]:
    """Multi-head latent attention (DeepSeek V2/V3): the down-projections to the latent and their norms are shared by
    all heads and stay whole; the up-projections carry the head dimension and are split by head."""
    t = {"kv_a_proj_with_mqa.weight": _REP, "kv_a_layernorm.weight": _REP, "kv_b_proj.weight": _COLW, "o_proj.weight": _ROWW}
    if q_lora_rank:
        t.update({"q_a_proj.weight": _REP, "q_a_layernorm.weight": _REP, "q_b_proj.weight": _COLW})
    else:
        t["q_proj.weight"] = _COLW
    return _apply(prefix, t)


def plan_ffn(prefix: str) -> Dict[str, ShardingDirective]:
    return _apply(prefix, {"gate_proj.weight": _COLW, "up_proj.weight": _COLW, "down_proj.weight": _ROWW})


def plan_gdn(prefix: str) -> Dict[str, ShardingDirective]:
    """Gated delta-net mixer (Qwen3-Next): every input projection, the depth-wise convolution and the per-head decay
    parameters are split over heads; the output projection is split by input columns like attention's."""
    t = {f"in_proj_{n}.weight": _COLW for n in ("qkv", "z", "b", "a")}
    t.update({"conv1d.weight": _COLW, "dt_bias": _COLW, "A_log": _COLW, "norm.weight": _REP, "o_proj.weight": _ROWW})
    return _apply(prefix, t)


def _stacked_experts(prefix: str, total: int, projs=("gate_proj", "up_proj", "down_proj"), kinds=("weight",)):
    d = ShardingDirective("expert_sharded", 0, total)
    return {f"{prefix}.{p}.{k}": d for p in projs for k in kinds}


def plan_deepseek_moe(prefix: str, total_experts: int, has_shared: bool) -> Dict[str, ShardingDirective]:
    t = {f"{prefix}.gate.weight": _REP, f"{prefix}.gate.e_score_correction_bias": _REP}
    if has_shared:
        t.update(plan_ffn(f"{prefix}.shared_experts"))
    t.update(_stacked_experts(f"{prefix}.switch_mlp", total_experts))
    return t


def plan_qwen_moe(prefix: str, total_experts: int) -> Dict[str, ShardingDirective]:
    t = {f"{prefix}.gate.weight": _REP, f"{prefix}.shared_expert_gate.weight": _REP}
    t.update(plan_ffn(f"{prefix}.shared_expert"))
    t.update(_stacked_experts(f"{prefix}.switch_mlp", total_experts))
    return t


def plan_llama4_moe(prefix: str, total_experts: int) -> Dict[str, ShardingDirective]:
    t = {f"{prefix}.router.weight": _REP}
    t.update(plan_ffn(f"{prefix}.shared_expert"))
    t.update(_stacked_experts(f"{prefix}.experts", total_experts))
    return t


def plan_gpt_oss_moe(prefix: str, total_experts: int) -> Dict[str, ShardingDirective]:
    """GPT-OSS experts carry a bias per expert ([E, out]): axis 0 is the expert axis for weights and biases alike."""
    t = {f"{prefix}.router.weight": _REP, f"{prefix}.router.bias": _REP}
    t.update(_stacked_experts(f"{prefix}.experts", total_experts, kinds=("weight", "bias")))
    return t


def build_plan(arch: str, config: dict, world: int) -> Dict[str, ShardingDirective]:
    """Full tensor name -> directive for a checkpoint of family ``arch`` (a Hugging Face ``architectures`` entry or
    ``model_type``). ``world <= 1`` gives an empty plan. Layer kinds follow the configuration: DeepSeek's dense prefix and
    MoE frequency, Llama-4's interleave step, Qwen's sparse step, Qwen3-Next's ``layer_types`` (or its attention
    interval when the list is missing or has the wrong length)."""
    if world <= 1:
        return {}
    g = config.get
    n_layers = int(g("num_hidden_layers", 32))
    heads = int(g("num_attention_heads", 32))
    if heads % world:
        raise ValueError(f"{heads} attention heads do not divide over {world} ranks")
    experts = int(g("num_experts") or g("num_local_experts") or g("n_routed_experts") or 0)
    mt = str(g("model_type", "") or "")
    low = arch.lower()
    hybrid = g("gdn_heads") is not None or g("mixer_pattern") is not None or "qwen3next" in low.replace("_", "")
    deepseek = "deepseek" in low or mt in ("deepseek_v2", "deepseek_v3")
    llama4 = "llama4" in low or mt == "llama4"
    gpt_oss = "gptoss" in low.replace("_", "") or mt == "gpt_oss"
    qwen_moe = any(k in low.replace("_", "") for k in ("qwen2moe", "qwen3moe")) or hybrid
    layer_types = g("layer_types")
    if not (isinstance(layer_types, list) and len(layer_types) == n_layers):
        layer_types = None
    attn_every = int(g("full_attention_interval") or g("attention_interval") or g("attn_layer_period") or 4)
    plan: Dict[str, ShardingDirective] = {"model.embed_tokens.weight": _REP}
    for i in range(n_layers):
        lp = f"model.layers.{i}"
        # ---- token mixer
        if hybrid:
            full = layer_types[i] == "full_attention" if layer_types else (i + 1) % attn_every == 0
            plan.update(plan_attention(f"{lp}.self_attn") if full else plan_gdn(f"{lp}.linear_attn"))
        elif deepseek:
            plan.update(plan_mla(f"{lp}.self_attn", g("q_lora_rank")))
        else:
            plan.update(plan_attention(f"{lp}.self_attn"))
        # ---- channel mixer
        if deepseek:
            moe = experts > 0 and i >= int(g("first_k_dense_replace", 0) or 0) and i % max(int(g("moe_layer_freq", 1) or 1), 1) == 0
            plan.update(plan_deepseek_moe(f"{lp}.mlp", experts, bool(g("n_shared_experts"))) if moe else plan_ffn(f"{lp}.mlp"))
        elif llama4 and experts > 0:
            moe = i % max(int(g("interleave_moe_layer_step", 1) or 1), 1) == 0
            plan.update(plan_llama4_moe(f"{lp}.feed_forward", experts) if moe else plan_ffn(f"{lp}.mlp"))
        elif gpt_oss and experts > 0:
            plan.update(plan_gpt_oss_moe(f"{lp}.mlp", experts))
        elif qwen_moe and experts > 0:
            moe = (i + 1) % max(int(g("decoder_sparse_step", 1) or 1), 1) == 0
            plan.update(plan_qwen_moe(f"{lp}.mlp", experts) if moe else plan_ffn(f"{lp}.mlp"))
        else:
            plan.update(plan_ffn(f"{lp}.mlp"))
        plan[f"{lp}.input_layernorm.weight"] = _REP
        plan[f"{lp}.post_attention_layernorm.weight"] = _REP
    plan["model.norm.weight"] = _REP
    plan["lm_head.weight"] = _REP
    return plan


def num_sharded(plan: Dict[str, ShardingDirective]) -> int:
    return sum(1 for d in plan.values() if d.kind != "replicated")


def directive_for(plan: Dict[str, ShardingDirective], name: str) -> ShardingDirective:
    if "experts" in plan and "experts" in name:     # expert weights are split by expert, never inside one
        return plan["experts"]
    best = None
    for pat, d in plan.items():
        if pat in name and (best is None or len(pat) > len(best[0])):
            best = (pat, d)
    return best[1] if best else ShardingDirective("replicated")


# --------------------------------------------------------------------------- expert parallel
def expert_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """(first expert, count) owned by ``rank``; the first total % world ranks hold one more."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    base, rem = divmod(total, world)
    if rank < rem:
        return rank * (base + 1), base + 1
    return rem * (base + 1) + (rank - rem) * base, base


def rank_for_expert(expert: int, total: int, world: int) -> int:
    if not (0 <= expert < total):
        raise ValueError("expert out of range")
    base, rem = divmod(total, world)
    big = rem * (base + 1)
    return expert // (base + 1) if expert < big else rem + (expert - big) // base


def weighted_placement(total: int, weights: Sequence[float]) -> List[Tuple[int, int]]:
    """Contiguous ranges proportional to ``weights`` (e.g. free memory per rank)."""
    s = float(sum(weights))
    counts = [int(math.floor(total * w / s)) for w in weights]
    order = sorted(range(len(weights)), key=lambda i: -(total * weights[i] / s - counts[i]))
    for i in order[: total - sum(counts)]:
        counts[i] += 1
    out, off = [], 0
    for c in counts:
        out.append((off, c))
        off += c
    return out


def expert_capacity(num_tokens: int, top_k: int, num_experts: int, factor: float = 1.25) -> int:
    return max(int(math.ceil(num_tokens * top_k / num_experts * factor)), 1)


def apply_capacity(expert_ids, capacity: int, num_experts: int):
    """Keep at most ``capacity`` assignments per expert in arrival order. Returns a boolean keep-mask."""
    import torch
    flat = expert_ids.reshape(-1)
    onehot = torch.nn.functional.one_hot(flat, num_experts)
    pos = (torch.cumsum(onehot, 0) * onehot).sum(-1) - 1
    return (pos < capacity).view(expert_ids.shape)


def load_balancing_loss(router_probs, expert_ids, num_experts: int):
    """Switch-transformer auxiliary loss: E * sum_e (fraction of assignments to e) * (mean router prob of e)."""
    import torch
    f = torch.bincount(expert_ids.reshape(-1), minlength=num_experts).float()
    f = f / f.sum().clamp(min=1.0)
    p = router_probs.float().mean(0)
    return num_experts * (f * p).sum()


# --------------------------------------------------------------------------- ZeRO
def zero_owner_map(param_names: Sequence[str], world: int) -> Dict[str, int]:
    return {n: i % world for i, n in enumerate(sorted(param_names))}


def zero_owned(param_names: Sequence[str], rank: int, world: int) -> List[str]:
    return [n for n, o in zero_owner_map(param_names, world).items() if o == rank]


def flat_shard(total_chunks: int, rank: int, world: int) -> Tuple[int, int]:
    """Chunk range of the flat optimizer buffer owned by ``rank`` (what the fused DP kernel updates)."""
    per = -(-total_chunks // world)
    return min(per * rank, total_chunks), min(per * (rank + 1), total_chunks)


# --------------------------------------------------------------------------- pipeline schedules
def schedule_1f1b(num_stages: int, num_micro: int, stage: int) -> List[Tuple[str, Optional[int]]]:
    if num_micro < num_stages:
        raise ValueError("1F1B requires num_micro_batches >= num_stages")
    first, last = stage == 0, stage == num_stages - 1
    out: List[Tuple[str, Optional[int]]] = []

    def fwd(mb):
        if not first:
            out.append(("recv_activation", mb))
        out.append(("forward", mb))
        if not last:
            out.append(("send_activation", mb))

    def bwd(mb):
        if not last:
            out.append(("recv_gradient", mb))
        out.append(("backward", mb))
        if not first:
            out.append(("send_gradient", mb))
    warm = min(num_stages - stage - 1, num_micro)
    for mb in range(warm):
        fwd(mb)
    steady = num_micro - warm
    for i in range(steady):
        fwd(warm + i)
        bwd(i)
    for i in range(steady, num_micro):
        bwd(i)
    out.append(("weight_update", None))
    return out


def bubble_fraction(num_stages: int, num_micro: int) -> float:
    return 1.0 if num_micro == 0 else (num_stages - 1.0) / (num_micro + num_stages - 1.0)


def schedule_zero_bubble(num_stages: int, num_micro: int, stage: int) -> List[Tuple[str, Optional[int]]]:
    """ZB-H1-style schedule: backward split into B (input grad, on the critical path) and W (weight grad,
    deferred into what would be the cooldown bubble)."""
    if num_micro < num_stages:
        raise ValueError("zero-bubble schedule requires num_micro_batches >= num_stages")
    first, last = stage == 0, stage == num_stages - 1
    out: List[Tuple[str, Optional[int]]] = []
    pending_w: List[int] = []
    warm = min(num_stages - stage - 1, num_micro)

    def fwd(mb):
        if not first:
            out.append(("recv_activation", mb))
        out.append(("forward", mb))
        if not last:
            out.append(("send_activation", mb))

    def b(mb):
        if not last:
            out.append(("recv_gradient", mb))
        out.append(("backward_input", mb))
        if not first:
            out.append(("send_gradient", mb))
        pending_w.append(mb)
    for mb in range(warm):
        fwd(mb)
    steady = num_micro - warm
    for i in range(steady):
        fwd(warm + i)
        b(i)
        if len(pending_w) > stage:          # later stages defer fewer W steps
            out.append(("backward_weight", pending_w.pop(0)))
    for i in range(steady, num_micro):
        b(i)
        if pending_w:
            out.append(("backward_weight", pending_w.pop(0)))
    while pending_w:
        out.append(("backward_weight", pending_w.pop(0)))
    out.append(("weight_update", None))
    return out


# --------------------------------------------------------------------------- pipeline layer assignment
def assign_layers_proportional(num_layers: int, capacities: Sequence[float]) -> List[Tuple[int, int]]:
    """Contiguous [start, end) per stage, sizes proportional to ``capacities``; every stage gets >= 1 layer."""
    n = len(capacities)
    if num_layers < n:
        raise ValueError("fewer layers than stages")
    ranges = weighted_placement(num_layers - n, capacities)
    out, off = [], 0
    for _, c in ranges:
        out.append((off, off + c + 1))
        off += c + 1
    return out


def assign_layers_bandwidth_aware(layer_cost: Sequence[float], stage_speed: Sequence[float],
                                  link_seconds: Sequence[float]) -> List[Tuple[int, int]]:
    """Exhaustive search over contiguous splits minimising the slowest stage (compute/speed + outgoing link)."""
    L, S = len(layer_cost), len(stage_speed)
    prefix = [0.0]
    for c in layer_cost:
        prefix.append(prefix[-1] + c)
    best, best_cuts = float("inf"), None
    for cuts in itertools.combinations(range(1, L), S - 1):
        b = (0,) + cuts + (L,)
        worst = 0.0
        for s in range(S):
            t = (prefix[b[s + 1]] - prefix[b[s]]) / stage_speed[s] + (link_seconds[s] if s < S - 1 else 0.0)
            worst = max(worst, t)
        if worst < best:
            best, best_cuts = worst, b
    return [(best_cuts[s], best_cuts[s + 1]) for s in range(S)]
