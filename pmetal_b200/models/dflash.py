"""DFlash: block-diffusion drafting for speculative decoding.

A small transformer proposes a whole block of tokens in one pass: its input is the target's embedding of
``[last accepted token, MASK, MASK, ...]`` and it cross-reads hidden states tapped from chosen layers of the target's
latest forward pass (keys/values are computed over ``[tapped context || block]``, queries over the block only, no
causal mask). The target verifies the block with one forward pass; the longest prefix on which its argmax agrees with
the draft is accepted plus the target's own next token, the cache is rolled back over the rejected tail, and the
tapped hidden states of the accepted positions condition the next draft. At temperature 0 the output equals plain
greedy decoding of the target whatever the draft proposes.

Reference: crates/pmetal-models/src/architectures/dflash_draft.rs:236-300 (attention), :443-470 (model forward),
crates/pmetal-models/src/dflash_decoder.rs:298-470 (loop, "parallel-replay" verification). Checkpoint names:
``layers.N.self_attn.{q,k,v,o}_proj``, ``{q,k}_norm``, ``layers.N.mlp.*``, ``fc``, ``hidden_norm``, ``norm``."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from .architectures.generic import GenericDecoderLM, KVCache, Norm, apply_rope


@dataclass
class DFlashConfig:
    hidden_size: int
    num_hidden_layers: int
    intermediate_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    target_layer_ids: List[int]
    mask_token_id: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    block_size: int = 16
    attention_bias: bool = False

    @classmethod
    def from_dict(cls, d: dict) -> "DFlashConfig":
        ex = d.get("dflash_config") or {}
        return cls(d["hidden_size"], d["num_hidden_layers"], d["intermediate_size"], d["num_attention_heads"],
                   d["num_key_value_heads"], d["head_dim"], d["vocab_size"], list(ex.get("target_layer_ids", [])),
                   int(ex.get("mask_token_id", 0)), d.get("rms_norm_eps", 1e-6), d.get("rope_theta", 1e6),
                   d.get("block_size", 16), d.get("attention_bias", False))


class _Attention(nn.Module):
    def __init__(self, c: DFlashConfig):
        super().__init__()
        self.c = c
        H, d = c.hidden_size, c.head_dim
        self.q_proj = nn.Linear(H, c.num_attention_heads * d, bias=c.attention_bias)
        self.k_proj = nn.Linear(H, c.num_key_value_heads * d, bias=c.attention_bias)
        self.v_proj = nn.Linear(H, c.num_key_value_heads * d, bias=c.attention_bias)
        self.o_proj = nn.Linear(c.num_attention_heads * d, H, bias=False)
        self.q_norm, self.k_norm = Norm(d, "rms", c.rms_norm_eps), Norm(d, "rms", c.rms_norm_eps)

    def forward(self, x, ctx, inv_freq):
        c = self.c
        B, Tq, _ = x.shape
        Tc = ctx.shape[1]
        q = self.q_norm(self.q_proj(x).view(B, Tq, c.num_attention_heads, c.head_dim)).transpose(1, 2)
        kv_in = torch.cat((ctx, x), 1)
        k = self.k_norm(self.k_proj(kv_in).view(B, Tc + Tq, c.num_key_value_heads, c.head_dim)).transpose(1, 2)
        v = self.v_proj(kv_in).view(B, Tc + Tq, c.num_key_value_heads, c.head_dim).transpose(1, 2)
        pos_k = torch.arange(Tc + Tq, device=x.device)[None, :, None].float() * inv_freq
        cos_k, sin_k = pos_k.cos().expand(B, -1, -1), pos_k.sin().expand(B, -1, -1)
        q = apply_rope(q, cos_k[:, Tc:], sin_k[:, Tc:], False)            # queries sit after the context rows
        k = apply_rope(k, cos_k, sin_k, False)
        g = c.num_attention_heads // c.num_key_value_heads
        if g > 1:
            k, v = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
        o = F.scaled_dot_product_attention(q, k, v)                       # no mask: the block sees itself entirely
        return self.o_proj(o.transpose(1, 2).reshape(B, Tq, -1))


class _Mlp(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.gate_proj = nn.Linear(c.hidden_size, c.intermediate_size, bias=False)
        self.up_proj = nn.Linear(c.hidden_size, c.intermediate_size, bias=False)
        self.down_proj = nn.Linear(c.intermediate_size, c.hidden_size, bias=False)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class _Layer(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.input_layernorm, self.post_attention_layernorm = Norm(c.hidden_size, "rms", c.rms_norm_eps), Norm(c.hidden_size, "rms", c.rms_norm_eps)
        self.self_attn, self.mlp = _Attention(c), _Mlp(c)

    def forward(self, x, ctx, inv_freq):
        x = x + self.self_attn(self.input_layernorm(x), ctx, inv_freq)
        return x + self.mlp(self.post_attention_layernorm(x))


class DFlashDraftModel(nn.Module):
    def __init__(self, c: DFlashConfig):
        super().__init__()
        self.c = c
        self.layers = nn.ModuleList([_Layer(c) for _ in range(c.num_hidden_layers)])
        self.fc = nn.Linear(len(c.target_layer_ids) * c.hidden_size, c.hidden_size, bias=False)
        self.hidden_norm, self.norm = Norm(c.hidden_size, "rms", c.rms_norm_eps), Norm(c.hidden_size, "rms", c.rms_norm_eps)
        self.register_buffer("inv_freq", 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2).float() / c.head_dim)),
                             persistent=False)

    def forward(self, noise_embedding: torch.Tensor, target_hidden: torch.Tensor) -> torch.Tensor:
        """noise_embedding [B, T_block, H]; target_hidden [B, T_ctx, L * H] -> block hidden states [B, T_block, H]."""
        ctx = self.hidden_norm(self.fc(target_hidden))
        x = noise_embedding
        for layer in self.layers:
            x = layer(x, ctx, self.inv_freq)
        return self.norm(x)

    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor], strict: bool = True):
        sd = {(k[len("model."):] if k.startswith("model.") else k): v for k, v in sd.items()}
        return self.load_state_dict(sd, strict=strict)


# ------------------------------------------------------------------------------------------------ draft tree
@dataclass
class DraftTree:
    """Budget-bounded tree of candidate continuations below the seed token (node 0 = root). ``tokens[i]`` / ``depths[i]``
    / ``parents[i]`` describe node i + 1; ``children[i]`` maps token id -> node index for node i."""
    tokens: List[int]
    depths: List[int]
    parents: List[int]
    children: List[Dict[int, int]]

    def visibility(self) -> torch.Tensor:
        """[N + 1, N + 1] bool: row i sees column j iff j is i or an ancestor of i."""
        n = len(self.tokens) + 1
        vis = torch.zeros(n, n, dtype=torch.bool)
        vis[0, 0] = True
        for i in range(1, n):
            vis[i] = vis[self.parents[i]]
            vis[i, i] = True
        return vis


def build_tree(draft_logits: torch.Tensor, budget: int) -> DraftTree:
    """Best-first expansion over the per-depth draft distributions ([horizon, vocab]): the state with the highest
    cumulative log-probability is materialised next; it spawns its sibling (next rank at the same depth, same parent)
    and its first child (rank 0 at the next depth). Ties pop in insertion order, so the tree is deterministic
    (crates/pmetal-models/src/ddtree.rs:164-280)."""
    import heapq
    tree = DraftTree([], [], [-1], [{}])
    horizon = draft_logits.shape[0]
    if budget <= 0 or horizon == 0:
        return tree
    k = max(1, min(budget, draft_logits.shape[1]))
    logp, ids = torch.log_softmax(draft_logits.float(), -1).topk(k, -1)
    logp, ids = logp.tolist(), ids.tolist()
    heap = [(-logp[0][0], 0, 1, 0, 0, logp[0][0])]          # (-logw, order, depth, rank, parent, logw)
    order = 1
    while heap and len(tree.tokens) < budget:
        _, _, depth, rank, parent, logw = heapq.heappop(heap)
        tok = ids[depth - 1][rank]
        index = len(tree.tokens) + 1
        tree.tokens.append(tok)
        tree.depths.append(depth)
        tree.parents.append(parent)
        tree.children.append({})
        tree.children[parent][tok] = index
        if rank + 1 < k:
            w = logw - logp[depth - 1][rank] + logp[depth - 1][rank + 1]
            heapq.heappush(heap, (-w, order, depth, rank + 1, parent, w))
            order += 1
        if depth < horizon:
            w = logw + logp[depth][0]
            heapq.heappush(heap, (-w, order, depth + 1, 0, index, w))
            order += 1
    return tree


def follow_verified_tree(tree: DraftTree, verifier_tokens: Sequence[int]) -> List[int]:
    """Walk from the root following the target's argmax at every visited node (``verifier_tokens[i]`` = argmax at node
    i). Returns the visited node indices, root first; the bonus token is the argmax at the last one."""
    path, node = [0], 0
    while True:
        nxt = tree.children[node].get(int(verifier_tokens[node]))
        if nxt is None:
            return path
        path.append(nxt)
        node = nxt


@dataclass
class DFlashStats:
    acceptance_lengths: List[int] = field(default_factory=list)
    total_drafted: int = 0
    total_accepted: int = 0

    @property
    def avg_acceptance_length(self) -> float:
        return sum(self.acceptance_lengths) / max(len(self.acceptance_lengths), 1)

    @property
    def acceptance_rate(self) -> float:
        return self.total_accepted / max(self.total_drafted, 1)


class DFlashDecoder:
    """Draft -> verify -> accept -> roll back loop over a ``GenericDecoderLM`` target with a contiguous KV cache."""

    def __init__(self, target: GenericDecoderLM, draft: DFlashDraftModel):
        self.target, self.draft = target, draft
        self.stats = DFlashStats()
        self._taps: Dict[int, torch.Tensor] = {}
        self._hooks = [target.model.layers[i].register_forward_hook(self._make_hook(i)) for i in draft.c.target_layer_ids]

    def _make_hook(self, i: int):
        def hook(_m, _inp, out):
            self._taps[i] = out
        return hook

    def close(self) -> None:
        for h in self._hooks:
            h.remove()

    def _forward(self, ids: torch.Tensor, cache: KVCache):
        self._taps.clear()
        logits = self.target(ids, cache)
        hidden = torch.cat([self._taps[i] for i in self.draft.c.target_layer_ids], -1)
        return logits, hidden

    @staticmethod
    def _rollback(cache: KVCache, n: int) -> None:
        for i in range(len(cache.k)):
            if cache.k[i] is not None:
                cache.k[i], cache.v[i] = cache.k[i][:, :, :-n], cache.v[i][:, :, :-n]

    @torch.no_grad()
    def generate_tree(self, prompt: Sequence[int], max_new_tokens: int, tree_budget: int = 12,
                      block_size: Optional[int] = None, stop_tokens: Sequence[int] = ()) -> List[int]:
        """Tree verification: the draft's per-position distributions become a tree of ``tree_budget`` candidates, the
        target scores all nodes in one forward pass under a tree attention mask (a node sees the context and its
        ancestors; its position is context length + depth), and the walk along the target's own argmax accepts a path
        through the tree. Keys / values of rejected nodes are dropped from the cache
        (crates/pmetal-models/src/dflash_decoder.rs:537-790). Greedy output equals plain greedy decoding."""
        c = self.draft.c
        bs = max(2, min(block_size or c.block_size, c.block_size))
        if tree_budget <= 0:
            return self.generate(prompt, max_new_tokens, block_size, stop_tokens)
        dev = self.target.model.embed_tokens.weight.device
        cache = self.target.new_cache()
        logits, hidden = self._forward(torch.tensor([list(prompt)], device=dev), cache)
        out = [int(logits[0, -1].argmax())]
        while len(out) < max_new_tokens and out[-1] not in stop_tokens:
            block = [out[-1]] + [c.mask_token_id] * (bs - 1)
            noise = self.target.model.embed_tokens(torch.tensor([block], device=dev))
            if self.target.c.embed_scale != 1.0:
                noise = noise * self.target.c.embed_scale
            dlogits = self.target.logits(self.draft(noise, hidden)[:, 1:])[0]
            tree = build_tree(dlogits, tree_budget)
            n = len(tree.tokens) + 1
            past = cache.length()
            ids = torch.tensor([[out[-1]] + tree.tokens], device=dev)
            pos = torch.tensor([[past] + [past + d for d in tree.depths]], device=dev)
            mask = torch.ones(1, 1, n, past + n, dtype=torch.bool, device=dev)
            mask[0, 0, :, past:] = tree.visibility().to(dev)
            self._taps.clear()
            vlogits = self.target(ids, cache, positions=pos, attn_mask=mask)
            vhidden = torch.cat([self._taps[i] for i in c.target_layer_ids], -1)
            verifier = vlogits[0].argmax(-1).tolist()
            path = follow_verified_tree(tree, verifier)
            keep = torch.tensor(list(range(past)) + [past + i for i in path], device=dev)
            for li in range(len(cache.k)):
                if cache.k[li] is not None:
                    cache.k[li], cache.v[li] = cache.k[li].index_select(2, keep), cache.v[li].index_select(2, keep)
            self.stats.acceptance_lengths.append(len(path))
            self.stats.total_drafted += len(tree.tokens)
            self.stats.total_accepted += len(path) - 1
            new = [tree.tokens[i - 1] for i in path[1:]] + [verifier[path[-1]]]
            for t in new:
                out.append(t)
                if t in stop_tokens or len(out) >= max_new_tokens:
                    break
            hidden = vhidden[:, torch.tensor(path, device=dev)]
        return out[:max_new_tokens]

    @torch.no_grad()
    def generate(self, prompt: Sequence[int], max_new_tokens: int, block_size: Optional[int] = None,
                 stop_tokens: Sequence[int] = ()) -> List[int]:
        c = self.draft.c
        bs = max(1, min(block_size or c.block_size, c.block_size))
        dev = self.target.model.embed_tokens.weight.device
        cache = self.target.new_cache()
        logits, hidden = self._forward(torch.tensor([list(prompt)], device=dev), cache)
        out = [int(logits[0, -1].argmax())]
        while len(out) < max_new_tokens and out[-1] not in stop_tokens:
            block = [out[-1]] + [c.mask_token_id] * (bs - 1)
            noise = self.target.model.embed_tokens(torch.tensor([block], device=dev))
            if self.target.c.embed_scale != 1.0:
                noise = noise * self.target.c.embed_scale
            dh = self.draft(noise, hidden)
            drafted = self.target.logits(dh[:, 1:]).argmax(-1)[0].tolist() if bs > 1 else []
            block[1:] = drafted
            vlogits, vhidden = self._forward(torch.tensor([block], device=dev), cache)
            verifier = vlogits[0].argmax(-1).tolist()
            matched = 0
            while matched < bs - 1 and drafted[matched] == verifier[matched]:
                matched += 1
            accepted_inputs = matched + 1
            self.stats.acceptance_lengths.append(accepted_inputs)
            self.stats.total_drafted += bs
            self.stats.total_accepted += matched
            if bs - accepted_inputs > 0:
                self._rollback(cache, bs - accepted_inputs)
            new = block[1:accepted_inputs] + [verifier[matched]]
            for t in new:
                out.append(t)
                if t in stop_tokens or len(out) >= max_new_tokens:
                    break
            hidden = vhidden[:, :accepted_inputs]
        return out[:max_new_tokens]


def load_dflash_pair(target_model: str, draft_model: str, device: str):
    """(target, draft, tokenizer or None): the target is ``random:<preset>`` or a checkpoint directory, the draft a
    DFlash checkpoint directory or ``random`` (a two-layer draft sized from the target, for smoke runs)."""
    import json
    import os

    from .loader import read_state_dict
    if target_model.startswith("random:"):
        from .config import preset
        target = GenericDecoderLM.from_hf_config(preset(target_model.split(":", 1)[1]).to_hf_dict()).init_weights(0.02, 0)
        tok = None
    else:
        from ..data.tokenizer import load_tokenizer
        with open(os.path.join(target_model, "config.json"), "r", encoding="utf-8") as fh:
            target = GenericDecoderLM.from_hf_config(json.load(fh))
        target.load_state_dict(read_state_dict(target_model), strict=False)
        tok = load_tokenizer(target_model)
    target = target.to(device).eval()
    c = target.c
    if draft_model == "random":
        n = c.num_layers
        dc = DFlashConfig(c.hidden_size, 2, c.intermediate_size, c.n_heads, c.n_kv_heads, c.head_dim, c.vocab_size,
                          sorted({n // 3, (2 * n) // 3, n - 1}), c.vocab_size - 1, c.norm_eps, c.rope_theta, 8)
        draft = DFlashDraftModel(dc)
    else:
        with open(os.path.join(draft_model, "config.json"), "r", encoding="utf-8") as fh:
            dc = DFlashConfig.from_dict(json.load(fh))
        draft = DFlashDraftModel(dc)
        draft.load_hf_state_dict(read_state_dict(draft_model), strict=False)
    return target, draft.to(device).eval(), tok
