"""Serving with a model cut over several ranks (``parallel.tp_model.shard_for_serving``): rank 0 owns the HTTP port,
the request queue, the block allocator, the prefix cache and the sampler; the other ranks own only their slice of the
weights and of the key/value pool, and repeat every model call of rank 0.

Before each model call the leader publishes a *step descriptor* over a CPU (gloo) group: the token ids and the batch
metadata of an eager cached forward, or the contents of the pinned staging buffers of a graph replay. A follower rebuilds
the same device-side metadata, runs the same forward on its slice (the all-reduces inside pair up with the leader's) and
discards the logits. Followers keep no allocator state: block numbers are decided on rank 0, and every rank's pool has
the same number of blocks, so a block number means the same place everywhere.

The reference serves a sharded model the same way: one coordinator ticks the scheduler and its peers run the layers they
hold for every step it announces (crates/pmetal-distributed/src/pipeline.rs:1-120 for the step protocol,
crates/pmetal-serve/src/lib.rs for the single HTTP owner)."""
from __future__ import annotations

import datetime
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

KIND_STOP, KIND_PAGED, KIND_GRAPH, KIND_CAPTURE = 0, 1, 2, 3
_HDR = 10


class StepChannel:
    """Leader-to-followers broadcast of step descriptors: a fixed header (kind, payload length, up to eight integers)
    and one int64 payload. ``muted`` > 0 suppresses publication (graph warm-up and capture run the forward on every rank
    by themselves)."""

    def __init__(self, group=None, leader: int = 0):
        self.group = group
        self.leader_rank = leader
        self.leader = dist.get_rank() == leader
        self.muted = 0
        self.published = 0

    @staticmethod
    def control_group():
        """A gloo group over all ranks whose waits do not time out while the server idles."""
        return dist.new_group(backend="gloo", timeout=datetime.timedelta(days=365))

    def publish(self, kind: int, scalars: List[int], payload: Optional[torch.Tensor] = None) -> None:
        hdr = torch.zeros(_HDR, dtype=torch.int64)
        hdr[0] = kind
        hdr[1] = 0 if payload is None else payload.numel()
        for i, v in enumerate(scalars):
            hdr[2 + i] = int(v)
        dist.broadcast(hdr, self.leader_rank, group=self.group)
        if payload is not None and payload.numel():
            dist.broadcast(payload, self.leader_rank, group=self.group)
        self.published += 1

    def receive(self) -> Tuple[int, List[int], torch.Tensor]:
        hdr = torch.zeros(_HDR, dtype=torch.int64)
        dist.broadcast(hdr, self.leader_rank, group=self.group)
        payload = torch.empty(int(hdr[1]), dtype=torch.int64)
        if payload.numel():
            dist.broadcast(payload, self.leader_rank, group=self.group)
        return int(hdr[0]), [int(v) for v in hdr[2:]], payload

    # ------------------------------------------------------------------ leader side
    def publish_paged(self, input_ids: torch.Tensor, meta, all_logits: bool, return_hidden: bool) -> None:
        host = getattr(meta, "host", None)
        if host is None:
            host = tuple(t.cpu() for t in (meta.slots, meta.positions, meta.seq_lens, meta.q_start, meta.q_lens,
                                           meta.block_table))
        slots, pos, seq_lens, q_start, q_lens, bt = host
        i64 = lambda x: torch.as_tensor(x).to(torch.int64).reshape(-1)      # noqa: E731
        bt = torch.as_tensor(bt)
        n, mb = bt.shape
        payload = torch.cat([i64(input_ids.cpu()), i64(slots), i64(pos), i64(seq_lens), i64(q_start), i64(q_lens), i64(bt)])
        self.publish(KIND_PAGED, [input_ids.numel(), n, mb, meta.max_q, meta.max_kv, int(all_logits) | int(return_hidden) << 1],
                     payload)

    def publish_graph(self, nb: int, mb: int, n: int, pad_block: int, h64: torch.Tensor, h32: torch.Tensor) -> None:
        self.publish(KIND_GRAPH, [nb, mb, n, pad_block], torch.cat([h64, h32.to(torch.int64)]))

    def stop(self) -> None:
        if self.leader:
            self.publish(KIND_STOP, [])


def meta_from_payload(sc: List[int], payload: torch.Tensor, device):
    """Inverse of ``StepChannel.publish_paged``: (input ids, BatchMeta, all_logits, return_hidden) on ``device``."""
    from ..models.kv_cache import BatchMeta
    T, n, mb, max_q, max_kv, flags = sc[:6]
    cuts = [T, T, T, n, n, n, n * mb]
    parts, o = [], 0
    for c in cuts:
        parts.append(payload[o:o + c])
        o += c
    ids, slots, pos, seq_lens, q_start, q_lens, bt = parts
    i32 = lambda x: x.to(torch.int32).to(device, non_blocking=True)      # noqa: E731
    meta = BatchMeta(list(range(n)), i32(bt.view(n, mb)), i32(seq_lens), i32(q_start), i32(q_lens),
                     slots.to(device, non_blocking=True), i32(pos), T, max_q, max_kv)
    return ids.to(device, non_blocking=True), meta, bool(flags & 1), bool(flags & 2)


@torch.no_grad()
def follow(model, cache, channel: StepChannel) -> int:
    """Follower loop: repeat the leader's model calls until it says stop. Returns the number of steps replayed."""
    from ..models.generation import GraphedDecoder
    graphed: Optional[GraphedDecoder] = None
    steps = 0
    while True:
        kind, sc, payload = channel.receive()
        if kind == KIND_STOP:
            return steps
        steps += 1
        if kind == KIND_PAGED:
            ids, meta, all_logits, hidden = meta_from_payload(sc, payload, cache.device)
            model.forward_paged(ids, cache, meta, all_logits=all_logits, return_hidden=hidden)
        elif kind in (KIND_GRAPH, KIND_CAPTURE):
            nb, mb, _, pad = sc[:4]
            if graphed is None:
                graphed = GraphedDecoder(model, cache, pad_block=pad)
            st = graphed._state(nb, mb)
            if kind == KIND_CAPTURE:
                continue
            done = st.get("copied")
            if done is not None:
                done.synchronize()          # the previous step's copies out of the pinned buffers have finished
            st["h64"].copy_(payload[:2 * nb])
            st["h32"].copy_(payload[2 * nb:].to(torch.int32))
            graphed._copy(st)
            if done is None:
                done = st["copied"] = torch.cuda.Event()
            done.record()
            st["graph"].replay()
        else:
            raise RuntimeError(f"unknown step kind {kind}")
