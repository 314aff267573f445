"""Pipeline parallelism: activation wire messages, stage execution for inference, and a 1F1B executor for training.

Wire format of an activation (crates/pmetal-distributed/src/activation_transport.rs:19-175): ``u64 nonce, u32 layer_id,
u32 ndim, u32 shape[ndim], u8 dtype tag (0 f16, 1 f32, 2 bf16), data``, little-endian; the fp16 codec of
activation_codec.rs:9-95 down-casts before sending. Between GPUs of one node messages travel as NCCL point-to-point
transfers (a small int64 header tensor followed by the payload) so they overlap with compute on the side stream;
``serialize`` / ``deserialize`` keep the byte format for the TCP transport and for tests.

The last stage samples greedily and returns a 4-byte token to stage 0, as the reference harness does
(pipeline.rs:36-600, pipeline_harness.rs:41-300). Schedules come from ``plans.schedule_1f1b`` /
``plans.schedule_zero_bubble``."""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

DTYPE_TAGS = {torch.float16: 0, torch.float32: 1, torch.bfloat16: 2}
TAG_DTYPES = {v: k for k, v in DTYPE_TAGS.items()}
MAX_DIMS = 8


@dataclass
class ActivationMessage:
    nonce: int
    layer_id: int
    tensor: torch.Tensor

    def serialize(self) -> bytes:
        t = self.tensor.detach().contiguous().cpu()
        if t.dtype not in DTYPE_TAGS:
            t = t.float()
        head = struct.pack("<QII", self.nonce, self.layer_id, t.dim()) + struct.pack(f"<{t.dim()}I", *t.shape)
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        return head + bytes([DTYPE_TAGS[t.dtype]]) + raw

    @classmethod
    def deserialize(cls, buf: bytes) -> "ActivationMessage":
        if len(buf) < 17:
            raise ValueError("activation message too short")
        nonce, layer, nd = struct.unpack_from("<QII", buf, 0)
        if nd > MAX_DIMS or len(buf) < 16 + 4 * nd + 1:
            raise ValueError("activation message header is malformed")
        shape = struct.unpack_from(f"<{nd}I", buf, 16)
        tag = buf[16 + 4 * nd]
        if tag not in TAG_DTYPES:
            raise ValueError(f"unknown dtype tag: {tag}")
        dt = TAG_DTYPES[tag]
        n = 1
        for d in shape:
            n *= d
        data = buf[17 + 4 * nd:]
        esz = torch.tensor([], dtype=dt).element_size()
        if len(data) != n * esz:
            raise ValueError(f"activation payload is {len(data)} bytes, expected {n * esz}")
        t = torch.frombuffer(bytearray(data), dtype=dt).reshape(shape) if n else torch.empty(shape, dtype=dt)
        return cls(nonce, layer, t)


def encode_fp16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float16)


def decode_fp16(t: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    return t.to(dtype)


# ------------------------------------------------------------------------------------------- device transport
def send_activation(msg: ActivationMessage, dst: int, group=None) -> None:
    t = msg.tensor.contiguous()
    head = torch.tensor([msg.nonce, msg.layer_id, DTYPE_TAGS.get(t.dtype, 1), t.dim()] + list(t.shape) +
                        [0] * (MAX_DIMS - t.dim()), dtype=torch.int64, device=t.device)
    dist.send(head, dst, group=group)
    dist.send(t if t.dtype in DTYPE_TAGS else t.float(), dst, group=group)


def recv_activation(src: int, device, group=None) -> ActivationMessage:
    head = torch.empty(4 + MAX_DIMS, dtype=torch.int64, device=device)
    dist.recv(head, src, group=group)
    h = head.tolist()
    shape = h[4:4 + h[3]]
    t = torch.empty(shape, dtype=TAG_DTYPES[h[2]], device=device)
    dist.recv(t, src, group=group)
    return ActivationMessage(h[0], h[1], t)


def pipeline_ring_step(msg: ActivationMessage, rank: int, world: int, group=None) -> ActivationMessage:
    """Every rank sends its activation to the next stage and receives from the previous one (bench primitive)."""
    t = msg.tensor.contiguous()
    r = torch.empty_like(t)
    reqs = dist.batch_isend_irecv([dist.P2POp(dist.isend, t, (rank + 1) % world, group),
                                   dist.P2POp(dist.irecv, r, (rank - 1) % world, group)])
    for q in reqs:
        q.wait()
    return ActivationMessage(msg.nonce, (msg.layer_id - 1) % world, r)


# ------------------------------------------------------------------------------------------- inference stages
class PipelineStage:
    """Holds layers [start, end) of a DecoderLM; stage 0 also embeds, the last stage also owns the head."""

    def __init__(self, model, start: int, end: int, rank: int, world: int, group=None):
        self.model, self.start, self.end, self.rank, self.world, self.group = model, start, end, rank, world, group
        self.first, self.last = rank == 0, rank == world - 1

    @torch.no_grad()
    def forward_range(self, ids: Optional[torch.Tensor], h: Optional[torch.Tensor]) -> torch.Tensor:
        """Run this stage's layers. Stage 0 takes token ids, the others hidden states [T, H]; the last stage's result
        is final-normed."""
        if ids is None:
            ids = torch.zeros(h.shape[0], dtype=torch.int64, device=h.device)
        return self.model.forward_hidden(ids, layer_range=(self.start, self.end), hidden_in=h)

    @torch.no_grad()
    def step(self, token_ids: Optional[torch.Tensor], nonce: int = 0) -> Optional[int]:
        """One full-sequence forward through the pipeline. Stage 0 passes ``token_ids``; returns the greedy next token on
        stage 0 (None elsewhere)."""
        dev = self.model.embed_tokens.device
        if self.first:
            h = self.forward_range(token_ids.to(dev), None)
        else:
            hin = decode_fp16(recv_activation(self.rank - 1, dev, self.group).tensor, self.model.embed_tokens.dtype)
            h = self.forward_range(None, hin)
        if not self.last:
            send_activation(ActivationMessage(nonce, self.end, encode_fp16(h)), self.rank + 1, self.group)
        tok = torch.zeros(1, dtype=torch.int32, device=dev)
        if self.last:
            tok[0] = int(self.model.logits(h[-1:]).argmax(-1))
        if self.world > 1:                      # 4-byte result back to the first stage
            if self.last:
                dist.send(tok, 0, group=self.group)
            elif self.first:
                dist.recv(tok, self.world - 1, group=self.group)
        return int(tok[0]) if self.first else None


# ------------------------------------------------------------------------------------------- 1F1B training executor
def run_schedule(schedule: Sequence[Tuple[str, Optional[int]]], stage_fn: Callable[[torch.Tensor], torch.Tensor],
                 inputs: Dict[int, torch.Tensor], rank: int, world: int, loss_fn: Optional[Callable] = None,
                 activation_like: Optional[torch.Tensor] = None, group=None, on_update: Optional[Callable] = None):
    """Executes a 1F1B schedule (``plans.schedule_1f1b``) on one stage. ``inputs`` holds micro-batch inputs on stage 0
    (and targets for ``loss_fn`` on the last stage). Activations and gradients travel as point-to-point transfers."""
    saved_in: Dict[int, torch.Tensor] = {}
    saved_out: Dict[int, torch.Tensor] = {}
    recv_act: Dict[int, torch.Tensor] = {}
    recv_grad: Dict[int, torch.Tensor] = {}
    losses: List[float] = []
    pending = []          # sends are asynchronous: a blocking send of activation i+1 would deadlock against the next
    keep = []             # stage's blocking send of gradient i (the two stages wait on each other's receive)
    for action, mb in schedule:
        if action == "recv_activation":
            t = torch.empty_like(activation_like)
            dist.recv(t, rank - 1, group=group)
            recv_act[mb] = t
        elif action == "forward":
            x = inputs[mb] if rank == 0 else recv_act.pop(mb)
            x = x.detach().requires_grad_(rank != 0)
            y = stage_fn(x)
            saved_in[mb], saved_out[mb] = x, y
        elif action == "send_activation":
            buf = saved_out[mb].detach().contiguous()
            keep.append(buf)
            pending.append(dist.isend(buf, rank + 1, group=group))
        elif action == "recv_gradient":
            t = torch.empty_like(saved_out[mb])
            dist.recv(t, rank + 1, group=group)
            recv_grad[mb] = t
        elif action == "backward":
            y = saved_out.pop(mb)
            if rank == world - 1 and loss_fn is not None:
                loss = loss_fn(y, mb)
                losses.append(float(loss.detach()))
                loss.backward()
            else:
                y.backward(recv_grad.pop(mb))
        elif action == "send_gradient":
            buf = saved_in.pop(mb).grad.contiguous()
            keep.append(buf)
            pending.append(dist.isend(buf, rank - 1, group=group))
        elif action == "weight_update":
            for r in pending:
                r.wait()
            pending.clear()
            keep.clear()
            if on_update:
                on_update()
    for r in pending:
        r.wait()
    return losses


# ------------------------------------------------------------------------------------------- local in-memory pipeline
def plan_local_pipeline(num_layers: int, stages: int) -> List[Tuple[int, int]]:
    """Contiguous, near-equal layer ranges for a pipeline whose stages live in one process and hand activations over
    in-memory channels (the reference plans such a pipeline across the two dies of an Ultra chip,
    crates/pmetal-distributed/src/ultrafusion.rs)."""
    stages = max(1, min(stages, num_layers))
    base, extra = divmod(num_layers, stages)
    out, start = [], 0
    for s in range(stages):
        n = base + (1 if s < extra else 0)
        out.append((start, start + n))
        start += n
    return out


def run_local_pipeline(stage_fns: Sequence, micro_batches: Sequence):
    """Run ``stage_fns[s](x)`` as a pipeline of threads connected by queues; results come back in input order."""
    import queue
    import threading
    qs = [queue.Queue(maxsize=2) for _ in range(len(stage_fns) + 1)]
    errors: List[BaseException] = []

    def worker(s):
        while True:
            item = qs[s].get()
            if item is None:
                qs[s + 1].put(None)
                return
            try:
                qs[s + 1].put(stage_fns[s](item))
            except BaseException as e:                      # the failure travels down the pipe instead of hanging it
                errors.append(e)
                qs[s + 1].put(None)
                return
    threads = [threading.Thread(target=worker, args=(s,), daemon=True) for s in range(len(stage_fns))]
    for t in threads:
        t.start()

    def feed():
        for mb in micro_batches:
            qs[0].put(mb)
        qs[0].put(None)
    threading.Thread(target=feed, daemon=True).start()
    out = []
    while True:
        item = qs[-1].get()
        if item is None:
            break
        out.append(item)
    for t in threads:
        t.join(timeout=5)
    if errors:
        raise errors[0]
    return out


class StreamMultiplexer:
    """Routes activation / result messages of concurrent requests by their nonce.

    The last pipeline stage answers on one channel for every request in flight; each request registers its nonce and
    waits on its own queue, a reader thread (or the caller) hands every incoming message to :meth:`dispatch`. Messages
    for a nonce nobody waits for are counted and dropped, so a cancelled request cannot block the channel
    (crates/pmetal-distributed/src/pipeline.rs: the request router of the pipeline harness)."""

    def __init__(self, max_pending: int = 1024):
        import threading
        self._lock = threading.Lock()
        self._queues: dict = {}
        self.max_pending = max_pending
        self.dropped = 0

    def register(self, nonce: int):
        """Queue on which the messages of ``nonce`` will arrive; raises when the nonce is in use or the table is full."""
        import queue
        with self._lock:
            if nonce in self._queues:
                raise KeyError(f"nonce {nonce} is already registered")
            if len(self._queues) >= self.max_pending:
                raise RuntimeError("too many requests in flight")
            q = self._queues[nonce] = queue.Queue()
            return q

    def dispatch(self, msg) -> bool:
        """Deliver ``msg`` (anything with a ``nonce``) to its request; False when nobody is waiting for it."""
        with self._lock:
            q = self._queues.get(msg.nonce)
            if q is None:
                self.dropped += 1
                return False
        q.put(msg)
        return True

    def wait(self, nonce: int, timeout: Optional[float] = None):
        """Next message of ``nonce`` (raises ``queue.Empty`` after ``timeout`` seconds)."""
        with self._lock:
            q = self._queues[nonce]
        return q.get(timeout=timeout)

    def close(self, nonce: int) -> None:
        with self._lock:
            self._queues.pop(nonce, None)

    def pending(self) -> int:
        with self._lock:
            return len(self._queues)
