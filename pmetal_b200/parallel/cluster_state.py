"""Cluster bookkeeping: topology, collective strategy choice, health monitor, master election, metrics.

Host-side state machines of the reference's distributed crate, re-targeted at one NVSwitch box:

* ``Topology`` (topology.rs:32-530): nodes are GPUs; every pair is one NVSwitch hop, so the ring order
  is simply the sorted device list and the bandwidth matrix is uniform.
* ``choose_all_reduce`` (collective.rs:158-171): the reference picks tree below 1 MiB or world < 4, else
  ring; on NVSwitch the same byte threshold selects one-shot (latency) versus two-shot
  reduce-scatter + all-gather (bandwidth). k-ary tree helpers are kept (collective.rs:200-442).
* ``HealthMonitor`` (health.rs:28-440): heartbeats every 5 s, a peer is unhealthy after 15 s of silence
  or 3 consecutive failures.
* ``ElectionManager`` (election.rs:32-490): Lamport clock + seniority; the candidate with the greatest
  (seniority, commands_seen, peer id) wins; a campaign ends at the timeout.
* ``Metrics`` (metrics.rs:19-415): counters, gauges and histograms with p50/p95/p99 over the last 1000 samples.
None of these touch a device; they are driven by the host threads of each rank and tested on CPU.
"""
from __future__ import annotations

import bisect
import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

ONE_SHOT_MAX_BYTES = 1 << 20


# --------------------------------------------------------------------------- topology
@dataclass
class NodeInfo:
    peer_id: str
    device_index: int = 0
    memory_bytes: int = 0
    link: str = "nvlink"        # nvlink | pcie | loopback


class Topology:
    LINK_GBPS = {"nvlink": 900.0 * 8, "pcie": 64.0 * 8, "loopback": 1e6}
    LINK_LATENCY_US = {"nvlink": 2.0, "pcie": 5.0, "loopback": 0.1}

    def __init__(self, nodes: Sequence[NodeInfo]):
        self.nodes = sorted(nodes, key=lambda n: n.peer_id)

    @classmethod
    def local_box(cls, n_gpus: Optional[int] = None) -> "Topology":
        import torch
        n = n_gpus if n_gpus is not None else (torch.cuda.device_count() if torch.cuda.is_available() else 0)
        nodes = []
        for i in range(n):
            mem = torch.cuda.get_device_properties(i).total_memory if torch.cuda.is_available() else 0
            nodes.append(NodeInfo(f"gpu{i:02d}", i, mem, "nvlink"))
        return cls(nodes)

    def ring_order(self) -> List[str]:
        return [n.peer_id for n in self.nodes]

    def ring_next(self, peer_id: str) -> str:
        ids = self.ring_order()
        return ids[(ids.index(peer_id) + 1) % len(ids)]

    def ring_prev(self, peer_id: str) -> str:
        ids = self.ring_order()
        return ids[(ids.index(peer_id) - 1) % len(ids)]

    def ring_bandwidth_gbps(self) -> float:
        return min((self.LINK_GBPS[n.link] for n in self.nodes), default=0.0)

    def is_fully_connected_nvlink(self) -> bool:
        return len(self.nodes) > 0 and all(n.link == "nvlink" for n in self.nodes)

    def status_table(self) -> List[dict]:
        return [{"peer": n.peer_id, "device": n.device_index, "memory_gib": round(n.memory_bytes / 2 ** 30, 1),
                 "link": n.link, "gbps": self.LINK_GBPS[n.link], "latency_us": self.LINK_LATENCY_US[n.link]}
                for n in self.nodes]


# --------------------------------------------------------------------------- collective strategies
def choose_all_reduce(nbytes: int, world: int, strategy: str = "auto") -> str:
    """Returns "one_shot" (every rank reads all peers) or "two_shot" (reduce-scatter then all-gather)."""
    if strategy != "auto":
        return strategy
    return "one_shot" if (nbytes < ONE_SHOT_MAX_BYTES or world < 4) else "two_shot"


def tree_parent(rank: int, arity: int = 2) -> Optional[int]:
    return None if rank == 0 else (rank - 1) // arity


def tree_children(rank: int, world: int, arity: int = 2) -> List[int]:
    return [c for c in range(rank * arity + 1, rank * arity + arity + 1) if c < world]


def tree_depth(world: int, arity: int = 2) -> int:
    d, n = 0, 1
    while n < world:
        n = n * arity + 1
        d += 1
    return d


# --------------------------------------------------------------------------- health
@dataclass
class PeerHealth:
    last_seen: float
    consecutive_failures: int = 0
    healthy: bool = True
    latency_ms: float = 0.0


class HealthMonitor:
    def __init__(self, interval: float = 5.0, timeout: float = 15.0, max_failures: int = 3,
                 clock: Callable[[], float] = time.monotonic):
        self.interval, self.timeout, self.max_failures, self.clock = interval, timeout, max_failures, clock
        self.peers: Dict[str, PeerHealth] = {}
        self._lock = threading.Lock()

    def add_peer(self, peer: str) -> None:
        with self._lock:
            self.peers[peer] = PeerHealth(self.clock())

    def remove_peer(self, peer: str) -> None:
        with self._lock:
            self.peers.pop(peer, None)

    def record_heartbeat(self, peer: str, latency_ms: float = 0.0) -> None:
        with self._lock:
            h = self.peers.setdefault(peer, PeerHealth(self.clock()))
            h.last_seen, h.consecutive_failures, h.healthy, h.latency_ms = self.clock(), 0, True, latency_ms

    def record_failure(self, peer: str) -> bool:
        """Returns True when this failure turned the peer unhealthy."""
        with self._lock:
            h = self.peers.setdefault(peer, PeerHealth(self.clock()))
            h.consecutive_failures += 1
            if h.healthy and h.consecutive_failures >= self.max_failures:
                h.healthy = False
                return True
            return False

    def check(self) -> List[str]:
        """Marks peers silent for longer than ``timeout`` unhealthy; returns the newly unhealthy ones."""
        now, out = self.clock(), []
        with self._lock:
            for p, h in self.peers.items():
                if h.healthy and now - h.last_seen > self.timeout:
                    h.healthy = False
                    out.append(p)
        return out

    def unhealthy(self) -> List[str]:
        with self._lock:
            return sorted(p for p, h in self.peers.items() if not h.healthy)

    def summary(self) -> dict:
        with self._lock:
            n = len(self.peers)
            bad = sum(1 for h in self.peers.values() if not h.healthy)
            lat = [h.latency_ms for h in self.peers.values() if h.healthy]
        return {"total_peers": n, "healthy": n - bad, "unhealthy": bad,
                "mean_latency_ms": sum(lat) / len(lat) if lat else 0.0}


# --------------------------------------------------------------------------- election
@dataclass
class ElectionMessage:
    clock: int
    seniority: float
    proposed_session: int
    commands_seen: int
    sender: str
    vote_for: str


class ElectionManager:
    def __init__(self, local_peer: str, election_timeout: float = 3.0, clock: Callable[[], float] = time.monotonic):
        self.local, self.timeout, self._now = local_peer, election_timeout, clock
        self.state = "idle"          # idle | campaigning | master | follower
        self.master: Optional[str] = None
        self.session = 0
        self.lamport = 0
        self.commands_seen = 0
        self.start = clock()
        self.candidates: Dict[str, Tuple[float, int, str]] = {}
        self.vote: Optional[str] = None
        self._deadline = 0.0
        self.events: List[dict] = []

    def seniority(self) -> float:
        return self._now() - self.start

    def _key(self, seniority: float, commands: int, peer: str):
        return (seniority, commands, peer)

    def start_election(self) -> ElectionMessage:
        self.lamport += 1
        self.session += 1
        self.state = "campaigning"
        self.candidates = {self.local: self._key(self.seniority(), self.commands_seen, self.local)}
        self.vote = self.local
        self._deadline = self._now() + self.timeout
        self.events.append({"event": "started", "session": self.session})
        return ElectionMessage(self.lamport, self.seniority(), self.session, self.commands_seen, self.local, self.local)

    def handle_message(self, m: ElectionMessage) -> Optional[ElectionMessage]:
        """Merge a peer's campaign message; returns our updated vote to broadcast when it changed."""
        self.lamport = max(self.lamport, m.clock) + 1
        if m.proposed_session < self.session:
            return None
        if m.proposed_session > self.session or self.state in ("idle", "master", "follower"):
            self.session = max(self.session, m.proposed_session)
            self.state = "campaigning"
            self.candidates = {self.local: self._key(self.seniority(), self.commands_seen, self.local)}
            self._deadline = self._now() + self.timeout
        self.candidates[m.sender] = self._key(m.seniority, m.commands_seen, m.sender)
        best = max(self.candidates.values())[2]
        if best != self.vote:
            self.vote = best
            return ElectionMessage(self.lamport, self.seniority(), self.session, self.commands_seen, self.local, best)
        return None

    def tick(self) -> Optional[dict]:
        """Finish the campaign once the timeout has passed."""
        if self.state != "campaigning" or self._now() < self._deadline:
            return None
        winner = max(self.candidates.values())[2]
        self.master = winner
        self.state = "master" if winner == self.local else "follower"
        ev = ({"event": "elected_master", "session": self.session} if winner == self.local
              else {"event": "new_master", "master": winner, "session": self.session})
        self.events.append(ev)
        return ev

    def report_masters(self, masters: Sequence[str]) -> Optional[dict]:
        if len(set(masters)) > 1:
            ev = {"event": "split_brain", "masters": sorted(set(masters))}
            self.events.append(ev)
            return ev
        return None


# --------------------------------------------------------------------------- metrics
class Histogram:
    def __init__(self, window: int = 1000):
        self.samples: deque = deque(maxlen=window)
        self.count, self.total = 0, 0.0

    def observe(self, v: float) -> None:
        self.samples.append(v)
        self.count += 1
        self.total += v

    def percentile(self, q: float) -> float:
        if not self.samples:
            return 0.0
        s = sorted(self.samples)
        return s[min(int(q * len(s)), len(s) - 1)]

    def snapshot(self) -> dict:
        return {"count": self.count, "mean": self.total / self.count if self.count else 0.0,
                "p50": self.percentile(0.50), "p95": self.percentile(0.95), "p99": self.percentile(0.99)}


class Metrics:
    def __init__(self):
        self.counters: Dict[str, float] = {}
        self.gauges: Dict[str, float] = {}
        self.hists: Dict[str, Histogram] = {}
        self._lock = threading.Lock()

    def inc(self, name: str, v: float = 1.0) -> None:
        with self._lock:
            self.counters[name] = self.counters.get(name, 0.0) + v

    def set(self, name: str, v: float) -> None:
        with self._lock:
            self.gauges[name] = v

    def observe(self, name: str, v: float) -> None:
        with self._lock:
            self.hists.setdefault(name, Histogram()).observe(v)

    def timer(self, name: str) -> "TimingGuard":
        return TimingGuard(self, name)

    def snapshot(self) -> dict:
        with self._lock:
            return {"counters": dict(self.counters), "gauges": dict(self.gauges),
                    "histograms": {k: h.snapshot() for k, h in self.hists.items()}}


class TimingGuard:
    def __init__(self, m: Metrics, name: str):
        self.m, self.name = m, name

    def __enter__(self):
        self.t0 = time.perf_counter()
        return self

    def __exit__(self, *a):
        self.m.observe(self.name, (time.perf_counter() - self.t0) * 1e3)
        self.m.inc(self.name + "_count")
