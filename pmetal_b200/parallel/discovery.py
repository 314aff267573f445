"""Node identity, peer discovery and link scoring for the cluster runtime.

The reference discovers Macs on a LAN with mDNS / libp2p, identifies them by an Ed25519 key under ``~/.pmetal`` and
scores the links between them (Thunderbolt / Ethernet / Wi-Fi) before fixing a ring order
(crates/pmetal-distributed/src/auto.rs:49-532, src/identity.rs, src/fabric/{mod,probe,score}.rs). On one NVSwitch node
the peers are the local GPUs: discovery enumerates them (or reads a static peer list for multi-process bootstrap),
the fabric probe classifies every GPU pair as NVLink / PCIe / none from the driver's peer-access answer, and the ring
order is deterministic (sorted peer ids) exactly as in the reference. The identity file format is kept: a 32-byte
Ed25519 private key, created with mode 0600 on first use; the peer id is the SHA-256 of the public key."""
from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

GRADIENT_PORT = 52416
DISCOVERY_PORT = 52415


# ------------------------------------------------------------------------------------------------ identity
class NodeIdentity:
    def __init__(self, private_bytes: bytes):
        from cryptography.hazmat.primitives import serialization
        from cryptography.hazmat.primitives.asymmetric.ed25519 import Ed25519PrivateKey
        self._key = Ed25519PrivateKey.from_private_bytes(private_bytes)
        self.public_bytes = self._key.public_key().public_bytes(serialization.Encoding.Raw, serialization.PublicFormat.Raw)
        self.peer_id = hashlib.sha256(self.public_bytes).hexdigest()[:32]

    @classmethod
    def load_or_create(cls, path: Optional[str] = None) -> "NodeIdentity":
        path = path or os.path.join(os.path.expanduser("~"), ".pmetal", "node_keypair")
        if os.path.exists(path):
            with open(path, "rb") as fh:
                raw = fh.read()
            if len(raw) != 32:
                raise ValueError(f"{path}: expected a 32-byte Ed25519 private key, found {len(raw)} bytes")
            return cls(raw)
        raw = os.urandom(32)
        os.makedirs(os.path.dirname(path), exist_ok=True)
        fd = os.open(path, os.O_WRONLY | os.O_CREAT | os.O_EXCL, 0o600)
        with os.fdopen(fd, "wb") as fh:
            fh.write(raw)
        return cls(raw)

    def sign(self, message: bytes) -> bytes:
        return self._key.sign(message)

    @staticmethod
    def verify(public_bytes: bytes, signature: bytes, message: bytes) -> bool:
        from cryptography.exceptions import InvalidSignature
        from cryptography.hazmat.primitives.asymmetric.ed25519 import Ed25519PublicKey
        try:
            Ed25519PublicKey.from_public_bytes(public_bytes).verify(signature, message)
            return True
        except InvalidSignature:
            return False


# ------------------------------------------------------------------------------------------------ fabric
@dataclass(frozen=True)
class LinkClass:
    name: str
    bandwidth_gbs: float      # nominal, per direction
    latency_us: float


NVLINK5 = LinkClass("nvlink5", 900.0, 2.0)
PCIE5 = LinkClass("pcie5", 64.0, 5.0)
HOST_TCP = LinkClass("tcp", 12.5, 50.0)
LOOPBACK = LinkClass("self", 7700.0, 0.5)
NONE = LinkClass("none", 0.0, float("inf"))


def classify_link(i: int, j: int, peer_access: Optional[bool], same_node: bool = True) -> LinkClass:
    """Link between devices i and j from what the driver reports."""
    if i == j:
        return LOOPBACK
    if not same_node:
        return HOST_TCP
    if peer_access is None:
        return NONE
    return NVLINK5 if peer_access else PCIE5


def link_score(link: LinkClass, nbytes: int = 64 << 20) -> float:
    """Lower is better: seconds to move ``nbytes`` once (latency + size / bandwidth), as the reference's LinkScore
    orders candidate links."""
    if link.bandwidth_gbs <= 0:
        return float("inf")
    return link.latency_us * 1e-6 + nbytes / (link.bandwidth_gbs * 1e9)


def probe_fabric(num_devices: Optional[int] = None, peer_access_fn=None) -> List[List[LinkClass]]:
    """Matrix of link classes between the local GPUs. ``peer_access_fn(i, j)`` defaults to the CUDA runtime's answer."""
    if peer_access_fn is None:
        import torch
        if num_devices is None:
            num_devices = torch.cuda.device_count() if torch.cuda.is_available() else 0

        def peer_access_fn(i, j):
            return bool(torch.cuda.can_device_access_peer(i, j))
    n = num_devices or 0
    return [[classify_link(i, j, None if i == j else peer_access_fn(i, j)) for j in range(n)] for i in range(n)]


# ------------------------------------------------------------------------------------------------ discovery
@dataclass
class Peer:
    peer_id: str
    addresses: List[Tuple[str, int]] = field(default_factory=list)
    device: Optional[int] = None
    memory_bytes: int = 0


def discover_local(identity: Optional[NodeIdentity] = None, num_devices: Optional[int] = None) -> List[Peer]:
    """One peer per local GPU; ids derive from the node identity so that they are stable across runs."""
    import torch
    n = num_devices if num_devices is not None else (torch.cuda.device_count() if torch.cuda.is_available() else 0)
    base = identity.peer_id if identity is not None else "local"
    peers = []
    for d in range(n):
        mem = torch.cuda.get_device_properties(d).total_memory if torch.cuda.is_available() and d < torch.cuda.device_count() else 0
        peers.append(Peer(f"{base}-gpu{d}", [("127.0.0.1", GRADIENT_PORT + d)], d, mem))
    return peers


def load_static_peers(path: str) -> List[Peer]:
    """``[{"peer_id": ..., "addresses": ["host:port", ...]}, ...]`` — the stand-in for LAN discovery."""
    with open(path, "r", encoding="utf-8") as fh:
        rows = json.load(fh)
    out = []
    for r in rows:
        addrs = []
        for a in r.get("addresses", []):
            host, _, port = a.rpartition(":")
            addrs.append((host, int(port)))
        out.append(Peer(r["peer_id"], addrs, r.get("device"), int(r.get("memory_bytes", 0))))
    return out


def ring_order(peers: Sequence[Peer]) -> List[Peer]:
    """Deterministic ring: peers sorted by id (crates/pmetal-distributed/src/topology.rs ring order)."""
    return sorted(peers, key=lambda p: p.peer_id)


def ring_neighbours(peers: Sequence[Peer], peer_id: str) -> Tuple[Peer, Peer]:
    order = ring_order(peers)
    i = next(k for k, p in enumerate(order) if p.peer_id == peer_id)
    return order[(i - 1) % len(order)], order[(i + 1) % len(order)]


def ring_bandwidth(fabric: List[List[LinkClass]], order: Sequence[int]) -> float:
    """Bandwidth of the slowest hop of a ring over device indices."""
    n = len(order)
    if n < 2:
        return LOOPBACK.bandwidth_gbs
    return min(fabric[order[i]][order[(i + 1) % n]].bandwidth_gbs for i in range(n))
