"""Error taxonomy of the distributed layer (crates/pmetal-distributed/src/error.rs:145-185)."""
from __future__ import annotations


class DistributedError(Exception):
    kind = "generic"

    def is_recoverable(self) -> bool:
        return self.kind in ("connection_timeout", "peer_timeout", "heartbeat_timeout", "election_timeout",
                             "topology_changed")

    def is_peer_failure(self) -> bool:
        return self.kind in ("peer_lost", "peer_unreachable", "peer_timeout", "peer_incoherent_data",
                             "health_check_failed", "heartbeat_timeout")

    def is_fatal(self) -> bool:
        return self.kind in ("split_brain", "shutting_down", "cancelled", "version_mismatch", "namespace_mismatch")


def _mk(name: str, kind: str):
    return type(name, (DistributedError,), {"kind": kind})


ConnectionTimeout = _mk("ConnectionTimeout", "connection_timeout")
PeerTimeout = _mk("PeerTimeout", "peer_timeout")
PeerLost = _mk("PeerLost", "peer_lost")
PeerUnreachable = _mk("PeerUnreachable", "peer_unreachable")
HeartbeatTimeout = _mk("HeartbeatTimeout", "heartbeat_timeout")
ElectionTimeout = _mk("ElectionTimeout", "election_timeout")
TopologyChanged = _mk("TopologyChanged", "topology_changed")
NamespaceMismatch = _mk("NamespaceMismatch", "namespace_mismatch")
VersionMismatch = _mk("VersionMismatch", "version_mismatch")
ProtocolError = _mk("ProtocolError", "protocol")
SplitBrain = _mk("SplitBrain", "split_brain")
ShuttingDown = _mk("ShuttingDown", "shutting_down")
DeviceWaitTimeout = _mk("DeviceWaitTimeout", "peer_timeout")
