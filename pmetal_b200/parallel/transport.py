"""Host-side TCP transport: ring wiring, length-prefixed frames, namespace (pre-shared key) handshake.

On the B200 box this channel only bootstraps a job (exchange of addresses / ids, CPU-rank tests, the
``cluster`` diagnostics); tensors move over NVLink. Wire behaviour follows the reference transport
(crates/pmetal-distributed/src/transport.rs:29-530, namespace.rs:30-150):

* every rank listens on its port and dials the next rank of the ring, trying each candidate address with
  exponential backoff (100 ms doubling to 5 s, at most ``max_retries`` rounds);
* right after connecting, the client sends the 8-byte magic ``PMETALD1`` followed by the 32-byte
  SHA3-256 of the namespace string; the server compares in constant time and answers one byte
  (1 = accepted, 0 = rejected); both sides fail with ``NamespaceMismatch`` on rejection;
* frames are a little-endian u32 length followed by the payload, capped at 512 MiB; reads time out
  after 60 s. ``PMETAL_NAMESPACE`` overrides the namespace string.
``in_memory_channel`` is the same interface over queues for same-process stages and tests.
"""
from __future__ import annotations

import hashlib
import hmac
import os
import queue
import socket
import struct
import threading
import time
from typing import List, Optional, Sequence, Tuple

from .errors import ConnectionTimeout, NamespaceMismatch, PeerLost, PeerTimeout, ProtocolError

MAGIC = b"PMETALD1"
MAX_FRAME = 512 * 1024 * 1024
READ_TIMEOUT = 60.0
HANDSHAKE_TIMEOUT = 5.0
NAMESPACE_ENV = "PMETAL_NAMESPACE"


class NetworkNamespace:
    def __init__(self, version: str = "pmetal-b200/0.1", cluster: Optional[str] = None):
        override = os.environ.get(NAMESPACE_ENV)
        self.namespace = override if override else (f"{version}/{cluster}" if cluster else version)
        self.psk = hashlib.sha3_256(self.namespace.encode("utf-8")).digest()


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    buf = bytearray()
    while len(buf) < n:
        try:
            chunk = sock.recv(n - len(buf))
        except socket.timeout as e:
            raise PeerTimeout(f"read timed out after {sock.gettimeout()} s") from e
        if not chunk:
            raise PeerLost("connection closed by peer")
        buf.extend(chunk)
    return bytes(buf)


def client_handshake(sock: socket.socket, psk: bytes) -> None:
    sock.settimeout(HANDSHAKE_TIMEOUT)
    sock.sendall(MAGIC + psk)
    try:
        ack = _recv_exact(sock, 1)
    except PeerTimeout as e:
        raise ProtocolError("namespace handshake ack timed out") from e
    if ack != b"\x01":
        raise NamespaceMismatch("remote side rejected the namespace key")


def server_handshake(sock: socket.socket, psk: bytes) -> None:
    sock.settimeout(HANDSHAKE_TIMEOUT)
    try:
        payload = _recv_exact(sock, 40)
    except PeerTimeout as e:
        raise ProtocolError("namespace handshake read timed out") from e
    ok = payload[:8] == MAGIC and hmac.compare_digest(payload[8:], psk)
    try:
        sock.sendall(b"\x01" if ok else b"\x00")
    except OSError:
        pass
    if not ok:
        raise NamespaceMismatch("peer presented a different namespace key")


class FramedSocket:
    def __init__(self, sock: socket.socket, read_timeout: float = READ_TIMEOUT):
        self.sock = sock
        sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        sock.settimeout(read_timeout)
        self._wlock, self._rlock = threading.Lock(), threading.Lock()

    def send(self, payload: bytes) -> None:
        if len(payload) > MAX_FRAME:
            raise ProtocolError(f"frame of {len(payload)} bytes exceeds the {MAX_FRAME} byte cap")
        with self._wlock:
            try:
                self.sock.sendall(struct.pack("<I", len(payload)) + payload)
            except OSError as e:
                raise PeerLost(f"send failed: {e}") from e

    def recv(self, timeout: Optional[float] = None) -> bytes:
        with self._rlock:
            if timeout is not None:
                self.sock.settimeout(timeout)
            (n,) = struct.unpack("<I", _recv_exact(self.sock, 4))
            if n > MAX_FRAME:
                raise ProtocolError(f"announced frame of {n} bytes exceeds the cap")
            return _recv_exact(self.sock, n)

    def close(self) -> None:
        try:
            self.sock.close()
        except OSError:
            pass


class QueueEndpoint:
    """One direction of an in-memory channel with the FramedSocket interface."""

    def __init__(self, q: "queue.Queue[bytes]"):
        self.q = q

    def send(self, payload: bytes) -> None:
        self.q.put(bytes(payload))

    def recv(self, timeout: Optional[float] = READ_TIMEOUT) -> bytes:
        try:
            return self.q.get(timeout=timeout)
        except queue.Empty as e:
            raise PeerTimeout(f"no message within {timeout} s") from e

    def close(self) -> None:
        pass


def in_memory_channel() -> Tuple[QueueEndpoint, QueueEndpoint]:
    q: "queue.Queue[bytes]" = queue.Queue()
    return QueueEndpoint(q), QueueEndpoint(q)


def connect_with_fallback(addresses: Sequence[Tuple[str, int]], psk: bytes, max_retries: int = 50,
                          connect_timeout: float = 2.0) -> FramedSocket:
    """Dial the first reachable address; retry the whole list with exponential backoff."""
    delay, last = 0.1, None
    for _ in range(max_retries):
        for host, port in addresses:
            try:
                s = socket.create_connection((host, port), timeout=connect_timeout)
            except OSError as e:
                last = e
                continue
            try:
                client_handshake(s, psk)
            except NamespaceMismatch:
                s.close()
                raise
            except Exception as e:  # try the next address
                s.close()
                last = e
                continue
            return FramedSocket(s)
        time.sleep(delay)
        delay = min(delay * 2, 5.0)
    raise ConnectionTimeout(f"could not reach any of {list(addresses)}: {last}")


class TcpRingTransport:
    """Rank r listens on ``nodes[r]`` and dials rank (r+1) % N; ``send`` goes to next, ``recv`` comes from prev."""

    def __init__(self, nodes: Sequence[Sequence[Tuple[str, int]]], rank: int, namespace: Optional[NetworkNamespace] = None,
                 max_retries: int = 50, accept_timeout: float = 60.0):
        self.rank, self.world = rank, len(nodes)
        self.ns = namespace or NetworkNamespace()
        host, port = nodes[rank][0]
        self._listener = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self._listener.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self._listener.bind(("0.0.0.0" if host not in ("127.0.0.1", "localhost") else host, port))
        self._listener.listen(4)
        self._listener.settimeout(accept_timeout)
        self.prev: Optional[FramedSocket] = None
        err: List[BaseException] = []

        def accept():
            deadline = time.time() + accept_timeout
            while time.time() < deadline:
                try:
                    conn, _ = self._listener.accept()
                except socket.timeout:
                    break
                try:
                    server_handshake(conn, self.ns.psk)
                except NamespaceMismatch as e:
                    conn.close()
                    err.append(e)
                    return
                except Exception:
                    conn.close()
                    continue
                self.prev = FramedSocket(conn)
                return
            err.append(ConnectionTimeout("previous rank never connected"))

        t = threading.Thread(target=accept, daemon=True)
        t.start()
        self.next = connect_with_fallback(nodes[(rank + 1) % self.world], self.ns.psk, max_retries)
        t.join()
        if err:
            self.close()
            raise err[0]

    def send(self, payload: bytes) -> None:
        self.next.send(payload)

    def recv(self, timeout: Optional[float] = None) -> bytes:
        return self.prev.recv(timeout)

    def close(self) -> None:
        for s in (self.prev, getattr(self, "next", None)):
            if s is not None:
                s.close()
        self._listener.close()
