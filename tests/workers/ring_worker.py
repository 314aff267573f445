"""Child process of the TCP ring test: builds a real RingBackend over loopback sockets."""
import os
import sys

import numpy as np

from pmetal_b200.parallel.ring import RingBackend
from pmetal_b200.parallel.transport import NetworkNamespace, TcpRingTransport

rank = int(os.environ["PMETAL_TEST_RANK"])
ports = [int(p) for p in os.environ["PMETAL_TEST_PORTS"].split(",")]
nodes = [[("127.0.0.1", p)] for p in ports]
t = TcpRingTransport(nodes, rank, NetworkNamespace("test"), max_retries=20, accept_timeout=30.0)
be = RingBackend(t, rank, len(ports), step_timeout=20.0)
buf = np.array([1.0, 2.0, 3.0] if rank == 0 else [4.0, 5.0, 6.0], dtype=np.float32)
be.barrier()
be.all_reduce(buf, "mean")
be.barrier()
print("RING_OK", buf.tolist(), flush=True)
t.close()
