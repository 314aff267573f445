import os
import socket
import subprocess
import sys
import threading

import numpy as np
import pytest

from pmetal_b200.parallel import plans
from pmetal_b200.parallel.cluster_state import (ElectionManager, HealthMonitor, Metrics, Topology, NodeInfo,
                                                choose_all_reduce, tree_children, tree_parent)
from pmetal_b200.parallel.compression import GradientCompressor, deserialize, serialize
from pmetal_b200.parallel.errors import (ConnectionTimeout, NamespaceMismatch, PeerLost, PeerTimeout, ProtocolError)
from pmetal_b200.parallel.ring import RingBackend, chunk_bounds
from pmetal_b200.parallel.transport import (FramedSocket, NetworkNamespace, client_handshake, connect_with_fallback,
                                            in_memory_channel, server_handshake)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_chunk_partition_covers_buffer():
    for n in (1, 2, 3, 8):
        for length in (0, 1, 7, 64, 1001):
            b = chunk_bounds(length, n)
            assert b[0][0] == 0 and b[-1][1] == length
            assert all(b[i][1] == b[i + 1][0] for i in range(n - 1))
            sizes = [hi - lo for lo, hi in b]
            assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)


class _MemRing:
    """N in-process ranks wired as a ring of queues."""

    def __init__(self, n):
        chans = [in_memory_channel() for _ in range(n)]      # chans[i]: rank i -> rank i+1
        self.t = []
        for r in range(n):
            tx, rx = chans[r][0], chans[(r - 1) % n][1]
            self.t.append(type("T", (), {"send": staticmethod(tx.send), "recv": staticmethod(rx.recv)})())


@pytest.mark.parametrize("world,length", [(2, 3), (3, 10), (4, 1000), (8, 37)])
def test_ring_all_reduce_mean_in_threads(world, length):
    ring = _MemRing(world)
    rng = np.random.default_rng(0)
    data = [rng.standard_normal(length).astype(np.float32) for _ in range(world)]
    expect = np.mean(np.stack(data), axis=0)
    out = [None] * world

    def run(r):
        be = RingBackend(ring.t[r], r, world, step_timeout=10.0)
        buf = data[r].copy()
        be.all_reduce(buf, "mean")
        be.barrier()
        out[r] = buf
    th = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    [t.start() for t in th]
    [t.join(30) for t in th]
    for r in range(world):
        assert np.allclose(out[r], expect, atol=1e-5)


def test_ring_over_tcp_in_child_processes(tmp_path):
    """Two real processes, real sockets: mean of [1,2,3] and [4,5,6] is [2.5,3.5,4.5]."""
    ports = [_free_port(), _free_port()]
    procs = []
    for r in range(2):
        env = dict(os.environ, PMETAL_TEST_RANK=str(r), PMETAL_TEST_PORTS=",".join(map(str, ports)),
                   PYTHONPATH=ROOT)
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "workers", "ring_worker.py")],
                                      env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=60)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert all("RING_OK [2.5, 3.5, 4.5]" in o for o in outs), outs


def test_ring_step_times_out_when_peer_never_sends():
    a_tx, _ = in_memory_channel()
    _, b_rx = in_memory_channel()
    t = type("T", (), {"send": staticmethod(a_tx.send), "recv": staticmethod(b_rx.recv)})()
    be = RingBackend(t, 0, 2, step_timeout=0.2)
    with pytest.raises(PeerTimeout) as e:
        be.all_reduce(np.ones(4, dtype=np.float32))
    assert e.value.is_recoverable() and e.value.is_peer_failure() and not e.value.is_fatal()


def _pair():
    srv = socket.socket()
    srv.bind(("127.0.0.1", 0))
    srv.listen(1)
    port = srv.getsockname()[1]
    return srv, port


def test_psk_handshake_accepts_same_namespace_and_rejects_other(monkeypatch):
    monkeypatch.delenv("PMETAL_NAMESPACE", raising=False)
    good, bad = NetworkNamespace("v1", "c"), NetworkNamespace("v1", "other")
    assert len(good.psk) == 32 and good.psk != bad.psk
    for client_ns, ok in ((good, True), (bad, False)):
        srv, port = _pair()
        res = {}

        def serve():
            conn, _ = srv.accept()
            try:
                server_handshake(conn, good.psk)
                res["srv"] = "ok"
            except NamespaceMismatch as e:
                res["srv"] = e
            conn.close()
        th = threading.Thread(target=serve)
        th.start()
        c = socket.create_connection(("127.0.0.1", port))
        if ok:
            client_handshake(c, client_ns.psk)
        else:
            with pytest.raises(NamespaceMismatch) as e:
                client_handshake(c, client_ns.psk)
            assert e.value.is_fatal()
        th.join(5)
        assert (res["srv"] == "ok") == ok
        c.close(); srv.close()
    monkeypatch.setenv("PMETAL_NAMESPACE", "override")
    assert NetworkNamespace("v1").namespace == "override"


def test_connect_falls_back_to_second_address_and_frames_roundtrip():
    ns = NetworkNamespace("t")
    srv, port = _pair()
    dead = _free_port()
    got = {}

    def serve():
        conn, _ = srv.accept()
        server_handshake(conn, ns.psk)
        fs = FramedSocket(conn)
        got["msg"] = fs.recv()
        fs.send(b"pong")
    th = threading.Thread(target=serve)
    th.start()
    fs = connect_with_fallback([("127.0.0.1", dead), ("127.0.0.1", port)], ns.psk, max_retries=3)
    fs.send(b"ping" * 1000)
    assert fs.recv() == b"pong"
    th.join(5)
    assert got["msg"] == b"ping" * 1000
    with pytest.raises(ConnectionTimeout):
        connect_with_fallback([("127.0.0.1", dead)], ns.psk, max_retries=1)
    # a peer that announces more bytes than it sends, then closes
    srv2, port2 = _pair()

    def short():
        conn, _ = srv2.accept()
        conn.sendall(b"\x10\x00\x00\x00abc")
        conn.close()
    th2 = threading.Thread(target=short)
    th2.start()
    c = FramedSocket(socket.create_connection(("127.0.0.1", port2)))
    with pytest.raises(PeerLost):
        c.recv()
    th2.join(5)
    srv.close(); srv2.close()


def test_compression_codecs_and_wire_format():
    rng = np.random.default_rng(1)
    g = rng.standard_normal(1000).astype(np.float32)
    c = GradientCompressor("topk", 0.05)
    z = c.compress(g)
    idx, val = z.data
    assert idx.size == 50 and np.all(np.diff(idx.astype(np.int64)) > 0)
    assert set(idx) == set(np.argsort(-np.abs(g))[:50])
    d = c.decompress(z)
    assert np.allclose(d + c.error, g)                       # residual carries the unsent part
    z2 = c.compress(np.zeros_like(g))                         # error feedback is re-injected
    assert np.count_nonzero(c.decompress(z2)) == 50
    for strat, tol in (("fp16", 2e-3), ("bf16", 2e-2), ("int8", 0.05)):
        q = GradientCompressor(strat, use_error_feedback=False)
        zz = q.compress(g)
        back = q.decompress(deserialize(serialize(zz)))
        assert np.max(np.abs(back - g)) <= tol * np.abs(g).max() + 1e-6
    ob = GradientCompressor("onebit", use_error_feedback=False)
    zb = ob.compress(g)
    back = ob.decompress(deserialize(serialize(zb)))
    assert np.all(np.sign(back) == np.where(g > 0, 1, -1)) and abs(abs(back[0]) - np.abs(g).mean()) < 1e-5
    r = GradientCompressor("random", 0.1, use_error_feedback=False)
    zr = r.compress(np.ones(5000, dtype=np.float32))
    assert 300 < zr.data[0].size < 700 and np.allclose(zr.data[1], 10.0)
    s = serialize(z)
    assert s[:4] == (1000).to_bytes(4, "little") and s[4] == 1
    for bad in (b"", b"\x01\x00\x00\x00\x09", s[:-3], serialize(zb)[:-1]):
        with pytest.raises(ValueError):
            deserialize(bad)
    full = GradientCompressor("powersgd").compress(g)
    assert full.kind == "full"


def test_plans():
    assert [plans.expert_range(10, r, 4) for r in range(4)] == [(0, 3), (3, 3), (6, 2), (8, 2)]
    assert all(plans.rank_for_expert(e, 10, 4) == next(r for r in range(4)
               if plans.expert_range(10, r, 4)[0] <= e < sum(plans.expert_range(10, r, 4))) for e in range(10))
    assert plans.rank_for_expert(2, 3, 8) == 2
    assert plans.shard_bounds(10, 0, 4) == (0, 3) and plans.shard_bounds(10, 3, 4) == (8, 10)
    tp = plans.build_tp_plan("qwen3_moe", {"num_attention_heads": 32, "num_key_value_heads": 4, "num_experts": 128}, 8)
    assert plans.directive_for(tp, "layers.0.self_attn.q_proj.weight").kind == "all_to_sharded"
    assert plans.directive_for(tp, "layers.0.self_attn.o_proj.weight") == plans.ShardingDirective("sharded_to_all", 1)
    assert plans.directive_for(tp, "layers.0.self_attn.k_proj.weight").kind == "replicated"   # 4 kv heads, 8 ranks
    assert plans.directive_for(tp, "layers.3.mlp.experts.7.down_proj").kind == "expert_sharded"
    assert plans.expert_capacity(1024, 2, 8) == 320
    import torch
    keep = plans.apply_capacity(torch.tensor([[0], [0], [1], [0]]), 2, 2)
    assert keep.flatten().tolist() == [True, True, True, False]
    s = plans.schedule_1f1b(4, 8, 1)
    assert [a for a in s if a[0] == "forward"] == [("forward", i) for i in range(8)]
    assert s[:6] == [("recv_activation", 0), ("forward", 0), ("send_activation", 0), ("recv_activation", 1),
                     ("forward", 1), ("send_activation", 1)] and s[-1] == ("weight_update", None)
    assert abs(plans.bubble_fraction(4, 8) - 3 / 11) < 1e-12
    zb = plans.schedule_zero_bubble(4, 8, 0)
    assert sorted(m for a, m in zb if a == "backward_weight") == list(range(8))
    assert [m for a, m in zb if a == "backward_input"] == list(range(8))
    assert plans.zero_owner_map(["b", "a", "c"], 2) == {"a": 0, "b": 1, "c": 0}
    assert plans.assign_layers_proportional(28, [1, 1, 2]) == [(0, 7), (7, 14), (14, 28)]
    assert plans.assign_layers_bandwidth_aware([1] * 6, [1.0, 2.0], [0.0]) == [(0, 2), (2, 6)]


def test_cluster_state_machines():
    t = [0.0]
    hm = HealthMonitor(clock=lambda: t[0])
    hm.add_peer("a"); hm.add_peer("b")
    t[0] = 10.0; hm.record_heartbeat("a")
    t[0] = 16.0
    assert hm.check() == ["b"] and hm.unhealthy() == ["b"]
    assert not hm.record_failure("a") and not hm.record_failure("a") and hm.record_failure("a")
    assert hm.summary()["unhealthy"] == 2
    hm.record_heartbeat("a"); assert hm.unhealthy() == ["b"]
    c1, c2 = [0.0], [0.0]
    e1, e2 = ElectionManager("p1", 3.0, lambda: c1[0]), ElectionManager("p2", 3.0, lambda: c2[0])
    c1[0], c2[0] = 100.0, 5.0                     # p1 is senior
    m1 = e1.start_election()
    r = e2.handle_message(m1)
    assert r is not None and r.vote_for == "p1"
    e1.handle_message(r)
    c1[0] += 4; c2[0] += 4
    assert e1.tick()["event"] == "elected_master" and e2.tick() == {"event": "new_master", "master": "p1", "session": 1}
    assert e1.report_masters(["p1", "p2"])["event"] == "split_brain"
    assert choose_all_reduce(1000, 8) == "one_shot" and choose_all_reduce(1 << 22, 8) == "two_shot"
    assert choose_all_reduce(1 << 22, 2) == "one_shot"
    assert tree_parent(0) is None and tree_parent(5, 2) == 2 and tree_children(1, 6, 2) == [3, 4]
    topo = Topology([NodeInfo("gpu01", 1), NodeInfo("gpu00", 0)])
    assert topo.ring_order() == ["gpu00", "gpu01"] and topo.ring_next("gpu01") == "gpu00"
    m = Metrics()
    for v in range(100):
        m.observe("all_reduce_ms", float(v))
    m.inc("bytes", 10); m.inc("bytes", 5)
    snap = m.snapshot()
    assert snap["counters"]["bytes"] == 15 and snap["histograms"]["all_reduce_ms"]["p95"] == 95.0


def test_ring_attention_pipeline_and_1f1b_over_gloo():
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for n in (2, 3):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
               "127.0.0.1", "--master-port", str(29720 + n), os.path.join(root, "tests", "workers", "cp_pp_worker.py")]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=120)
        assert r.returncode == 0 and "CP_PP_WORKER_OK" in r.stdout, r.stdout[-3000:]


def test_every_rank_resumes_and_sharded_moments_are_collected(tmp_path):
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29741", os.path.join(root, "tests", "workers", "dp_resume_worker.py")]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=180,
                       env=dict(os.environ, PMETAL_TEST_DIR=str(tmp_path)))
    assert r.returncode == 0 and r.stdout.count("DP_RESUME_WORKER_OK") == 2, r.stdout[-3000:]


def test_tensor_and_expert_parallel_serving_slices_over_gloo():
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29743", os.path.join(root, "tests", "workers", "tp_serve_worker.py")]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=240)
    assert r.returncode == 0 and r.stdout.count("TP_SERVE_WORKER_OK") == 2, r.stdout[-3000:]


def test_sharded_engine_with_follower_ranks_over_gloo():
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29747", os.path.join(root, "tests", "workers", "serve_replica_worker.py")]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=240)
    assert r.returncode == 0 and r.stdout.count("SERVE_REPLICA_WORKER_OK") == 2, r.stdout[-3000:]


def test_pretrain_replicas_stay_identical_over_gloo():
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29751", os.path.join(root, "tests", "workers", "pretrain_dp_worker.py")]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=240,
                       env=dict(os.environ, PMETAL_TEST_CPU="1"))
    assert r.returncode == 0 and r.stdout.count("PRETRAIN_DP_WORKER_OK") == 2, r.stdout[-3000:]


@pytest.mark.parametrize("world", [2, 3])
def test_context_parallel_attention_trains_over_gloo(world):
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29753 + world), os.path.join(root, "tests", "workers", "cp_train_worker.py")]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=240,
                       env=dict(os.environ, PMETAL_TEST_CPU="1"))
    assert r.returncode == 0 and r.stdout.count("CP_TRAIN_WORKER_OK") == world, r.stdout[-3000:]


def test_activation_message_wire_format():
    import struct

    import torch
    from pmetal_b200.parallel.pipeline import ActivationMessage
    t = torch.arange(6, dtype=torch.float32).reshape(1, 2, 3).to(torch.bfloat16)
    raw = ActivationMessage(9, 3, t).serialize()
    assert raw[:16] == struct.pack("<QII", 9, 3, 3) and raw[16:28] == struct.pack("<3I", 1, 2, 3) and raw[28] == 2
    assert len(raw) == 8 + 4 + 4 + 12 + 1 + 12
    back = ActivationMessage.deserialize(raw)
    assert back.nonce == 9 and back.layer_id == 3 and torch.equal(back.tensor, t)
    import pytest
    with pytest.raises(ValueError):
        ActivationMessage.deserialize(raw[:-1])
    with pytest.raises(ValueError):
        ActivationMessage.deserialize(raw[:28] + bytes([9]) + raw[29:])
    with pytest.raises(ValueError):
        ActivationMessage.deserialize(b"short")


def test_identity_fabric_discovery_and_bundle(tmp_path):
    import torch

    from pmetal_b200.parallel import cloud_bridge, discovery
    from pmetal_b200.parallel.pipeline import plan_local_pipeline, run_local_pipeline
    ident = discovery.NodeIdentity.load_or_create(str(tmp_path / "id" / "node_keypair"))
    again = discovery.NodeIdentity.load_or_create(str(tmp_path / "id" / "node_keypair"))
    assert ident.peer_id == again.peer_id and (tmp_path / "id" / "node_keypair").stat().st_mode & 0o777 == 0o600
    sig = ident.sign(b"hello")
    assert discovery.NodeIdentity.verify(ident.public_bytes, sig, b"hello")
    assert not discovery.NodeIdentity.verify(ident.public_bytes, sig, b"hellp")
    fab = discovery.probe_fabric(4, lambda i, j: (i // 2) == (j // 2))      # two NVLink islands joined over PCIe
    assert fab[0][1].name == "nvlink5" and fab[0][2].name == "pcie5" and fab[3][3].name == "self"
    assert discovery.ring_bandwidth(fab, [0, 1, 2, 3]) == 64.0 and discovery.ring_bandwidth(fab, [0, 1]) == 900.0
    assert discovery.link_score(discovery.NVLINK5) < discovery.link_score(discovery.PCIE5) < discovery.link_score(discovery.HOST_TCP)
    peers = [discovery.Peer("b"), discovery.Peer("c"), discovery.Peer("a")]
    assert [p.peer_id for p in discovery.ring_order(peers)] == ["a", "b", "c"]
    prev, nxt = discovery.ring_neighbours(peers, "a")
    assert (prev.peer_id, nxt.peer_id) == ("c", "b")
    (tmp_path / "peers.json").write_text('[{"peer_id": "x", "addresses": ["10.0.0.1:52416"], "device": 1}]')
    p = discovery.load_static_peers(str(tmp_path / "peers.json"))[0]
    assert p.addresses == [("10.0.0.1", 52416)] and p.device == 1
    # run bundle round trip
    torch.manual_seed(3)
    params = {"w": torch.randn(4, 3), "b": torch.randn(3)}
    opt = {"w.m": torch.zeros(4, 3), "w.v": torch.ones(4, 3)}
    meta = cloud_bridge.export_bundle(str(tmp_path / "bundle"), params, opt, step=17, config={"lr": 1e-4}, world_size=8)
    expect = torch.rand(3)
    torch.rand(10)
    p2, o2, m2 = cloud_bridge.import_bundle(str(tmp_path / "bundle"))
    assert torch.equal(torch.rand(3), expect)                                  # the generator state came back
    assert torch.equal(p2["w"], params["w"]) and torch.equal(o2["w.v"], opt["w.v"]) and m2["step"] == 17 == meta["step"]
    assert (tmp_path / "bundle" / "bootstrap_cluster.py").exists() and m2["num_params"] == 15
    # in-process pipeline over queues keeps order and surfaces a stage failure
    assert plan_local_pipeline(10, 3) == [(0, 4), (4, 7), (7, 10)] and plan_local_pipeline(2, 5) == [(0, 1), (1, 2)]
    assert run_local_pipeline([lambda x: x + 1, lambda x: x * 2], range(6)) == [2, 4, 6, 8, 10, 12]

    def boom(x):
        raise RuntimeError("stage failed")
    import pytest
    with pytest.raises(RuntimeError):
        run_local_pipeline([lambda x: x, boom], range(3))


def test_stream_multiplexer_routes_by_nonce():
    import queue
    import threading

    import torch

    from pmetal_b200.parallel.pipeline import ActivationMessage, StreamMultiplexer
    mux = StreamMultiplexer(max_pending=3)
    for n in (7, 8, 9):
        mux.register(n)
    with pytest.raises(KeyError):
        mux.register(7)
    with pytest.raises(RuntimeError):
        mux.register(10)
    msgs = [ActivationMessage(nonce=n, layer_id=i, tensor=torch.full((1, 1, 2), float(n))) for i, n in enumerate((9, 7, 8, 7))]
    t = threading.Thread(target=lambda: [mux.dispatch(m) for m in msgs])
    t.start()
    got7 = [mux.wait(7, timeout=5).layer_id for _ in range(2)]
    assert got7 == [1, 3] and mux.wait(8, timeout=5).nonce == 8 and float(mux.wait(9, timeout=5).tensor[0, 0, 0]) == 9.0
    t.join()
    mux.close(8)
    assert not mux.dispatch(msgs[2]) and mux.dropped == 1 and mux.pending() == 2        # late message of a closed request
    with pytest.raises(queue.Empty):
        mux.wait(7, timeout=0.05)


def test_per_architecture_tensor_plans():
    import pytest
    import torch
    from pmetal_b200.parallel import plans as P
    assert P.build_plan("LlamaForCausalLM", {"num_hidden_layers": 2, "num_attention_heads": 8}, 1) == {}
    with pytest.raises(ValueError):
        P.build_plan("LlamaForCausalLM", {"num_hidden_layers": 2, "num_attention_heads": 6}, 4)
    # dense llama: column / row split of attention and feed-forward, norms and embeddings whole
    p = P.build_plan("LlamaForCausalLM", {"num_hidden_layers": 2, "num_attention_heads": 8, "num_key_value_heads": 2}, 2)
    assert p["model.layers.0.self_attn.q_proj.weight"] == P.ShardingDirective("all_to_sharded", 0)
    assert p["model.layers.1.self_attn.o_proj.weight"] == P.ShardingDirective("sharded_to_all", 1)
    assert p["model.layers.1.self_attn.o_proj.bias"].kind == "replicated"
    assert p["model.layers.0.mlp.down_proj.weight"].kind == "sharded_to_all" and p["lm_head.weight"].kind == "replicated"
    assert p["model.layers.0.input_layernorm.weight"].kind == "replicated" and P.num_sharded(p) == 2 * (6 + 1 + 3)
    # deepseek: latent attention, dense prefix, shared experts, stacked routed experts
    cfg = {"num_hidden_layers": 4, "num_attention_heads": 16, "n_routed_experts": 64, "n_shared_experts": 2,
           "first_k_dense_replace": 1, "moe_layer_freq": 1, "q_lora_rank": 1536, "model_type": "deepseek_v3"}
    p = P.build_plan("DeepseekV3ForCausalLM", cfg, 4)
    assert p["model.layers.0.self_attn.q_a_proj.weight"].kind == "replicated"
    assert p["model.layers.0.self_attn.q_b_proj.weight"].kind == "all_to_sharded"
    assert p["model.layers.0.self_attn.kv_a_proj_with_mqa.weight"].kind == "replicated"
    assert p["model.layers.0.self_attn.kv_b_proj.weight"].kind == "all_to_sharded"
    assert "model.layers.0.mlp.gate_proj.weight" in p and "model.layers.0.mlp.switch_mlp.gate_proj.weight" not in p
    assert p["model.layers.1.mlp.switch_mlp.down_proj.weight"] == P.ShardingDirective("expert_sharded", 0, 64)
    assert p["model.layers.1.mlp.shared_experts.up_proj.weight"].kind == "all_to_sharded"
    assert p["model.layers.1.mlp.gate.weight"].kind == "replicated"
    cfg2 = dict(cfg, q_lora_rank=None)
    assert "model.layers.0.self_attn.q_proj.weight" in P.build_plan("DeepseekV2ForCausalLM", cfg2, 4)
    # qwen3-moe with a sparse step of 2: odd layers are sparse
    p = P.build_plan("Qwen3MoeForCausalLM", {"num_hidden_layers": 4, "num_attention_heads": 8, "num_experts": 16,
                                             "decoder_sparse_step": 2}, 2)
    assert "model.layers.0.mlp.gate_proj.weight" in p and "model.layers.1.mlp.switch_mlp.up_proj.weight" in p
    assert p["model.layers.1.mlp.shared_expert_gate.weight"].kind == "replicated"
    # llama-4 interleave, gpt-oss biases
    p = P.build_plan("Llama4ForCausalLM", {"num_hidden_layers": 4, "num_attention_heads": 8, "num_local_experts": 16,
                                           "interleave_moe_layer_step": 2, "model_type": "llama4"}, 2)
    assert p["model.layers.0.feed_forward.experts.gate_proj.weight"].total == 16 and "model.layers.1.mlp.up_proj.weight" in p
    assert p["model.layers.0.feed_forward.shared_expert.down_proj.weight"].kind == "sharded_to_all"
    p = P.build_plan("GptOssForCausalLM", {"num_hidden_layers": 2, "num_attention_heads": 8, "num_local_experts": 32}, 2)
    assert p["model.layers.1.mlp.experts.down_proj.bias"] == P.ShardingDirective("expert_sharded", 0, 32)
    # qwen3-next: layer_types decides between attention and the delta-net mixer; a wrong-length list falls back to
    # the attention interval
    cfg = {"num_hidden_layers": 4, "num_attention_heads": 8, "num_experts": 8, "gdn_heads": 4,
           "layer_types": ["linear_attention", "linear_attention", "linear_attention", "full_attention"]}
    p = P.build_plan("Qwen3NextForCausalLM", cfg, 2)
    assert p["model.layers.0.linear_attn.in_proj_qkv.weight"].kind == "all_to_sharded"
    assert p["model.layers.0.linear_attn.A_log"].kind == "all_to_sharded" and p["model.layers.0.linear_attn.o_proj.weight"].axis == 1
    assert "model.layers.3.self_attn.q_proj.weight" in p and "model.layers.3.linear_attn.conv1d.weight" not in p
    p = P.build_plan("Qwen3NextForCausalLM", dict(cfg, layer_types=["full_attention"], full_attention_interval=2), 2)
    assert "model.layers.1.self_attn.q_proj.weight" in p and "model.layers.0.linear_attn.dt_bias" in p
    # shards of a stacked expert tensor and of a row-split weight
    w = torch.arange(8 * 3 * 2, dtype=torch.float32).reshape(8, 3, 2)
    assert P.shard_weight(w, P.ShardingDirective("expert_sharded", 0, 8), 1, 4).shape == (2, 3, 2)
    m = torch.arange(12.0).reshape(3, 4)
    assert torch.equal(P.shard_weight(m, P.ShardingDirective("sharded_to_all", 1), 1, 2), m[:, 2:])


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_training_matches_the_unsharded_model_over_gloo(world):
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29760 + world), os.path.join(root, "tests", "workers", "ep_train_worker.py")]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300,
                       env=dict(os.environ, PMETAL_TEST_CPU="1"))
    assert r.returncode == 0 and r.stdout.count("EP_TRAIN_WORKER_OK") == world, r.stdout[-3000:]
