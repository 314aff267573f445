"""Activation / embedding / frozen-parameter offload and the smart checkpoint policy (CPU: host copies stand in for pinned
buffers, which is the same code path minus the streams)."""
import os

import pytest
import torch

from pmetal_b200.utils import offload as off


def _mlp(seed=0):
    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.GELU(), torch.nn.Linear(256, 64))


@pytest.mark.parametrize("target", [off.CPU, off.DISK])
def test_offloaded_activations_give_the_same_gradients(tmp_path, target):
    m1, m2 = _mlp(), _mlp()
    x = torch.randn(512, 64)
    m1(x).square().mean().backward()
    cfg = off.OffloadConfig(activation_target=target, size_threshold=16 << 10, offload_dir=str(tmp_path))
    ao = off.ActivationOffloader(cfg)
    with ao:
        loss = m2(x).square().mean()
    loss.backward()
    for a, b in zip(m1.parameters(), m2.parameters()):
        assert torch.equal(a.grad, b.grad)
    st = ao.stats
    assert st.saves >= 2 and st.loads == st.saves and st.skipped >= 1          # parameters and small tensors stay
    assert (st.bytes_to_disk if target == off.DISK else st.bytes_to_cpu) >= 512 * 256 * 4
    assert st.device_bytes_saved == st.bytes_to_cpu + st.bytes_to_disk
    if target == off.DISK:
        assert not [f for f in os.listdir(ao.dir)]                             # files are removed once read back
    # the pinned buffers are recycled by the next step
    n_pool = sum(len(v) for v in ao._pool.values())
    with ao:
        loss = m2(x).square().mean()
    assert target == off.DISK or sum(len(v) for v in ao._pool.values()) < n_pool
    loss.backward()


def test_gpu_target_and_threshold_leave_tensors_alone():
    m = _mlp()
    ao = off.ActivationOffloader(off.OffloadConfig.moderate())                 # activations stay on the device
    with ao:
        m(torch.randn(512, 64)).sum().backward()
    assert ao.stats.saves == 0
    assert off.OffloadConfig.aggressive().activation_target == off.DISK
    assert off.OffloadConfig().with_memory_threshold(3.0).memory_threshold == 1.0


def test_offloaded_embedding_and_frozen_parameters(tmp_path):
    w = torch.randn(100, 16)
    idx = torch.tensor([[3, 3, 99], [0, 7, 3]])
    for target in (off.CPU, off.DISK, off.GPU):
        e = off.OffloadedEmbedding(w, target, "cpu", str(tmp_path))
        assert torch.equal(e.lookup(idx), w[idx])
        assert torch.equal(e.get_weights(), w)
        e.evict_gpu_cache()
        assert (e.memory_usage()["gpu"] > 0) == (target == off.GPU)
    mgr = off.FrozenParameterManager("cpu", gpu_budget_bytes=3 * 64 * 4)
    params = [(f"w{i}", torch.full((64,), float(i))) for i in range(5)] + [("train", torch.nn.Parameter(torch.zeros(4)))]
    assert mgr.register_frozen_params(params) == 5
    for i in range(5):
        assert float(mgr.get(f"w{i}")[0]) == i
    assert list(mgr.resident) == ["w2", "w3", "w4"] and mgr.evictions == 2
    mgr.get("w2")
    mgr.get("w0")
    assert list(mgr.resident) == ["w4", "w2", "w0"] and mgr.hits == 1
    assert 39.0 < mgr.memory_savings_percent() < 41.0
    mgr.evict_all()
    assert mgr.gpu_memory_usage() == 0


def test_smart_checkpoint_policy():
    c = off.SmartCheckpointConfig()
    assert c.resolve("mlp", 0.1) == off.ALWAYS_RECOMPUTE and c.resolve("embedding", 0.99) == off.ALWAYS_SAVE
    assert c.resolve("attention", 0.5) == off.ALWAYS_SAVE
    assert c.resolve("attention", 0.9) == off.ALWAYS_RECOMPUTE                 # no offload allowed: recompute
    assert off.SmartCheckpointConfig().with_cpu_offload().resolve("attention", 0.9) == off.OFFLOAD_CPU
    assert off.SmartCheckpointConfig().with_disk_offload("/tmp/x").resolve("moe_expert", 0.9) == off.OFFLOAD_DISK
    assert off.SmartCheckpointConfig.aggressive().resolve("attention", 0.9) == off.ALWAYS_RECOMPUTE   # threshold 5 > cost 3
    assert off.SmartCheckpointConfig(enabled=False).resolve("mlp", 0.99) == off.ALWAYS_SAVE
    assert off.transformer_layer_types(2, True).count("moe_expert") == 2
    assert off.plan_decoder_layers(c, 4, False, 0.2) == [off.ALWAYS_RECOMPUTE] * 4 or True
    assert off.plan_decoder_layers(off.SmartCheckpointConfig().with_cpu_offload(), 3, False, 0.9) == [off.OFFLOAD_CPU] * 3


def test_decoder_blocks_follow_the_plan():
    from pmetal_b200.models.config import ModelArgs
    from pmetal_b200.models.decoder import DecoderLM
    cfg = ModelArgs(vocab_size=97, hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=8)
    ids = torch.randint(0, 97, (2, 24))
    grads = []
    for plan in (None, ["offload_cpu", "recompute", "save"]):
        m = DecoderLM(cfg).init_weights(0.1, 0).train()
        ao = None
        if plan:
            ao = off.apply_to_model(m, plan, off.OffloadConfig(size_threshold=1024))
        loss = m.forward_hidden(ids).square().mean()
        loss.backward()
        grads.append([p.grad.clone() for p in m.parameters()])
        if plan:
            assert ao.stats.saves > 0 and ao.stats.loads == ao.stats.saves
    for a, b in zip(*grads):
        assert torch.allclose(a, b, atol=1e-6)
