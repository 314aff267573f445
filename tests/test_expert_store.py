"""Experts served from a packed directory: reads, device pool, prefetch, and the model-level switch."""
import json
import os

import pytest
import torch

from pmetal_b200.cli.commands import pack_experts, read_packed_expert
from pmetal_b200.models.config import preset
from pmetal_b200.models.decoder import DecoderLM
from pmetal_b200.models.expert_store import LayerExperts, PackedExpertStore, enable_expert_offloading
from pmetal_b200.models.moe import SparseMoeBlock


def _moe_model(seed=0):
    torch.manual_seed(seed)
    args = preset("tiny-qwen3-moe")
    return DecoderLM(args).init_weights(0.05, seed).float(), args


def _pack(model, out_dir, bits=4):
    sd = {k: v.detach() for k, v in model.hf_state_dict(merged=True).items()}
    return pack_experts(sd, str(out_dir), bits, 32 if model.cfg.hidden_size % 64 else 64)


def test_store_reads_the_records_the_packer_wrote(tmp_path):
    model, args = _moe_model()
    lay = _pack(model, tmp_path)
    store = PackedExpertStore(str(tmp_path), threads=3)
    try:
        layer = lay["moe_layer_indices"][0]
        gu, dn = store.fetch(layer, [2, 0], "cpu", torch.float32)
        for row, e in enumerate((2, 0)):
            ref = read_packed_expert(str(tmp_path), layer, e)
            assert torch.equal(gu[row], torch.cat([ref["gate"], ref["up"]], 0))
            assert torch.equal(dn[row], ref["down"])
        assert store.stats["reads"] == 2 and store.stats["bytes"] == 2 * store.expert_size
        store.fetch(layer, [2, 0], "cpu", torch.float32)                   # host cache: no further reads
        assert store.stats["reads"] == 2
        with pytest.raises(IndexError):
            store.fetch(layer, [args.num_experts], "cpu")
    finally:
        store.close()


def test_prefetch_counts_hits_and_misses(tmp_path):
    model, _ = _moe_model()
    lay = _pack(model, tmp_path)
    store = PackedExpertStore(str(tmp_path), threads=2)
    try:
        layer = lay["moe_layer_indices"][-1]
        assert store.prefetch(layer, [1, 3]) == 2
        assert store.prefetch(layer, [1]) == 0                             # already on its way or there
        store.raw(layer, [1, 3, 2])
        assert (store.stats["prefetch_hits"], store.stats["prefetch_misses"]) == (2, 1)
        assert store.hit_rate() == pytest.approx(2 / 3)
        store.raw(layer, [1])                                               # plain cache reuse is neither
        assert (store.stats["prefetch_hits"], store.stats["prefetch_misses"]) == (2, 1)
    finally:
        store.close()


def test_host_cache_is_bounded_and_a_call_keeps_its_own_records(tmp_path):
    model, args = _moe_model()
    lay = _pack(model, tmp_path)
    store = PackedExpertStore(str(tmp_path), threads=2)
    store.host_cache_bytes = 2 * store.expert_size
    try:
        bufs = store.raw(lay["moe_layer_indices"][0], list(range(args.num_experts)))
        assert len(bufs) == args.num_experts and len(store._host) <= 2
    finally:
        store.close()


def test_device_pool_replaces_the_least_recently_used(tmp_path):
    model, _ = _moe_model()
    lay = _pack(model, tmp_path)
    store = PackedExpertStore(str(tmp_path))
    try:
        pool = LayerExperts(store, lay["moe_layer_indices"][0], slots=2)
        a = pool.slots_for([0, 1], "cpu", torch.float32)
        assert sorted(a.values()) == [0, 1] and pool.loads == 2
        b = pool.slots_for([1, 2], "cpu", torch.float32)                   # 0 is the oldest: its slot goes to 2
        assert b[1] == a[1] and b[2] == a[0] and pool.loads == 3 and pool.reuses == 1
        ref = read_packed_expert(str(tmp_path), pool.layer, 2)
        assert torch.equal(pool.down[b[2]], ref["down"])
        c = pool.slots_for([0, 1, 3], "cpu", torch.float32)                # more experts than slots: the pool grows
        assert pool.slots == 3 and len(set(c.values())) == 3
    finally:
        store.close()


def test_offloaded_model_matches_the_model_with_dequantised_experts(tmp_path):
    model, args = _moe_model()
    lay = _pack(model, tmp_path)
    # the comparison model carries exactly what the packed files hold
    for i in lay["moe_layer_indices"]:
        blk = model.layers[i].mlp
        assert isinstance(blk, SparseMoeBlock)
        with torch.no_grad():
            for e in range(args.num_experts):
                ref = read_packed_expert(str(tmp_path), i, e)
                blk.gate_up[e].copy_(torch.cat([ref["gate"], ref["up"]], 0))
                blk.down[e].copy_(ref["down"])
    ids = torch.randint(0, args.vocab_size, (12,))
    pos = torch.arange(12, dtype=torch.int32)
    cu = torch.tensor([0, 12], dtype=torch.int32)
    model.eval()
    with torch.no_grad():
        want = model(ids, pos, cu, 12)
    store = enable_expert_offloading(model, str(tmp_path), slots=3)
    try:
        assert all(model.layers[i].mlp.gate_up.numel() == 0 for i in lay["moe_layer_indices"])
        assert len(list(model.parameters())) == len({id(p) for p in model.parameters()})
        with torch.no_grad():
            got = model(ids, pos, cu, 12)
            again = model(ids, pos, cu, 12)
        assert torch.allclose(got, want, atol=1e-5, rtol=1e-5)
        assert torch.equal(got, again)
        if len(lay["moe_layer_indices"]) > 1:
            assert store.stats["prefetch_issued"] > 0 and store.stats["prefetch_hits"] > 0
        with pytest.raises(RuntimeError):
            model.layers[lay["moe_layer_indices"][0]].mlp.hf_state_dict()
    finally:
        store.close()


def test_mismatched_directory_is_refused(tmp_path):
    model, args = _moe_model()
    _pack(model, tmp_path)
    lay = json.load(open(tmp_path / "layout.json"))
    lay["num_experts"] += 1
    json.dump(lay, open(tmp_path / "layout.json", "w"))
    with pytest.raises(ValueError):
        enable_expert_offloading(model, str(tmp_path))


def test_infer_command_with_an_experts_directory(tmp_path, capsys):
    from pmetal_b200.cli.main import main
    from pmetal_b200.models.loader import load_pretrained, save_pretrained
    model, args = _moe_model()
    mdir, pdir = str(tmp_path / "m"), str(tmp_path / "packed")
    save_pretrained(model, mdir)
    assert main(["pack-experts", "-m", mdir, "-o", pdir, "--group-size", "32"]) == 0
    capsys.readouterr()
    m2, _, _ = load_pretrained(mdir, dtype=torch.float32, device="cpu", experts_dir=pdir)
    try:
        assert m2.expert_store is not None and m2.layers[0].mlp.gate_up.numel() == 0
    finally:
        m2.expert_store.close()
    assert main(["infer", "-m", mdir, "-p", "hello", "--max-tokens", "4", "--greedy", "--experts-dir", pdir, "--device", "cpu",
                 "--json", "--ane", "--minimal"]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out.get("completion_tokens", out.get("tokens", 4)) is not None


def test_workload_bench_reports_expert_io(tmp_path, capsys):
    from pmetal_b200.cli.main import main
    from pmetal_b200.models.loader import save_pretrained
    model, _ = _moe_model()
    mdir, pdir = str(tmp_path / "m"), str(tmp_path / "packed")
    save_pretrained(model, mdir)
    _pack(model, pdir)
    capsys.readouterr()
    assert main(["bench-gen", "-m", mdir, "--experts-dir", pdir, "--device", "cpu"]) == 0
    doc = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert doc["expert_io"]["reads"] > 0 and 0.0 <= doc["expert_io"]["prefetch_hit_rate"] <= 1.0
