import torch

from pmetal_b200.data.dataloader import DataLoader, PackedDataLoader, synthetic_documents
from pmetal_b200.data.packing import (PackerConfig, PackingStats, Sample, SequencePacker, collate_packs,
                                      compute_pack_seq_len)
from pmetal_b200.ops.reference import seq_starts_from_cu


def _s(n, base=0):
    ids = list(range(base, base + n))
    return Sample(ids, list(ids))


def test_ffd_matches_linear_first_fit():
    import random
    rng = random.Random(0)
    samples = [_s(rng.randint(1, 100), i * 1000) for i in range(300)]
    packs = SequencePacker(PackerConfig(max_length=128)).pack(samples)
    # plain O(n^2) first-fit decreasing
    order = sorted(range(len(samples)), key=lambda i: -len(samples[i]))
    bins = []
    for i in order:
        n = len(samples[i])
        for b in bins:
            if sum(len(x) for x in b) + n <= 128:
                b.append(samples[i])
                break
        else:
            bins.append([samples[i]])
    assert [p.seq_lengths for p in packs] == [[len(x) for x in b] for b in bins]
    assert all(p.total_tokens() <= 128 for p in packs)
    assert sum(p.num_sequences for p in packs) == 300


def test_pack_fields_and_boundary_mask():
    packs = SequencePacker(PackerConfig(max_length=16, algorithm="greedy")).pack([_s(5), _s(6, 100), _s(7, 200)])
    assert len(packs) == 2
    p = packs[0]
    assert p.cu_seqlens == [0, 5, 11] and p.position_ids == list(range(5)) + list(range(6))
    assert p.labels[5] == -100 and p.labels[0] == 0 and p.labels[6] == 101
    m = p.dense_mask()
    assert m[6, 5] == 0 and m[6, 4] == float("-inf") and m[4, 5] == float("-inf")
    st = PackingStats.from_batches(packs, 16)
    assert st.num_sequences == 3 and abs(st.efficiency - 18 / 32) < 1e-9


def test_collate_fixed_shape():
    packs = SequencePacker(PackerConfig(max_length=32)).pack([_s(20), _s(10, 50), _s(25, 100)])
    t = collate_packs(packs, 32)
    assert t.input_ids.shape == (64,) and t.total_tokens == 55
    cu = t.cu_seqlens
    ss = seq_starts_from_cu(cu, 64)
    assert torch.equal(ss, t.seq_start)
    assert t.labels[32].item() == -100          # first token of the second pack
    assert (t.labels[25:32] == -100).all() and (t.labels[62:] == -100).all()


def test_pack_seq_len_rule():
    assert compute_pack_seq_len(list(range(50, 400)), 8192) == 512
    assert compute_pack_seq_len([], 4096) == 4096
    assert compute_pack_seq_len([5000] * 10, 4096) == 4096


def test_dataloader_rank_sharding():
    samples = [_s(3, i * 10) for i in range(10)]
    a = DataLoader(samples, 2, shuffle=True, seed=1, rank=0, world_size=2)
    b = DataLoader(samples, 2, shuffle=True, seed=1, rank=1, world_size=2)
    ia, ib = a._indices(), b._indices()
    assert sorted(ia + ib) == list(range(10)) and not set(ia) & set(ib)
    batch = next(iter(DataLoader([_s(3), _s(5)], 2, shuffle=False, pad_token_id=9)))
    assert batch["input_ids"][0].tolist() == [0, 1, 2, 9, 9] and batch["labels"][0, 3:].tolist() == [-100, -100]


def test_packed_loader():
    docs = synthetic_documents(50, 16, 200, 1000, seed=0)
    dl = PackedDataLoader(docs, 256, packs_per_batch=2, shuffle=False)
    b = next(iter(dl))
    assert b.input_ids.shape == (512,) and dl.stats.efficiency > 0.8
