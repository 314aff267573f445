"""Native packing / collation / checkpoint reads / KV block pool against their Python counterparts."""
import numpy as np
import pytest
import torch

from pmetal_b200.data.dataloader import PackedDataLoader, synthetic_documents
from pmetal_b200.data.fastpack import FastPackedLoader, TokenStore, pack_lengths
from pmetal_b200.data.packing import PackerConfig, Sample, SequencePacker


def _fields(t):
    return (t.input_ids, t.labels, t.position_ids, t.cu_seqlens, t.seq_start)


@pytest.mark.parametrize("algorithm", ["ffd", "greedy"])
def test_native_loader_equals_python_loader(algorithm):
    docs = synthetic_documents(300, 1, 700, 1000, seed=3)
    docs[5] = Sample(list(range(900)), list(range(900)))            # longer than a pack: truncated to pack_len
    for s in docs[:40]:
        s.labels = [-100 if i % 3 == 0 else t for i, t in enumerate(s.labels)]
    ref = PackedDataLoader(docs, 512, packs_per_batch=3, shuffle=True, seed=7, rank=1, world_size=2, pad_token_id=9,
                           algorithm=algorithm)
    fast = FastPackedLoader(TokenStore.from_samples(docs), 512, packs_per_batch=3, shuffle=True, seed=7, rank=1,
                            world_size=2, pad_token_id=9, algorithm=algorithm, threads=3, pin=False)
    assert len(ref) == len(fast) and ref.stats == fast.stats
    n = 0
    for a, b in zip(ref, fast):
        for x, y in zip(_fields(a), _fields(b)):
            assert x.dtype == y.dtype and torch.equal(x, y)
        assert (a.total_tokens, a.num_sequences, a.max_seqlen) == (b.total_tokens, b.num_sequences, b.max_seqlen)
        n += 1
    assert n == len(ref) and n > 3


def test_pack_lengths_matches_python_bins_and_drops_short_documents():
    rng = np.random.default_rng(0)
    lens = rng.integers(1, 300, size=2000)
    bins, n = pack_lengths(lens, 512, "ffd", min_length=4)
    assert (bins[lens < 4] == -1).all() and (bins[lens >= 4] >= 0).all()
    load = np.bincount(bins[bins >= 0], weights=lens[bins >= 0], minlength=n)
    assert load.max() <= 512 and n == len(load)
    samples = [Sample(list(range(int(k)))) for k in lens]
    py = SequencePacker(PackerConfig(max_length=512, min_length=4)).pack(samples)
    assert len(py) == n
    assert sorted(p.total_tokens() for p in py) == sorted(int(x) for x in load)


def test_parallel_checkpoint_read(tmp_path):
    from pmetal_b200.utils.safetensors_io import load_file, load_file_parallel, save_file
    g = torch.Generator().manual_seed(0)
    tensors = {"a": torch.randn(300, 70, generator=g), "b": torch.randn(5, generator=g).to(torch.bfloat16),
               "c": torch.randint(0, 100, (33,), generator=g), "empty": torch.zeros(0, 4), "s": torch.tensor(3.5)}
    path = str(tmp_path / "m.safetensors")
    save_file(tensors, path)
    a, b = load_file(path), load_file_parallel(path, threads=3)
    assert set(a) == set(b) == set(tensors)
    for k in tensors:
        assert b[k].dtype == tensors[k].dtype and b[k].shape == tensors[k].shape and torch.equal(a[k], b[k])
    only = load_file_parallel(path, names=["c"])
    assert list(only) == ["c"] and torch.equal(only["c"], tensors["c"])
    with open(path, "r+b") as fh:                                   # a truncated file is an error, not garbage
        fh.truncate(200)
    with pytest.raises((ValueError, OSError)):
        load_file_parallel(path)


def test_block_pool_fork_copy_on_write_and_tables():
    from pmetal_b200.models.block_pool import BlockPool
    pool = BlockPool(num_blocks=8, block_size=4)
    pool.add(1)
    slots, copies = pool.reserve(1, 6)
    assert slots == [0, 1, 2, 3, 4, 5] and copies == [] and pool.num_free == 6 and pool.length(1) == 6
    pool.fork(1, 2)                                                # shares blocks 0 and 1
    assert pool.num_free == 6 and pool.ref(0) == 2 and pool.ref(1) == 2
    assert pool.blocks_needed(2, 1) == 1                           # the shared tail block must be copied first
    slots, copies = pool.reserve(2, 3)                             # copy-on-write of the tail, then one more block
    assert copies == [(1, 2)] and slots == [2 * 4 + 2, 2 * 4 + 3, 3 * 4 + 0]
    assert pool.ref(1) == 1 and pool.ref(2) == 1 and pool.num_free == 4
    table, lens = pool.tables([1, 2], max_blocks=4)
    assert table.tolist() == [[0, 1, 0, 0], [0, 2, 3, 0]] and lens.tolist() == [6, 9]
    pool.truncate(2, 4)
    assert pool.num_free == 6 and pool.length(2) == 4
    with pytest.raises(MemoryError):
        pool.reserve(1, 100)
    assert pool.length(1) == 6 and pool.num_free == 6              # a refused reservation changes nothing
    pool.free(1)
    assert pool.ref(0) == 1 and pool.num_free == 7
    pool.free(2)
    assert pool.num_free == 8
    with pytest.raises(KeyError):
        pool.length(2)


def test_block_pool_tracks_the_paged_cache_allocator_under_random_operations():
    """The native pool and the Python allocator inside PagedKVCache hand out the same blocks for the same requests."""
    import random
    from pmetal_b200.models.block_pool import BlockPool
    from pmetal_b200.models.kv_cache import BLOCK, PagedKVCache
    cache = PagedKVCache(1, 1, 8, num_blocks=24, dtype=torch.float32, device="cpu")
    pool = BlockPool(24, BLOCK)
    rnd = random.Random(0)
    live, next_id = [], 0
    for _ in range(400):
        op = rnd.choice(["add", "append", "append", "append", "fork", "truncate", "free"])
        if op == "add" or not live:
            cache.add_sequence(next_id); pool.add(next_id); live.append(next_id); next_id += 1
        elif op == "append":
            s, n = rnd.choice(live), rnd.randint(1, 90)
            if pool.blocks_needed(s, n) > pool.num_free:
                with pytest.raises(MemoryError):
                    pool.reserve(s, n)
                continue
            assert cache.reserve(s, n) == pool.reserve(s, n)[0]
        elif op == "fork":
            s = rnd.choice(live)
            cache.fork(s, next_id); pool.fork(s, next_id); live.append(next_id); next_id += 1
        elif op == "truncate":
            s = rnd.choice(live)
            n = rnd.randint(0, cache.length(s))
            cache.truncate(s, n); pool.truncate(s, n)
        else:
            s = live.pop(rnd.randrange(len(live)))
            cache.free_sequence(s); pool.free(s)
        assert cache.num_free() == pool.num_free
        for s in live:
            assert cache.length(s) == pool.length(s)
    table, lens = pool.tables(live, max_blocks=24)
    for i, s in enumerate(live):
        bl = cache.seqs[s].blocks
        assert table[i, :len(bl)].tolist() == bl and lens[i] == cache.length(s)
