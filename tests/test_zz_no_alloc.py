"""The allocation-free split-KV paged attention entry point (``pm_paged_attn_static``) against ``pm_paged_attn``.

Collected last on purpose (file name), so that it also runs after every other GPU test has used the library."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(hq, hkv, lens, qlens):
    from pmetal_b200.models.kv_cache import PagedKVCache
    from pmetal_b200.ops import native as nat
    if not nat.available():
        pytest.fail(f"native library missing: {nat.load_error()}")
    g = torch.Generator(device="cuda").manual_seed(5)
    d = 128
    cache = PagedKVCache(1, hkv, d, 256, torch.bfloat16, "cuda")
    for i, (L, n) in enumerate(zip(lens, qlens)):
        cache.add_sequence(i)
        if L - n > 0:
            slots = torch.tensor(cache.reserve(i, L - n), device="cuda")
            k = torch.randn(L - n, hkv, d, device="cuda", generator=g).to(torch.bfloat16)
            v = torch.randn(L - n, hkv, d, device="cuda", generator=g).to(torch.bfloat16)
            nat.kv_append(k, v, cache.k[0], cache.v[0], slots)
    meta = cache.prepare(list(range(len(lens))), qlens)
    kn = torch.randn(meta.total_q, hkv, d, device="cuda", generator=g).to(torch.bfloat16)
    vn = torch.randn(meta.total_q, hkv, d, device="cuda", generator=g).to(torch.bfloat16)
    nat.kv_append(kn, vn, cache.k[0], cache.v[0], meta.slots)
    q = torch.randn(meta.total_q, hq, d, device="cuda", generator=g).to(torch.bfloat16)
    return nat, cache, meta, q


def _call_static(nat, cache, meta, q, n_split, window=0):
    L = nat.lib()
    fn = L.pm_paged_attn_static
    fn.restype = ctypes.c_int
    out = torch.empty_like(q)
    vp = lambda t: ctypes.c_void_p(t.data_ptr())      # noqa: E731
    rc = fn(vp(q), vp(cache.k[0]), vp(cache.v[0]), vp(out), vp(meta.block_table), vp(meta.seq_lens), vp(meta.q_start),
            vp(meta.q_lens), ctypes.c_int(meta.block_table.shape[0]), ctypes.c_int(meta.block_table.shape[1]),
            ctypes.c_int(q.shape[0]), ctypes.c_int(meta.max_q), ctypes.c_int(q.shape[1]),
            ctypes.c_int(cache.k[0].shape[2]), ctypes.c_int(n_split), ctypes.c_float(128 ** -0.5), ctypes.c_int(window),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


def test_static_scratch_matches_caller_scratch_twice():
    nat, cache, meta, q = _setup(4, 2, [700, 65, 1300], [1, 3, 2])
    scale = 128 ** -0.5
    for n_split, qq in ((3, q), (5, (q.float() * 0.5).to(torch.bfloat16))):       # two calls in a row, new inputs
        want = nat.paged_attn(qq, cache.k[0], cache.v[0], meta, scale, 0, n_split=n_split)
        free_before = torch.cuda.mem_get_info()[0]
        rc, got = _call_static(nat, cache, meta, qq, n_split)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.cuda.mem_get_info()[0] == free_before        # nothing was taken from the device
        assert torch.equal(got, want)
    one = nat.paged_attn(q, cache.k[0], cache.v[0], meta, scale, 0, n_split=1)
    rc, got = _call_static(nat, cache, meta, q, 4)
    assert rc == 0
    torch.testing.assert_close(got.float(), one.float(), atol=2e-2, rtol=2e-2)
    nat.check_status()


def test_static_scratch_rejects_oversize():
    nat, cache, meta, q = _setup(4, 2, [200], [2])
    L = nat.lib()
    L.pm_paged_attn_static_max_rows.restype = ctypes.c_int
    L.pm_paged_attn_static_strerror.restype = ctypes.c_char_p
    max_rows = L.pm_paged_attn_static_max_rows()
    assert max_rows == 4096
    too_many = max_rows // (q.shape[0] * q.shape[1]) + 1
    rc, _ = _call_static(nat, cache, meta, q, too_many)
    assert rc == -3
    assert b"exceeds" in L.pm_paged_attn_static_strerror(ctypes.c_int(rc))
    rc, _ = _call_static(nat, cache, meta, q, 0)
    assert rc == -2
    torch.cuda.synchronize()
