"""Numerics of every CUDA kernel against the fp32 PyTorch statement of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _nat():
    from pmetal_b200.ops import native
    if not native.available():
        pytest.fail(f"native library not loaded: {native.load_error()}")
    return native


def _close(a, b, rtol=2e-2, atol=2e-2, what=""):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    ref = b.abs().max().item()
    assert err <= atol + rtol * ref, f"{what}: max err {err} vs ref max {ref}"


def _rand(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device="cuda") * scale).to(dtype)


@pytest.mark.parametrize("M,N,K,bn", [(256, 256, 512, 128), (384, 512, 1024, 256), (200, 192, 320, 64),
                                      (1000, 96, 136, 32), (128, 128, 64, 128), (4096, 4096, 1024, 256)])
def test_gemm_kmajor(M, N, K, bn):
    nat = _nat()
    torch.manual_seed(0)
    x, w = _rand(M, K), _rand(N, K, scale=K ** -0.5)
    y = nat.gemm(x, w, bn=bn)
    nat.check_status()
    _close(y, x.float() @ w.float().t(), what="gemm")


@pytest.mark.parametrize("M,N,K", [(64, 768, 2048), (17, 2048, 512), (128, 96, 1000), (100, 2560, 2048), (33, 40, 4096)])
def test_gemm_single_row_block_splits_k_inside_the_kernel(M, N, K, monkeypatch):
    """At most 128 rows and few column tiles: the reduction is cut over several CTAs whose partial tiles meet in a
    workspace; the last arrival of each tile adds them in a fixed order. Same result as the unsplit launch up to the
    rounding of the sum order, bit-identical from call to call, residual and scale applied once."""
    nat = _nat()
    torch.manual_seed(2)
    x, w, r = _rand(M, K), _rand(N, K, scale=K ** -0.5), _rand(M, N)
    n0 = nat.LAUNCHES
    ys = [nat.gemm(x, w, alpha=0.5, residual=r) for _ in range(3)]
    assert nat.LAUNCHES - n0 == 3                     # no separate reduction launch
    nat.check_status()
    ref = 0.5 * (x.float() @ w.float().t()) + r.float()
    _close(ys[0], ref, what="split-k gemm")
    assert torch.equal(ys[0], ys[1]) and torch.equal(ys[0], ys[2])
    monkeypatch.setattr(nat, "SPLIT_K", False)
    _close(nat.gemm(x, w, alpha=0.5, residual=r), ys[0], rtol=1e-2, atol=1e-2, what="split vs unsplit")


def test_gemm_tile_width_from_the_tuner(tmp_path, monkeypatch):
    """With the tuner on, the first call of a shape times the candidate tile widths and records the winner; later
    calls read it from the cache file and give the same result."""
    nat = _nat()
    from pmetal_b200.utils import tuna
    monkeypatch.setenv("PMETAL_TUNA_CACHE", str(tmp_path))
    monkeypatch.setattr(tuna, "_GLOBAL", None)
    monkeypatch.setattr(nat, "TUNA", True)
    torch.manual_seed(0)
    x, w = _rand(512, 256), _rand(384, 256, scale=1 / 16)
    y = nat.gemm(x, w)
    nat.check_status()
    _close(y, x.float() @ w.float().t(), what="tuned gemm")
    key = tuna.Tuner.make_key("gemm_bn", 512, 384, 256)
    table = tuna.Tuner(str(tmp_path / "tuna.json")).table
    assert key in table and table[key]["best"] in (32, 64, 128, 256) and len(table[key]["ms"]) >= 3
    n0 = nat.LAUNCHES
    y2 = nat.gemm(x, w)
    assert nat.LAUNCHES - n0 == 1 and torch.equal(y, y2)          # cache hit: one launch, no timing runs


def test_gemm_alpha_residual_pad():
    nat = _nat()
    torch.manual_seed(1)
    x, w, r = _rand(300, 256), _rand(48, 256, scale=1 / 16), _rand(300, 64)
    y = nat.gemm(x, w, alpha=0.5, residual=r, pad_n_to=64, bn=64)
    nat.check_status()
    ref = torch.zeros(300, 64, device="cuda")
    ref[:, :48] = 0.5 * (x.float() @ w.float().t())
    _close(y, ref + r.float(), what="gemm alpha/residual/pad")


@pytest.mark.parametrize("segs,r", [((256, 128, 128), 16), ((512,), 16), ((256, 256), 8), ((256, 128, 128), 64)])
def test_gemm_lora_forward(segs, r):
    nat = _nat()
    torch.manual_seed(2)
    M, K, N = 640, 512, sum(segs)
    x, w = _rand(M, K), _rand(N, K, scale=K ** -0.5)
    a, b = _rand(len(segs) * r, K, scale=K ** -0.5), _rand(N, r, scale=0.2)
    res = _rand(M, N)
    t = nat.lora_t(x, a, 2.0)
    y = nat.gemm_lora(x, w, t, b, segs, r, res)
    nat.check_status()
    ref = x.float() @ w.float().t() + res.float()
    n0 = 0
    for i, sz in enumerate(segs):
        ti = 2.0 * (x.float() @ a[i * r:(i + 1) * r].float().t())
        _close(t[:, i * r:(i + 1) * r], ti, what="lora_t")
        ref[:, n0:n0 + sz] += ti.to(torch.bfloat16).float() @ b[n0:n0 + sz].float().t()
        n0 += sz
    assert torch.all(t[:, len(segs) * r:] == 0)
    _close(y, ref, what="gemm_lora")


@pytest.mark.parametrize("mn", [True, False])
def test_lora_backward_pieces(mn):
    nat = _nat()
    old = nat.MN_MAJOR
    nat.MN_MAJOR = mn
    try:
        torch.manual_seed(3)
        segs, r = (256, 128, 128), 16
        M, K, N = 1024, 512, sum(segs)
        x, dy = _rand(M, K), _rand(M, N)
        w = _rand(N, K, scale=K ** -0.5)
        a, b = _rand(len(segs) * r, K, scale=K ** -0.5), _rand(N, r, scale=0.2)
        t = nat.lora_t(x, a, 2.0)
        dt = nat.lora_dt(dy, b, segs, r, 2.0)
        n0 = 0
        dt_ref = torch.zeros(M, len(segs) * r, device="cuda")
        for i, sz in enumerate(segs):
            dt_ref[:, i * r:(i + 1) * r] = 2.0 * (dy[:, n0:n0 + sz].float() @ b[n0:n0 + sz].float())
            n0 += sz
        _close(dt[:, :len(segs) * r], dt_ref, what="lora_dt")
        for wt in (w.t().contiguous(), None):
            dx = nat.gemm_lora_dx(dy, w, wt, dt, a)
            _close(dx, dy.float() @ w.float() + dt[:, :len(segs) * r].float() @ a.float(), what="gemm_lora_dx")
        da = torch.zeros(len(segs) * r, K, device="cuda")
        nat.lora_da(dt, x, len(segs) * r, da)
        _close(da, dt[:, :len(segs) * r].float().t() @ x.float(), rtol=2e-2, atol=0.5, what="lora_da")
        db = torch.zeros(N, r, device="cuda")
        nat.lora_db(dy, t, segs, r, db)
        db_ref = torch.zeros(N, r, device="cuda")
        n0 = 0
        for i, sz in enumerate(segs):
            db_ref[n0:n0 + sz] = dy[:, n0:n0 + sz].float().t() @ t[:, i * r:(i + 1) * r].float()
            n0 += sz
        _close(db, db_ref, rtol=2e-2, atol=0.5, what="lora_db")
        nat.check_status()
    finally:
        nat.MN_MAJOR = old


def test_lora_gradients_are_bitwise_reproducible_in_deterministic_mode():
    """dA and dB are reductions over all tokens. The default path sums CTA partials with fp32 atomics (order varies);
    the deterministic mode gives one CTA each output tile, so two runs must agree bit for bit."""
    nat = _nat()
    old = nat.DETERMINISTIC
    try:
        torch.manual_seed(4)
        segs, r = (512, 256, 256), 16
        M, K, N = 8192, 1024, sum(segs)
        x, dy = _rand(M, K), _rand(M, N)
        a, b = _rand(len(segs) * r, K, scale=K ** -0.5), _rand(N, r, scale=0.2)
        t = nat.lora_t(x, a, 2.0)
        dt = nat.lora_dt(dy, b, segs, r, 2.0)
        outs = {}
        for det in (True, True, False):
            nat.DETERMINISTIC = det
            da = torch.zeros(len(segs) * r, K, device="cuda")
            db = torch.zeros(N, r, device="cuda")
            nat.lora_da(dt, x, len(segs) * r, da)
            nat.lora_db(dy, t, segs, r, db)
            nat.lora_da(dt, x, len(segs) * r, da)          # accumulation over micro-batches goes the same way
            outs.setdefault(det, []).append((da, db))
        nat.check_status()
        (da1, db1), (da2, db2) = outs[True]
        assert torch.equal(da1, da2) and torch.equal(db1, db2)
        _close(da1, outs[False][0][0], rtol=1e-3, atol=1e-2, what="deterministic vs atomic dA")
        _close(db1, outs[False][0][1], rtol=1e-3, atol=1e-2, what="deterministic vs atomic dB")
        _close(da1, 2 * (dt[:, :len(segs) * r].float().t() @ x.float()), rtol=2e-2, atol=1.0, what="dA")
    finally:
        nat.DETERMINISTIC = old


def test_cta_pair_gemm_with_lora_segments_at_the_training_shape():
    """The 256 x 256 CTA-pair kernel on the benchmark's QKV projection (16384 tokens, 3 LoRA segments) and its input
    gradient, against fp32."""
    nat = _nat()
    torch.manual_seed(6)
    M, K, segs, r = 16384, 1024, (2048, 1024, 1024), 16
    N = sum(segs)
    x, w = _rand(M, K), _rand(N, K, scale=K ** -0.5)
    a, b = _rand(len(segs) * r, K, scale=K ** -0.5), _rand(N, r, scale=0.2)
    res = None
    t = nat.lora_t(x, a, 2.0)
    y = nat.gemm_lora(x, w, t, b, segs, r, res)
    nat.check_status()
    ref = x.float() @ w.float().t()
    n0 = 0
    for i, sz in enumerate(segs):
        ref[:, n0:n0 + sz] += t[:, i * r:(i + 1) * r].float() @ b[n0:n0 + sz].float().t()
        n0 += sz
    _close(y, ref, what="2-SM gemm + lora (training shape)")
    dy = _rand(M, N)
    dt = nat.lora_dt(dy, b, segs, r, 2.0)
    for wt in (w.t().contiguous(), None):
        dx = nat.gemm_lora_dx(dy, w, wt, dt, a)
        _close(dx, dy.float() @ w.float() + dt[:, :len(segs) * r].float() @ a.float(), rtol=2e-2, atol=5e-2,
               what="2-SM dX + lora (training shape)")
    nat.check_status()


@pytest.mark.parametrize("T,H", [(777, 1024), (130, 2048), (99, 768), (61, 2560)])
def test_rmsnorm(T, H):
    """H = 768 ... 2048 take the register-resident backward, 2560 the looping one."""
    nat = _nat()
    from pmetal_b200.ops import reference as ref
    torch.manual_seed(4)
    x, res, w = _rand(T, H), _rand(T, H), (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
    h, y, rstd = nat.rmsnorm_fwd(x, w, 1e-6, res)
    hr = (x.float() + res.float()).bfloat16()
    assert torch.equal(h, hr)
    _close(y, ref.rms_norm(hr.float(), w.float(), 1e-6), what="rmsnorm fwd")
    dy, dh = _rand(T, H), _rand(T, H)
    dx, dw = nat.rmsnorm_bwd(dy, h, w, rstd, dh, True)
    hf = hr.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    ref.rms_norm(hf, wf, 1e-6).backward(dy.float())
    _close(dx, hf.grad + dh.float(), what="rmsnorm dx")
    _close(dw, wf.grad, rtol=3e-2, atol=0.5, what="rmsnorm dw")


@pytest.mark.parametrize("T,H", [(64, 2048), (5, 1024), (300, 4096), (17, 2560)])
def test_rmsnorm_few_rows(T, H):
    """The one-CTA-per-row variant used for decode-sized inputs, with and without the residual add."""
    nat = _nat()
    from pmetal_b200.ops import reference as ref
    torch.manual_seed(5)
    x, res, w = _rand(T, H), _rand(T, H), (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
    h, y, rstd = nat.rmsnorm_fwd(x, w, 1e-6, res)
    hr = (x.float() + res.float()).bfloat16()
    assert torch.equal(h, hr)
    _close(y, ref.rms_norm(hr.float(), w.float(), 1e-6), what="rmsnorm fwd (rows)")
    _, y2, rstd2 = nat.rmsnorm_fwd(x, w, 1e-6)
    _close(y2, ref.rms_norm(x.float(), w.float(), 1e-6), what="rmsnorm fwd (rows, no residual)")
    _close(rstd2, (x.float().pow(2).mean(-1) + 1e-6).rsqrt(), rtol=1e-3, atol=1e-3, what="rstd")


def test_rope_table_from_frequency_schedule():
    """llama3 / yarn tables from the host-built frequency vector equal the fp32 reference, attention factor included."""
    nat = _nat()
    from pmetal_b200.models.rope import rope_inv_freq
    pos = torch.randint(0, 30000, (257,), device="cuda", dtype=torch.int32)
    for sc in ({"rope_type": "llama3", "factor": 8.0, "original_max_position_embeddings": 8192},
               {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 8192}):
        inv, att = rope_inv_freq(128, 5e5, sc, 32768)
        cs, sn = nat.rope_table_freqs(pos, inv.cuda(), att)
        ang = pos.double()[:, None] * inv.double().cuda()[None, :]
        _close(cs, (ang.cos() * att).float(), rtol=0, atol=2e-3, what="cos " + sc["rope_type"])
        _close(sn, (ang.sin() * att).float(), rtol=0, atol=2e-3, what="sin " + sc["rope_type"])


@pytest.mark.parametrize("T,hq,hkv", [(300, 4, 2), (1101, 4, 2), (2050, 3, 1)])
def test_qknorm_rope(T, hq, hkv):
    """300 tokens run one warp per head; the larger cases run the 16-lanes-per-head kernels, with a ragged last warp
    and with q and k heads sharing a warp."""
    nat = _nat()
    from pmetal_b200.ops import reference as ref
    torch.manual_seed(5)
    d = 128
    qkv = _rand(T, (hq + 2 * hkv) * d)
    qw = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
    kw = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
    pos = torch.randint(0, 5000, (T,), device="cuda", dtype=torch.int32)
    cs, sn = nat.rope_table(pos, d, 1e6, 1.0)
    cr, sr = ref.rope_cos_sin(pos, d, 1e6)
    _close(cs, cr, rtol=0, atol=2e-3, what="cos")
    _close(sn, sr, rtol=0, atol=2e-3, what="sin")
    q, k = nat.qknorm_rope_fwd(qkv, qw, kw, cs, sn, hq, hkv, 1e-6)
    x = qkv.float().requires_grad_(True)
    qr = ref.apply_rope(ref.rms_norm(x[:, :hq * d].view(T, hq, d), qw.float(), 1e-6), cr, sr)
    kr = ref.apply_rope(ref.rms_norm(x[:, hq * d:(hq + hkv) * d].view(T, hkv, d), kw.float(), 1e-6), cr, sr)
    _close(q, qr, what="q rope")
    _close(k, kr, what="k rope")
    dq, dk = _rand(T, hq, d), _rand(T, hkv, d)
    dqkv = torch.zeros_like(qkv)
    nat.qknorm_rope_bwd(dq, dk, qkv, qw, kw, cs, sn, hq, hkv, 1e-6, dqkv)
    (qr * dq.float()).sum().add((kr * dk.float()).sum()).backward()
    _close(dqkv[:, :(hq + hkv) * d], x.grad[:, :(hq + hkv) * d], what="qknorm_rope bwd")


@pytest.mark.parametrize("act", ["silu", "gelu_tanh", "gelu"])
def test_gated_activations(act):
    """act(gate) * up forward and backward, with separate matrices and with the two halves of one fused projection."""
    from pmetal_b200.ops import functional as F
    torch.manual_seed(21)
    T, I = 333, 768
    fn = {"silu": torch.nn.functional.silu, "gelu_tanh": lambda x: torch.nn.functional.gelu(x, approximate="tanh"),
          "gelu": torch.nn.functional.gelu}[act]
    fused = _rand(T, 2 * I, scale=2.0).requires_grad_(True)
    for halves in (True, False):
        if halves:
            g, u = fused.chunk(2, -1)
        else:
            g, u = _rand(T, I, scale=2.0).requires_grad_(True), _rand(T, I).requires_grad_(True)
        n0 = _nat().LAUNCHES if hasattr(_nat(), "LAUNCHES") else 0
        y = F.glu(g, u, act)
        dy = _rand(T, I)
        grads = torch.autograd.grad(y, (fused,) if halves else (g, u), dy)
        gr = (fused if halves else g).detach().float().requires_grad_(True)
        if halves:
            g32, u32 = gr.chunk(2, -1)
            want = fn(g32) * u32
            wg = torch.autograd.grad(want, gr, dy.float())
        else:
            ur = u.detach().float().requires_grad_(True)
            want = fn(gr) * ur
            wg = torch.autograd.grad(want, (gr, ur), dy.float())
        _close(y, want, what=f"{act} forward")
        for a, b in zip(grads, wg):
            _close(a, b, what=f"{act} backward")
    _nat().check_status()


@pytest.mark.parametrize("T", [200, 1500])
def test_rope_without_qk_norm(T):
    """Architectures without QK-norm pass no weights: the kernels only rotate (and un-rotate in backward)."""
    nat = _nat()
    from pmetal_b200.ops import reference as ref
    torch.manual_seed(15)
    hq, hkv, d = 4, 2, 128
    qkv = _rand(T, (hq + 2 * hkv) * d)
    pos = torch.arange(T, device="cuda", dtype=torch.int32)
    cs, sn = nat.rope_table(pos, d, 1e4, 1.0)
    q, k = nat.qknorm_rope_fwd(qkv, None, None, cs, sn, hq, hkv, 1e-6)
    _close(q, ref.apply_rope(qkv[:, :hq * d].float().view(T, hq, d), cs, sn), what="q rope only")
    _close(k, ref.apply_rope(qkv[:, hq * d:(hq + hkv) * d].float().view(T, hkv, d), cs, sn), what="k rope only")
    dq, dk = _rand(T, hq, d), _rand(T, hkv, d)
    dqkv = torch.zeros_like(qkv)
    nat.qknorm_rope_bwd(dq, dk, qkv, None, None, cs, sn, hq, hkv, 1e-6, dqkv)
    _close(dqkv[:, :hq * d].view(T, hq, d), ref.apply_rope(dq.float(), cs, -sn), what="dq un-rotated")
    _close(dqkv[:, hq * d:(hq + hkv) * d].view(T, hkv, d), ref.apply_rope(dk.float(), cs, -sn), what="dk un-rotated")


def test_swiglu():
    nat = _nat()
    from pmetal_b200.ops import reference as ref
    torch.manual_seed(6)
    gu = _rand(513, 2 * 768)
    out = nat.swiglu_fwd(gu)
    x = gu.float().requires_grad_(True)
    r = ref.swiglu(x)
    _close(out, r, what="swiglu fwd")
    d = _rand(513, 768)
    r.backward(d.float())
    _close(nat.swiglu_bwd(d, gu), x.grad, what="swiglu bwd")


def _doc_bounds(T, lens):
    cu = [0]
    for n in lens:
        cu.append(min(cu[-1] + n, T))
    if cu[-1] < T:
        cu.append(T)
    return torch.tensor(cu, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("T,lens,hq,hkv,window", [(256, [256], 2, 1, 0), (512, [100, 37, 200, 175], 4, 2, 0),
                                                  (1000, [333, 64, 1, 450, 152], 4, 2, 0),
                                                  (768, [500, 268], 2, 2, 96)])
def test_attention_fwd_bwd(T, lens, hq, hkv, window):
    nat = _nat()
    from pmetal_b200.ops import reference as ref
    torch.manual_seed(7)
    d = 128
    cu = _doc_bounds(T, lens)
    ss = ref.seq_starts_from_cu(cu, T)
    q, k, v = _rand(T, hq, d), _rand(T, hkv, d), _rand(T, hkv, d)
    scale = d ** -0.5
    o, lse = nat.attn_fwd(q, k, v, ss, scale, window)
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    orf = ref.varlen_attention(qf, kf, vf, cu, scale, True, window)
    _close(o, orf, what="attn fwd")
    do = _rand(T, hq, d)
    orf.backward(do.float())
    dq, dk, dv = nat.attn_bwd(do, q, k, v, o, lse, ss, scale, window)
    _close(dq, qf.grad, rtol=3e-2, atol=3e-2, what="attn dq")
    _close(dk, kf.grad, rtol=3e-2, atol=3e-2, what="attn dk")
    _close(dv, vf.grad, rtol=3e-2, atol=3e-2, what="attn dv")


def _packed_lens(T, lo, hi, seed):
    g = torch.Generator().manual_seed(seed)
    lens, tot = [], 0
    while tot < T:
        n = int(torch.randint(lo, hi + 1, (1,), generator=g))
        lens.append(min(n, T - tot))
        tot += lens[-1]
    return lens


def test_attention_training_shape():
    """The benchmark's shape: 4 packs x 4096 tokens of documents U[64, 2048], 16 query / 8 kv heads."""
    nat = _nat()
    from pmetal_b200.ops import reference as ref
    torch.manual_seed(17)
    T, hq, hkv, d = 16384, 16, 8, 128
    cu = _doc_bounds(T, _packed_lens(T, 64, 2048, 3))
    ss = ref.seq_starts_from_cu(cu, T)
    q, k, v = _rand(T, hq, d), _rand(T, hkv, d), _rand(T, hkv, d)
    scale = d ** -0.5
    o, lse = nat.attn_fwd(q, k, v, ss, scale, 0)
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    orf = ref.varlen_attention(qf, kf, vf, cu, scale, True, 0)
    _close(o, orf, what="attn fwd (training shape)")
    do = _rand(T, hq, d)
    orf.backward(do.float())
    dq, dk, dv = nat.attn_bwd(do, q, k, v, o, lse, ss, scale, 0)
    nat.check_status()
    _close(dq, qf.grad, rtol=3e-2, atol=3e-2, what="attn dq (training shape)")
    _close(dk, kf.grad, rtol=3e-2, atol=3e-2, what="attn dk (training shape)")
    _close(dv, vf.grad, rtol=3e-2, atol=3e-2, what="attn dv (training shape)")


def test_attention_fwd_growing_logits():
    """Keys whose scores grow along the sequence force the running maximum up tile after tile, so the forward
    kernel has to rescale the output accumulator it keeps in tensor memory."""
    nat = _nat()
    from pmetal_b200.ops import reference as ref
    torch.manual_seed(19)
    T, hq, hkv, d = 1536, 2, 1, 128
    cu = _doc_bounds(T, [T])
    ss = ref.seq_starts_from_cu(cu, T)
    base = torch.randn(d, device="cuda")
    base = base / base.norm()
    ramp = torch.linspace(0.0, 40.0, T, device="cuda")[:, None, None]          # up to e^40 between first and last key
    q = (base[None, None, :] * math.sqrt(d) + 0.1 * torch.randn(T, hq, d, device="cuda")).to(torch.bfloat16)
    k = (base[None, None, :] * ramp + 0.1 * torch.randn(T, hkv, d, device="cuda")).to(torch.bfloat16)
    v = _rand(T, hkv, d)
    scale = d ** -0.5
    o, lse = nat.attn_fwd(q, k, v, ss, scale, 0)
    nat.check_status()
    orf = ref.varlen_attention(q.float(), k.float(), v.float(), cu, scale, True, 0)
    _close(o, orf, what="attn fwd (growing logits)")
    s = torch.einsum("qhd,khd->hqk", q.float(), k.float().repeat_interleave(hq // hkv, 1)) * scale
    s = s.masked_fill(~torch.tril(torch.ones(T, T, dtype=torch.bool, device="cuda")), float("-inf"))
    _close(lse, torch.logsumexp(s, -1), rtol=1e-3, atol=2e-2, what="attn lse (growing logits)")


def test_linear_ce():
    nat = _nat()
    torch.manual_seed(8)
    T, H, V = 700, 256, 5000
    h, w = _rand(T, H), _rand(V, H, scale=H ** -0.5)
    lab = torch.randint(0, V, (T,), device="cuda")
    lab[::7] = -100
    for wt in (w.t().contiguous(), None):
        loss, _, n, dh = nat.linear_ce(h, w, wt, lab, -100, 256, True)
        hf = h.float().requires_grad_(True)
        ref = torch.nn.functional.cross_entropy(hf @ w.float().t(), lab, ignore_index=-100, reduction="sum")
        ref.backward()
        assert int(n) == int((lab != -100).sum())
        assert abs(loss.item() - ref.item()) / ref.item() < 5e-3
        _close(dh, hf.grad, rtol=3e-2, atol=2e-3, what="linear_ce dh")
    nat.check_status()


@pytest.mark.parametrize("smooth,cap,mul", [(0.1, 0.0, 1.0), (0.0, 30.0, 1.0), (0.05, 20.0, 1.0), (0.0, 0.0, 0.25), (0.0, 10.0, 0.5)])
def test_linear_ce_label_smoothing_and_softcap(smooth, cap, mul):
    """The chunked loss with a smoothed target, c tanh(x / c) logits and a factor on the logits against fp32 autograd
    (V not a multiple of 8)."""
    nat = _nat()
    torch.manual_seed(18)
    T, H, V = 520, 256, 4003
    h, w = _rand(T, H, scale=3.0), _rand(V, H, scale=H ** -0.5)
    lab = torch.randint(0, V, (T,), device="cuda")
    lab[::5] = -100
    loss, _, n, dh = nat.linear_ce(h, w, None, lab, -100, 256, True, 0.0, None, smooth, cap, mul)
    hf = h.float().requires_grad_(True)
    lg = (hf @ w.float().t()) * mul
    lg = lg + (lg.bfloat16().float() - lg).detach()          # the kernel reads bf16 logits
    if cap > 0:
        lg = cap * torch.tanh(lg / cap)
    ref = torch.nn.functional.cross_entropy(lg, lab, ignore_index=-100, reduction="sum", label_smoothing=smooth)
    ref.backward()
    assert abs(loss.item() - ref.item()) / ref.item() < 5e-3, (loss.item(), ref.item())
    _close(dh, hf.grad, rtol=3e-2, atol=3e-3, what="smoothed / capped linear_ce dh")
    from pmetal_b200.ops import functional as F
    s2, n2 = F.linear_cross_entropy(h, w, lab, softcap=cap, label_smoothing=smooth, logit_scale=mul)
    assert abs(s2.item() - ref.item()) / ref.item() < 5e-3 and int(n2) == int(n)
    nat.check_status()


def test_trainable_dense_linear_and_head_with_z_loss():
    """Full-parameter training pieces against fp32 autograd: y = x W^T (+ residual) with the weight gradient accumulated
    into the fp32 master's .grad, and the chunked cross entropy with the z term and a trainable head."""
    nat = _nat()
    from pmetal_b200.ops import functional as F
    torch.manual_seed(12)
    T, K, N, V = 1500, 256, 384, 3000
    x = _rand(T, K).requires_grad_(True)
    res = _rand(T, N)
    w = (torch.randn(N, K, device="cuda") * K ** -0.5).requires_grad_(True)
    w.shadow = w.detach().bfloat16()
    w.grad = torch.full_like(w, 0.25)                 # accumulation: what is there stays
    y = F.dense_linear(x, w, w.shadow, res)
    dy = _rand(T, N)
    y.backward(dy)
    xr = x.detach().float().requires_grad_(True)
    wr = w.shadow.float().requires_grad_(True)
    (xr @ wr.t() + res.float()).backward(dy.float())
    _close(y, xr @ wr.t() + res.float(), what="dense fwd")
    _close(x.grad, xr.grad, what="dense dx")
    _close(w.grad - 0.25, wr.grad, rtol=2e-2, atol=2e-2 * float(wr.grad.abs().max()), what="dense dw")
    # head: cross entropy + z term, gradients for hidden states and head weight
    h = _rand(T, K).requires_grad_(True)
    hw = (torch.randn(V, K, device="cuda") * K ** -0.5).requires_grad_(True)
    hw.shadow = hw.detach().bfloat16()
    lab = torch.randint(0, V, (T,), device="cuda")
    lab[::5] = -100
    z_coef = 0.05
    total, ce, z = F.linear_cross_entropy_z(h, hw, lab, z_coef, chunk=512)
    (total * 3.0).backward()
    hf = h.detach().float().requires_grad_(True)
    wf = hw.shadow.float().requires_grad_(True)
    lg = hf @ wf.t()
    m = lab != -100
    lse = torch.logsumexp(lg, -1)
    ce_ref = torch.nn.functional.cross_entropy(lg, lab, ignore_index=-100, reduction="sum") / m.sum()
    z_ref = ((lse ** 2) * m).sum() / m.sum()
    ((ce_ref + z_coef * z_ref) * 3.0).backward()
    assert abs(float(ce) - float(ce_ref)) < 5e-3 * float(ce_ref) and abs(float(z) - float(z_ref)) < 1e-2 * float(z_ref)
    assert abs(float(total) - float(ce_ref + z_coef * z_ref)) < 5e-3 * float(total)
    _close(h.grad, hf.grad, rtol=3e-2, atol=3e-2 * float(hf.grad.abs().max()), what="ce+z dh")
    _close(hw.grad, wf.grad, rtol=3e-2, atol=3e-2 * float(wf.grad.abs().max()), what="ce+z dW head")
    nat.check_status()


@pytest.mark.parametrize("scheme,dq", [("nf4", True), ("nf4", False), ("fp4", False)])
def test_gemm_expands_4bit_weight_in_flight(scheme, dq, monkeypatch):
    """Forward and input-gradient GEMMs that read the packed 4-bit weight directly, with and without the low-rank
    second product, against fp32 products with the dequantised weight (which is what the unfused path feeds the GEMM)."""
    nat = _nat()
    from pmetal_b200.lora import nf4
    monkeypatch.setattr(nat, "FUSED_Q4", True)
    torch.manual_seed(13)
    M, K, segs, r = 700, 384, (512, 256, 256), 16
    N = sum(segs)
    w = torch.randn(N, K, device="cuda") * K ** -0.5
    q = nf4.quantize(w, scheme, 64, double_quant=dq).to("cuda")
    wd = nf4.dequantize(q, torch.float32).bfloat16().float()
    assert nat.q4_gemm_ok(q, M, segs)
    x, res = _rand(M, K), _rand(M, N)
    a = _rand(len(segs) * r, K, scale=K ** -0.5)
    b = _rand(N, r, scale=0.2)
    t = nat.lora_t(x, a, 2.0)
    y = nat.gemm_q4_lora(x, q, t, b, segs, r, res)
    nat.check_status()
    ref = x.float() @ wd.t() + res.float()
    o = 0
    for i, sz in enumerate(segs):
        ref[:, o:o + sz] += t[:, i * r:(i + 1) * r].float() @ b[o:o + sz].float().t()
        o += sz
    _close(y, ref, what=f"{scheme} fused forward + lora")
    _close(nat.gemm_q4_lora(x, q, None, None, segs, r), x.float() @ wd.t(), what=f"{scheme} fused forward")
    dy = _rand(M, N)
    dt = nat.lora_dt(dy, b, segs, r, 2.0)
    dx = nat.gemm_q4_lora_dx(dy, q, dt, a)
    nat.check_status()
    _close(dx, dy.float() @ wd + dt[:, :len(segs) * r].float() @ a.float(), rtol=2e-2, atol=5e-2, what=f"{scheme} fused dx + lora")
    _close(nat.gemm_q4_lora_dx(dy, q, None, None), dy.float() @ wd, rtol=2e-2, atol=5e-2, what=f"{scheme} fused dx")
    # a shape with several tiles per pair and a ragged last column tile
    M2, K2, N2 = 1100, 1152, 2560 + 128
    w2 = torch.randn(N2, K2, device="cuda") * K2 ** -0.5
    q2 = nf4.quantize(w2, scheme, 64, double_quant=dq).to("cuda")
    wd2 = nf4.dequantize(q2, torch.float32).bfloat16().float()
    x2, dy2 = _rand(M2, K2), _rand(M2, N2)
    _close(nat.gemm_q4_lora(x2, q2, None, None, (N2,), 0), x2.float() @ wd2.t(), what=f"{scheme} fused forward (large)")
    _close(nat.gemm_q4_lora_dx(dy2, q2, None, None), dy2.float() @ wd2, rtol=2e-2, atol=8e-2, what=f"{scheme} fused dx (large)")
    nat.check_status()


@pytest.mark.parametrize("d,qk_norm", [(64, False), (96, True), (80, False)])
def test_attention_block_small_heads_run_on_the_128_wide_kernels(d, qk_norm):
    """Head sizes below 128 go through the tensor-core attention kernels zero-padded to 128 channels; forward and the
    gradient of the fused projection match the fp32 per-document reference."""
    nat = _nat()
    from pmetal_b200.ops import functional as F
    from pmetal_b200.ops import reference as ref
    torch.manual_seed(3)
    hq, hkv = 4, 2
    lens = [300, 17, 511, 200]
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    pos = torch.cat([torch.arange(n) for n in lens]).to(torch.int32).cuda()
    cos, sin = ref.rope_cos_sin(pos, d, 10000.0)
    qkv = (_rand(T, (hq + 2 * hkv) * d, scale=0.7)).requires_grad_(True)
    qw = kw = None
    if qk_norm:
        qw = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
        kw = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
    n0 = nat.LAUNCHES
    o = F.attention_block(qkv, qw, kw, cos, sin, cu, None, hq, hkv, d, 1e-6)
    assert nat.LAUNCHES > n0                                   # the native kernels ran
    do = _rand(T, hq * d)
    o.backward(do)
    with F.force_reference():
        q32 = qkv.detach().float().requires_grad_(True)
        o_ref = F.attention_block(q32, None if qw is None else qw.float(), None if kw is None else kw.float(), cos, sin, cu,
                                  None, hq, hkv, d, 1e-6)
        o_ref.backward(do.float())
    _close(o, o_ref, rtol=3e-2, atol=3e-2, what=f"attention d={d}")
    _close(qkv.grad, q32.grad, rtol=5e-2, atol=5e-2 * float(q32.grad.abs().max()), what=f"attention d={d} grad")
    nat.check_status()


def test_adamw_and_sumsq():
    nat = _nat()
    from pmetal_b200.ops import reference as ref
    torch.manual_seed(9)
    n = 4096
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda") * 3
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    sh = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    lr_mult = torch.tensor([1.0, 2.0, 1.0, 0.5], device="cuda")
    wd = torch.tensor([0.01, 0.0, 0.01, 0.1], device="cuda")
    gn = torch.zeros(1, device="cuda")
    nat.sumsq(g, gn)
    assert abs(gn.item() - (g.double() ** 2).sum().item()) / gn.item() < 1e-4
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    coef = min(1.0, 1.0 / (math.sqrt(gn.item()) * 0.5 + 1e-6)) * 0.5
    for step in (1, 2):
        nat.adamw_flat(p, g, m, v, sh, lr_mult, wd, gn, 1e-3, 0.9, 0.999, 1e-8, step, 0.5, 1.0)
        for c in range(4):
            s = slice(c * 1024, (c + 1) * 1024)
            ref.adamw_step(pr[s], g[s] * coef, mr[s], vr[s], step, 1e-3 * lr_mult[c].item(), 0.9, 0.999, 1e-8,
                           wd[c].item())
    _close(p, pr, rtol=1e-5, atol=1e-6, what="adamw p")
    _close(sh, pr, rtol=1e-2, atol=1e-2, what="adamw shadow")
    # step 0 = the variant without bias correction
    p2, m2, v2 = torch.randn(1024, device="cuda"), torch.zeros(1024, device="cuda"), torch.zeros(1024, device="cuda")
    g2 = torch.randn(1024, device="cuda")
    p2r, m2r, v2r = p2.clone(), m2.clone(), v2.clone()
    one, zero = torch.ones(1, device="cuda"), torch.zeros(1, device="cuda")
    nat.adamw_flat(p2, g2, m2, v2, None, one, zero, gn, 1e-3, 0.9, 0.999, 1e-8, 0, 1.0, 0.0)
    ref.adamw_step(p2r, g2, m2r, v2r, 0, 1e-3, 0.9, 0.999, 1e-8, 0.0)
    _close(p2, p2r, rtol=1e-5, atol=1e-6, what="adamw without bias correction")


@pytest.mark.parametrize("hq,hkv,lens,qlens", [(4, 2, [70, 1, 300], [1, 1, 1]), (8, 1, [200, 64], [5, 3]),
                                               (2, 2, [5000], [1]), (4, 2, [130, 257], [130, 2])])
def test_paged_attention_and_append(hq, hkv, lens, qlens):
    nat = _nat()
    from pmetal_b200.models.kv_cache import PagedKVCache
    torch.manual_seed(11)
    d = 128
    cache = PagedKVCache(1, hkv, d, 256, torch.bfloat16, "cuda")
    ks, vs = [], []
    for i, (L, n) in enumerate(zip(lens, qlens)):
        cache.add_sequence(i)
        k, v = _rand(L, hkv, d), _rand(L, hkv, d)
        ks.append(k); vs.append(v)
        if L - n > 0:
            slots = torch.tensor(cache.reserve(i, L - n), device="cuda")
            nat.kv_append(k[:L - n], v[:L - n], cache.k[0], cache.v[0], slots)
    meta = cache.prepare(list(range(len(lens))), qlens)
    knew = torch.cat([k[L - n:] for k, L, n in zip(ks, lens, qlens)])
    vnew = torch.cat([v[L - n:] for v, L, n in zip(vs, lens, qlens)])
    nat.kv_append(knew, vnew, cache.k[0], cache.v[0], meta.slots)
    for i in range(len(lens)):
        kk, vv = cache.gather(0, i)
        assert torch.equal(kk, ks[i]) and torch.equal(vv, vs[i])
    q = _rand(meta.total_q, hq, d)
    scale = d ** -0.5
    outs = [nat.paged_attn(q, cache.k[0], cache.v[0], meta, scale, 0, n_split=s) for s in (1, 3)]
    rep = hq // hkv
    qs = meta.q_start.tolist()
    for i, (L, n) in enumerate(zip(lens, qlens)):
        qq = q[qs[i]:qs[i] + n].float().transpose(0, 1)
        kk = ks[i].float().transpose(0, 1).repeat_interleave(rep, 0)
        vv = vs[i].float().transpose(0, 1).repeat_interleave(rep, 0)
        sc = qq @ kk.transpose(1, 2) * scale
        qpos = torch.arange(L - n, L, device="cuda")[:, None]
        sc = sc.masked_fill(torch.arange(L, device="cuda")[None, :] > qpos, float("-inf"))
        ref = (sc.softmax(-1) @ vv).transpose(0, 1)
        for o in outs:
            _close(o[qs[i]:qs[i] + n], ref, what=f"paged attn seq {i}")


@pytest.mark.parametrize("hq,hkv,lens,qlens,window,sink", [(4, 2, [70, 1, 300], [1, 1, 1], 0, 0),
                                                           (8, 2, [2000, 130], [1, 3], 0, 0),
                                                           (4, 2, [900, 333], [1, 2], 256, 16),
                                                           (2, 2, [5000], [1], 512, 64)])
def test_paged_attention_int8_cache_and_sink_window(hq, hkv, lens, qlens, window, sink):
    """int8 blocks (quantised by the append kernel, expanded by the attention kernel) against the same attention over
    the de-quantised values, and the sink + window mask with recycled blocks against dense masked attention."""
    nat = _nat()
    from pmetal_b200.models.kv_cache import PagedKVCache
    torch.manual_seed(13)
    d = 128
    cache = PagedKVCache(1, hkv, d, 256, torch.bfloat16, "cuda", quant="int8", window=window, sink=sink)
    ks, vs = [], []
    for i, (L, n) in enumerate(zip(lens, qlens)):
        cache.add_sequence(i)
        k, v = _rand(L, hkv, d), _rand(L, hkv, d)
        ks.append(k); vs.append(v)
        if L - n > 0:
            slots = torch.tensor(cache.reserve(i, L - n), device="cuda")
            cache.append(0, k[:L - n], v[:L - n], slots)
    meta = cache.prepare(list(range(len(lens))), qlens)      # recycles the blocks behind the window
    knew = torch.cat([k[L - n:] for k, L, n in zip(ks, lens, qlens)])
    vnew = torch.cat([v[L - n:] for v, L, n in zip(vs, lens, qlens)])
    cache.append(0, knew, vnew, meta.slots)
    # the append kernel's codes and scales equal the PyTorch quantiser's
    qk, sk = cache.quantize_rows(knew)
    flat = cache.k[0].view(-1, hkv, d)[meta.slots]
    assert (flat.int() - qk.int()).abs().max() <= 1
    assert torch.allclose(cache.k_scale[0].view(-1, hkv, 2)[meta.slots], sk, rtol=1e-6)
    if window:
        assert cache.live_blocks(0) < -(-lens[0] // 64)            # blocks behind the window went back to the pool
        assert cache.live_blocks(0) <= -(-window // 64) + 2 + -(-sink // 64)
    q = _rand(meta.total_q, hq, d)
    scale = d ** -0.5
    outs = [cache.attention(0, q, meta, scale)] + [nat.paged_attn(q, cache.k[0], cache.v[0], meta, scale, window, n_split=3,
                                                                  sink=sink, k_scale=cache.k_scale[0],
                                                                  v_scale=cache.v_scale[0])]
    rep = hq // hkv
    qs = meta.q_start.tolist()
    for i, (L, n) in enumerate(zip(lens, qlens)):
        qq = q[qs[i]:qs[i] + n].float().transpose(0, 1)

        def dq(x):
            c, sc = cache.quantize_rows(x)
            return (c.float().reshape(L, hkv, 2, 64) * sc[..., None]).reshape(L, hkv, d)
        kk = dq(ks[i]).transpose(0, 1).repeat_interleave(rep, 0)
        vv = dq(vs[i]).transpose(0, 1).repeat_interleave(rep, 0)
        sc = qq @ kk.transpose(1, 2) * scale
        qpos = torch.arange(L - n, L, device="cuda")[:, None]
        kpos = torch.arange(L, device="cuda")[None, :]
        mask = kpos <= qpos
        if window:
            mask &= (kpos > qpos - window) | (kpos < sink)
        sc = sc.masked_fill(~mask, float("-inf"))
        ref = (sc.softmax(-1) @ vv).transpose(0, 1)
        for o in outs:
            _close(o[qs[i]:qs[i] + n], ref, what=f"int8 paged attn seq {i}")
        # and the quantisation error itself is small against the unquantised attention
        kk0 = ks[i].float().transpose(0, 1).repeat_interleave(rep, 0)
        vv0 = vs[i].float().transpose(0, 1).repeat_interleave(rep, 0)
        sc0 = (qq @ kk0.transpose(1, 2) * scale).masked_fill(~mask, float("-inf"))
        _close(outs[0][qs[i]:qs[i] + n], (sc0.softmax(-1) @ vv0).transpose(0, 1), rtol=5e-2, atol=5e-2,
               what=f"int8 vs bf16 attention seq {i}")
    nat.check_status()


@pytest.mark.parametrize("hq,hkv,lens,qlens", [(4, 2, [700, 64, 1], [1, 1, 1]), (8, 2, [2000, 130], [1, 3])])
def test_paged_attention_rotated_4bit_cache(hq, hkv, lens, qlens):
    """Rotated 4-bit code-book cache: the append kernel (rotation, norm, 16-level quantiser) against the PyTorch
    quantiser, and attention in the rotated basis (query rotated in, output rotated back) against dense attention over
    the de-quantised, de-rotated keys and values."""
    nat = _nat()
    from pmetal_b200.models.kv_cache import PagedKVCache
    from pmetal_b200.models.turboquant import unpack_bits
    torch.manual_seed(14)
    d = 128
    cache = PagedKVCache(1, hkv, d, 128, torch.bfloat16, "cuda", quant="tq4")
    tq = cache.tq
    ks, vs = [], []
    for i, (L, n) in enumerate(zip(lens, qlens)):
        cache.add_sequence(i)
        k, v = _rand(L, hkv, d), _rand(L, hkv, d)
        ks.append(k); vs.append(v)
        if L - n > 0:
            cache.append(0, k[:L - n], v[:L - n], torch.tensor(cache.reserve(i, L - n), device="cuda"))
    meta = cache.prepare(list(range(len(lens))), qlens)
    knew = torch.cat([k[L - n:] for k, L, n in zip(ks, lens, qlens)])
    vnew = torch.cat([v[L - n:] for v, L, n in zip(vs, lens, qlens)])
    cache.append(0, knew, vnew, meta.slots)
    # rotation kernel against the PyTorch transform, and its inverse
    x = _rand(50, 3, d)
    _close(nat.tq_rotate(x, tq.sign), tq.rotate(x.float()), what="rotate")
    _close(nat.tq_rotate(nat.tq_rotate(x, tq.sign), tq.sign, inverse=True), x, what="rotate and back")
    # codes: the kernel and the PyTorch quantiser agree except where a coordinate sits on a threshold
    want = tq.encode(knew.float())
    got = cache.k[0].view(-1, hkv, d // 2)[meta.slots]
    cw, cg = unpack_bits(want.codes, 4, d).int(), unpack_bits(got, 4, d).int()
    assert float((cw != cg).float().mean()) < 0.01 and int((cw - cg).abs().max()) <= 1
    sc = cache.k_scale[0].view(-1, hkv, 2)[meta.slots]
    assert torch.allclose(sc[..., 0], knew.float().norm(dim=-1) / d ** 0.5, rtol=1e-3) and torch.equal(sc[..., 0], sc[..., 1])
    q = _rand(meta.total_q, hq, d)
    scale = d ** -0.5
    out = cache.attention(0, q, meta, scale)
    rep = hq // hkv
    qs = meta.q_start.tolist()
    for i, (L, n) in enumerate(zip(lens, qlens)):
        kd, vd = cache.gather(0, i)                               # de-quantised, back in the original basis
        qq = q[qs[i]:qs[i] + n].float().transpose(0, 1)
        kk = kd.float().transpose(0, 1).repeat_interleave(rep, 0)
        vv = vd.float().transpose(0, 1).repeat_interleave(rep, 0)
        s_ = qq @ kk.transpose(1, 2) * scale
        qpos = torch.arange(L - n, L, device="cuda")[:, None]
        kpos = torch.arange(L, device="cuda")[None, :]
        s_ = s_.masked_fill(~(kpos <= qpos), float("-inf"))
        _close(out[qs[i]:qs[i] + n], (s_.softmax(-1) @ vv).transpose(0, 1), rtol=4e-2, atol=4e-2, what=f"4-bit paged attn seq {i}")
        rel = (kd.float() - ks[i].float()).norm() / ks[i].float().norm()
        assert float(rel) < 0.12
    nat.check_status()


def test_generation_with_int8_and_rotating_cache_on_gpu():
    _nat()
    from pmetal_b200.models.config import ModelArgs
    from pmetal_b200.models.decoder import DecoderLM
    from pmetal_b200.models.generation import Generator
    from pmetal_b200.models.sampling import SamplingParams
    cfg = ModelArgs(vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                    num_attention_heads=4, num_key_value_heads=2, head_dim=128)
    m = DecoderLM(cfg).init_weights(0.05, 0).to("cuda").to(torch.bfloat16).eval()
    for p in m.parameters():
        p.requires_grad_(False)
    prompt = torch.randint(0, 2048, (300,), generator=torch.Generator().manual_seed(3)).tolist()
    plain = Generator(m, num_blocks=64).generate([prompt], SamplingParams.greedy(24)).tokens[0]
    # logits of a prefill and of decode steps over the int8 cache stay close to the 16-bit ones (token-for-token
    # equality is too strict for a random model whose logits are nearly flat)
    ga, gb = Generator(m, num_blocks=64), Generator(m, cache=m.new_cache(64, quant="int8"))
    sa, sb = ga.new_seq(), gb.new_seq()
    la, lb = ga.prefill([sa], [prompt]).float(), gb.prefill([sb], [prompt]).float()
    assert (la - lb).abs().max() < 0.05 * la.abs().max(), ((la - lb).abs().max(), la.abs().max())
    for t in plain[:6]:
        tok = torch.tensor([t], device="cuda")
        la, lb = ga.decode_step([sa], tok).float(), gb.decode_step([sb], tok).float()
        assert (la - lb).abs().max() < 0.05 * la.abs().max(), ((la - lb).abs().max(), la.abs().max())
    # a window wider than the text must not change the result (other kernels run: compare logits, not tokens)
    gc = Generator(m, cache=m.new_cache(64, window=4096, sink=4))
    sc = gc.new_seq()
    la, lc = Generator(m, num_blocks=64), None
    sa2 = la.new_seq()
    l0, l1 = la.prefill([sa2], [prompt]).float(), gc.prefill([sc], [prompt]).float()
    assert (l0 - l1).abs().max() < 0.03 * l0.abs().max()
    tok = torch.tensor([plain[0]], device="cuda")
    l0, l1 = la.decode_step([sa2], tok).float(), gc.decode_step([sc], tok).float()
    assert (l0 - l1).abs().max() < 0.03 * l0.abs().max()
    rot = m.new_cache(64, quant="int8", window=128, sink=64)
    g = Generator(m, cache=rot)
    out = g.generate([prompt], SamplingParams.greedy(24))
    assert len(out.tokens[0]) == 24


def test_generation_native_matches_reference_path():
    _nat()
    from pmetal_b200.models.config import ModelArgs
    from pmetal_b200.models.decoder import DecoderLM
    from pmetal_b200.models.generation import Generator
    from pmetal_b200.models.sampling import SamplingParams
    from pmetal_b200.ops import functional as F
    cfg = ModelArgs(vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                    num_attention_heads=2, num_key_value_heads=1, head_dim=128)
    m = DecoderLM(cfg).init_weights(0.05, 0).to("cuda").to(torch.bfloat16).eval()
    for p in m.parameters():
        p.requires_grad_(False)
    prompts = [torch.randint(0, 2048, (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (7, 150)]
    g = Generator(m, num_blocks=64)
    meta_logits = g.prefill([g.new_seq(), g.new_seq()], prompts)
    with F.force_reference():
        g2 = Generator(m, num_blocks=64)
        ref_logits = g2.prefill([g2.new_seq(), g2.new_seq()], prompts)
    _close(meta_logits, ref_logits, rtol=5e-2, atol=5e-2, what="prefill logits")
    out = Generator(m, num_blocks=64).generate(prompts, SamplingParams.greedy(8))
    assert all(len(t) == 8 for t in out.tokens)


@pytest.mark.parametrize("tq,tk,shift", [(256, 384, 384), (300, 200, 0), (128, 500, 100), (260, 260, 0)])
def test_attention_rectangular_blocks(tq, tk, shift):
    """Key j visible to query i iff j <= i + shift: full past blocks (ring attention) and offset causal blocks."""
    nat = _nat()
    torch.manual_seed(3)
    hq, hkv, d = 4, 2, 128
    q, k, v = _rand(tq, hq, d), _rand(tk, hkv, d), _rand(tk, hkv, d)
    ss = torch.zeros(tq, dtype=torch.int32, device="cuda")
    out, lse = nat.attn_fwd_rect(q, k, v, ss, d ** -0.5, shift)
    kk = k.float().repeat_interleave(2, 1).permute(1, 0, 2)
    vv = v.float().repeat_interleave(2, 1).permute(1, 0, 2)
    s = torch.einsum("thd,hsd->hts", q.float(), kk) * d ** -0.5
    i = torch.arange(tq, device="cuda")[:, None]
    j = torch.arange(tk, device="cuda")[None, :]
    s = s.masked_fill(j > i + shift, float("-inf"))
    ref = torch.einsum("hts,hsd->thd", torch.softmax(s, -1), vv)
    _close(out, ref, what="rect attention out")
    assert torch.allclose(lse, torch.logsumexp(s, -1), atol=2e-2, rtol=2e-3)


def test_ring_attention_partial_merge_matches_full():
    """Two chunks on one device: diagonal causal block + full past block merged by log-sum-exp."""
    _nat()
    from pmetal_b200.parallel import cp
    torch.manual_seed(4)
    T, hq, hkv, d = 256, 4, 2, 128
    q, k, v = _rand(2 * T, hq, d), _rand(2 * T, hkv, d), _rand(2 * T, hkv, d)
    o1, l1 = cp._block_attention(q[T:], k[T:], v[T:], d ** -0.5, True)
    o0, l0 = cp._block_attention(q[T:], k[:T], v[:T], d ** -0.5, False)
    out, _ = cp.merge_partials([o1, o0], [l1, l0])
    ss = torch.zeros(2 * T, dtype=torch.int32, device="cuda")
    from pmetal_b200.ops import native
    full, _ = native.attn_fwd(q, k, v, ss, d ** -0.5)
    _close(out, full[T:].float(), what="merged ring partials")
