"""Library-level extras: 8-bit Adam, schedule-free AdamW, parameter groups, GaLore, NEFTune, mHC, gated delta-net."""
import math

import pytest
import torch

from pmetal_b200.lora.galore import GaLoreProjector, neftune_noise
from pmetal_b200.models import gdn, mhc
from pmetal_b200.trainer.extra_optimizers import Adam8bit, ScheduleFreeAdamW, build_param_groups


def _quadratic(opt_cls, steps=200, **kw):
    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.randn(8192))
    target = torch.randn(8192)
    opt = opt_cls([w], **kw)
    for _ in range(steps):
        opt.zero_grad()
        loss = ((w - target) ** 2).mean()
        loss.backward()
        opt.step()
    return float(((w - target) ** 2).mean().detach()), opt


def test_adam8bit_tracks_adam_and_saves_memory():
    l8, opt = _quadratic(Adam8bit, lr=0.05)
    lref, _ = _quadratic(torch.optim.Adam, lr=0.05)
    assert l8 < 0.05 and abs(l8 - lref) < 0.05
    assert opt.state_bytes() < 8192 * 8 * 0.3          # vs two fp32 moments


def test_schedule_free_converges_and_eval_swaps():
    loss, opt = _quadratic(ScheduleFreeAdamW, lr=0.1, steps=300)
    assert loss < 0.05
    p = opt.param_groups[0]["params"][0]
    y = p.detach().clone()
    opt.eval()
    x = p.detach().clone()
    opt.train()
    assert torch.allclose(p, y, atol=1e-5) and not torch.equal(x, y)


def test_param_groups():
    m = torch.nn.ModuleDict({"embed_tokens": torch.nn.Embedding(4, 4), "norm": torch.nn.LayerNorm(4), "lin": torch.nn.Linear(4, 4)})
    named = list(m.named_parameters()) + [("layers.0.q_proj.lora_b", torch.nn.Parameter(torch.zeros(2, 2)))]
    groups = {g["name"]: g for g in build_param_groups(named, 1e-3, 0.1, 5e-5, 16.0)}
    assert groups["embedding"]["lr"] == 5e-5 and groups["no_decay"]["weight_decay"] == 0.0
    assert groups["lora_b"]["lr"] == pytest.approx(1.6e-2) and groups["regular"]["weight_decay"] == 0.1


def test_galore_and_neftune():
    torch.manual_seed(0)
    g = torch.randn(64, 8) @ torch.randn(8, 256)          # rank-8 gradient
    pr = GaLoreProjector(rank=8, update_gap=10, scale=1.0)
    low = pr.project(g)
    assert low.shape == (8, 256)
    assert torch.allclose(pr.project_back(low), g, atol=1e-3)
    basis = pr.ortho.clone()
    for _ in range(9):
        pr.project(g + 0.01)
    assert torch.equal(basis, pr.ortho)
    pr.project(torch.randn(64, 256))
    assert not torch.equal(basis, pr.ortho)               # refreshed at the gap
    e = torch.zeros(2, 10, 16)
    n = neftune_noise(e, 5.0)
    assert n.abs().max() <= 5.0 / math.sqrt(160) + 1e-6 and n.abs().max() > 0
    assert torch.equal(neftune_noise(e, 5.0, training=False), e)


def test_mhc_sinkhorn_and_layer():
    torch.manual_seed(0)
    m = mhc.sinkhorn_knopp(torch.randn(4, 4), 50)
    assert torch.allclose(m.sum(-1), torch.ones(4), atol=1e-4) and torch.allclose(m.sum(-2), torch.ones(4), atol=1e-4)
    layer = mhc.MhcLayer(4)
    x = torch.randn(5, 8)
    xs = mhc.expand_streams(x, 4)
    out = layer(xs, lambda h: torch.zeros_like(h))
    assert torch.allclose(mhc.collapse_streams(out), x, atol=1e-4)      # doubly stochastic mixing keeps the mean
    out = layer(xs, lambda h: h * 2)
    assert torch.allclose(mhc.collapse_streams(out), x + 2 * x, atol=1e-4)     # pre sums to 1, post starts at 1
    dyn = mhc.MhcLayer(4, dynamic=True, hidden=8)
    o = dyn(xs, lambda h: h)
    o.sum().backward()
    assert dyn.dynamic.weight.grad is not None and o.shape == xs.shape


def test_mhc_per_token_mappings():
    torch.manual_seed(1)
    n, C, T = 4, 16, 9
    layer = mhc.MhcDynamicLayer(n, C, sinkhorn_iters=30)
    x = torch.randn(T, C)
    xs = mhc.expand_streams(x, n)
    out = layer(xs, lambda h: torch.zeros_like(h))
    assert torch.allclose(mhc.collapse_streams(out), x, atol=1e-4)            # fresh layer: mean-preserving mixing
    out = layer(xs, lambda h: 3 * h)
    assert torch.allclose(mhc.collapse_streams(out), x + 3 * x, atol=1e-3)    # reads the mean stream, writes with gain 1
    with torch.no_grad():
        layer.phi.normal_(0, 0.3)
        layer.alpha.fill_(1.0)
    pre, post, res = mhc.compute_mappings(xs + torch.randn(T, n, C), layer.phi, layer.bias, layer.alpha, 30)
    assert pre.shape == (T, n) and float(pre.detach().min()) > 0 and float(post.detach().max()) < 2
    # the last half step normalises the columns exactly; the rows are as close as 30 iterations bring them
    assert torch.allclose(res.sum(-1), torch.ones(T, n), atol=5e-2) and torch.allclose(res.sum(-2), torch.ones(T, n), atol=1e-4)
    assert not torch.allclose(res[0], res[1])                                  # the mixing depends on the token
    fr, fc = mhc.amax_gain(res.detach())
    assert abs(float(fr) - 1) < 5e-2 and abs(float(fc) - 1) < 1e-3
    o = layer(xs.requires_grad_(True), lambda h: torch.tanh(h))
    o.square().mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in layer.parameters()) and xs.grad is not None


def test_gdn_chunked_equals_recurrent():
    torch.manual_seed(0)
    T, H, dk, dv = 150, 3, 16, 24
    q, k = torch.randn(T, H, dk) * 0.3, torch.nn.functional.normalize(torch.randn(T, H, dk), dim=-1)
    v = torch.randn(T, H, dv)
    g, beta = torch.rand(T, H) * 0.3 + 0.7, torch.rand(T, H)
    y1, s1 = gdn.gdn_recurrent(q, k, v, g, beta)
    y2, s2 = gdn.gdn_chunked(q, k, v, g, beta, chunk=32)
    assert torch.allclose(y1, y2, atol=1e-4) and torch.allclose(s1, s2, atol=1e-4)
    y3, s3 = gdn.gdn_chunked(q[100:], k[100:], v[100:], g[100:], beta[100:], S0=gdn.gdn_recurrent(q[:100], k[:100], v[:100], g[:100], beta[:100])[1])
    assert torch.allclose(y3, y1[100:], atol=1e-4)


def test_turboquant_rotation_codebook_and_attention():
    from pmetal_b200.models import turboquant as tq
    torch.manual_seed(0)
    x = torch.randn(7, 128)
    assert torch.allclose(tq.fwht(tq.fwht(x)) / 128, x, atol=1e-4)
    c, t = tq.lloyd_max_normal(2)
    assert torch.allclose(c, torch.tensor([-1.5104, -0.4528, 0.4528, 1.5104]), atol=2e-3) and t.numel() == 3
    c1, _ = tq.lloyd_max_normal(1)
    assert torch.allclose(c1.abs(), torch.full((2,), math.sqrt(2 / math.pi)), atol=1e-3)
    codes = torch.randint(0, 4, (5, 128), dtype=torch.uint8)
    assert torch.equal(tq.unpack_bits(tq.pack_bits(codes, 2), 2, 128), codes)
    T = tq.TurboQuant(128, bits=4)
    assert torch.allclose(T.unrotate(T.rotate(x)), x, atol=1e-4)
    keys = torch.randn(300, 128) * 2
    ck = T.encode(keys)
    rel = (T.decode(ck) - keys).norm() / keys.norm()
    assert rel < 0.12 and T.compression_ratio(ck, 300) > 3.8
    rel2 = (tq.TurboQuant(128, bits=2).decode(tq.TurboQuant(128, bits=2).encode(keys)) - keys).norm() / keys.norm()
    assert rel < rel2 < 0.4
    q = torch.randn(4, 128)
    s = T.scores(q, ck)
    assert torch.allclose(s, q @ keys.t(), atol=0.15 * (q @ keys.t()).abs().max())
    vals = torch.randn(300, 128)
    out = T.attention(q, ck, T.encode(vals), 128 ** -0.5)
    ref = torch.softmax(q @ keys.t() * 128 ** -0.5, -1) @ vals
    assert torch.nn.functional.cosine_similarity(out, ref, dim=-1).min() > 0.9
    # QJL residual sketch: inner-product estimates stay unbiased on average over many keys at 2 bits
    Tq = tq.TurboQuant(128, bits=2, qjl=True, seed=1)
    cq = Tq.encode(keys)
    err_q = (Tq.scores(q, cq) - q @ keys.t()).mean().abs()
    assert err_q < 0.1 and cq.qjl is not None


def test_tuner_cache(tmp_path):
    from pmetal_b200.utils.tuna import Tuner
    import time
    p = str(tmp_path / "t" / "tuna.json")
    t = Tuner(p, iters=3, warmup=1)
    calls = []

    def run(c):
        calls.append(c)
        if c == "bad":
            raise ValueError("invalid")
        time.sleep(0.004 if c == "slow" else 0.0005)
    key = Tuner.make_key("gemm", 128, 4096, 1024)
    assert t.tune(key, ["slow", "fast", "bad"], run) == "fast"
    n = len(calls)
    assert Tuner(p).tune(key, ["slow", "fast"], run) == "fast" and len(calls) == n      # served from the cache file
    assert Tuner(p).lookup(key) == "fast"
    with pytest.raises(RuntimeError):
        t.tune("other", ["bad"], run)
