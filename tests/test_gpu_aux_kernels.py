"""GPU numerics for the sampler, speculative verifier, MoE routing, GGUF / FP8 dequantisation, distillation and merge
kernels; each is compared with a plain PyTorch fp32 restatement of the same op."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _nat():
    from pmetal_b200.ops import native
    if not native.available():
        pytest.fail(f"native library missing: {native.load_error()}")
    return native


def _close(a, b, rtol=2e-2, atol=2e-2, what=""):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    ref = b.abs().max().item()
    assert err <= atol + rtol * ref, f"{what}: max err {err} vs ref max {ref}"


def _f(dev, *vals, dtype=torch.float32):
    return torch.tensor(vals, dtype=dtype, device=dev)


def test_sampler_greedy_topk_topp_minp_distribution():
    nat = _nat()
    dev = "cuda"
    torch.manual_seed(0)
    V = 5000
    logits = torch.randn(4, V, device=dev) * 2
    # greedy
    tok, lp = nat.sample(logits, torch.zeros(4, device=dev))
    assert torch.equal(tok.long(), logits.argmax(-1))
    ref_lp = torch.log_softmax(logits, -1).gather(1, tok.long()[:, None])[:, 0]
    assert torch.allclose(lp, ref_lp, atol=1e-3)
    # top-k = 1 at any temperature is greedy too
    tok, _ = nat.sample(logits, torch.full((4,), 0.7, device=dev), top_k=torch.ones(4, dtype=torch.int32, device=dev),
                        seeds=torch.arange(4, dtype=torch.int64, device=dev))
    assert torch.equal(tok.long(), logits.argmax(-1))
    # empirical distribution under temperature + top-k + top-p + min-p on one row, many draws
    row = torch.randn(1, 64, device=dev) * 1.5
    n = 20000
    rows = row.expand(n, 64).contiguous()
    temp, k, p_, mp = 0.8, 12, 0.9, 0.02
    tok, _ = nat.sample(rows, torch.full((n,), temp, device=dev), top_k=torch.full((n,), k, dtype=torch.int32, device=dev),
                        top_p=torch.full((n,), p_, device=dev), min_p=torch.full((n,), mp, device=dev),
                        seeds=torch.arange(n, dtype=torch.int64, device=dev) + 17, step=3)
    from pmetal_b200.models.sampling import SamplingParams, filtered_logprobs
    sp = SamplingParams(temperature=temp, top_k=k, top_p=p_, min_p=mp, repetition_penalty=1.0)
    logp = filtered_logprobs(row, sp)[0]              # filters act on the temperature-1 distribution
    keep2 = torch.isfinite(logp)
    target = torch.softmax(logp / temp, -1)
    emp = torch.bincount(tok.long(), minlength=64).float() / n
    assert emp[~keep2].sum() == 0
    assert (emp - target).abs().max() < 0.015
    # different seeds give different draws, same seed the same draw
    a, _ = nat.sample(rows[:8], torch.ones(8, device=dev), seeds=torch.full((8,), 5, dtype=torch.int64, device=dev))
    assert len(set(a.tolist())) == 1


def test_sampler_penalties_and_bf16():
    nat = _nat()
    dev = "cuda"
    V = 1000
    logits = torch.zeros(2, V, device=dev)
    logits[:, 10] = 5.0
    logits[:, 20] = 4.0
    counts = torch.zeros(2, V, dtype=torch.int32, device=dev)
    counts[1, 10] = 3
    tok, _ = nat.sample(logits.bfloat16(), torch.zeros(2, device=dev), counts=counts, rep_pen=_f(dev, 1.0, 2.0),
                        freq_pen=_f(dev, 0.0, 0.1), pres_pen=_f(dev, 0.0, 0.1))
    assert tok.tolist() == [10, 20]           # 5/2 - 0.3 - 0.1 = 2.1 < 4
    nat.count_tokens(counts, tok)
    assert counts[0, 10].item() == 1 and counts[1, 20].item() == 1


def test_spec_verify_greedy_and_stochastic():
    nat = _nat()
    dev = "cuda"
    torch.manual_seed(1)
    n, K, V = 3, 4, 300
    target = torch.randn(n, K + 1, V, device=dev)
    am = target.argmax(-1)
    draft = am[:, :K].clone().int()
    draft[1, 2] = (draft[1, 2] + 1) % V        # mismatch at position 2
    draft[2, 0] = (draft[2, 0] + 1) % V        # mismatch at position 0
    acc, nxt = nat.spec_verify(target, None, draft, 0.0)
    assert acc.tolist() == [4, 2, 0]
    assert nxt.tolist() == [am[0, 4].item(), am[1, 2].item(), am[2, 0].item()]
    # stochastic: identical draft and target distributions -> everything is accepted
    dl = target[:, :K].contiguous()
    toks = torch.distributions.Categorical(logits=dl).sample().int()
    acc, nxt = nat.spec_verify(target, dl, toks, 1.0, seeds=torch.arange(n, dtype=torch.int64, device=dev))
    assert acc.tolist() == [K] * n
    # the emitted token follows the target distribution: one position, many trials
    trials, V2 = 30000, 16
    tl = torch.randn(1, 2, V2, device=dev).expand(trials, 2, V2).contiguous()
    dlog = torch.randn(1, 1, V2, device=dev).expand(trials, 1, V2).contiguous()
    dt = torch.distributions.Categorical(logits=dlog[:, 0]).sample().int()[:, None]
    acc, nxt = nat.spec_verify(tl, dlog, dt, 1.0, seeds=torch.arange(trials, dtype=torch.int64, device=dev) * 7 + 1)
    first = torch.where(acc >= 1, dt[:, 0], nxt)       # token emitted at position 0
    emp = torch.bincount(first.long(), minlength=V2).float() / trials
    assert (emp - torch.softmax(tl[0, 0], -1)).abs().max() < 0.015


def test_moe_route_sort_gather_combine():
    nat = _nat()
    dev = "cuda"
    torch.manual_seed(2)
    T, E, k, H = 777, 64, 4, 256
    logits = torch.randn(T, E, device=dev)
    r = nat.moe_route(logits, k, renorm=True)
    p = torch.softmax(logits, -1)
    tw, ti = p.topk(k, -1)
    assert torch.equal(r["topk_idx"].long(), ti)
    assert torch.allclose(r["topk_w"], tw / tw.sum(-1, keepdim=True), atol=1e-5)
    flat = ti.reshape(-1)
    assert torch.equal(r["counts"].long(), torch.bincount(flat, minlength=E))
    assert r["offsets"][-1].item() == T * k
    perm = r["perm"].long()
    assert torch.equal(flat[perm], flat[perm].sort().values)            # grouped by expert
    stable = torch.sort(flat, stable=True).indices
    assert torch.equal(perm, stable)                                     # and stable within an expert
    assert torch.equal(r["inv"].long()[perm], torch.arange(T * k, device=dev))
    x = torch.randn(T, H, device=dev).bfloat16()
    g = nat.moe_gather(x, r["perm"], k)
    assert torch.equal(g, x[perm // k])
    y = nat.moe_combine(g, r["inv"], r["topk_w"], k)                      # identity experts -> y = x * sum(w) = x
    assert torch.allclose(y.float(), x.float(), atol=2e-2, rtol=2e-2)
    r2 = nat.moe_route(logits.bfloat16(), 2, renorm=False)
    p2 = torch.softmax(logits.bfloat16().float(), -1).topk(2, -1)
    assert torch.allclose(r2["topk_w"], p2.values, atol=1e-5)


@pytest.mark.parametrize("T,E,k", [(1, 128, 8), (32, 128, 8), (100, 64, 4), (9, 8, 2)])
def test_moe_route_single_launch_path(T, E, k):
    """Few tokens take the one-CTA kernel (routing + counts + offsets + stable sort); same contract as the large path."""
    nat = _nat()
    torch.manual_seed(T)
    logits = torch.randn(T, E, device="cuda")
    extra = torch.full((E + 1,), -1, dtype=torch.int32, device="cuda")
    r = nat.moe_route(logits, k, renorm=True, offsets_out=extra)
    tw, ti = torch.softmax(logits, -1).topk(k, -1)
    assert torch.equal(r["topk_idx"].long(), ti)
    assert torch.allclose(r["topk_w"], tw / tw.sum(-1, keepdim=True), atol=1e-5)
    flat = ti.reshape(-1)
    counts = torch.bincount(flat, minlength=E)
    assert torch.equal(r["counts"].long(), counts)
    off = torch.cat((torch.zeros(1, dtype=torch.long, device="cuda"), counts.cumsum(0)))
    assert torch.equal(r["offsets"].long(), off) and torch.equal(extra.long(), off)
    assert torch.equal(r["perm"].long(), torch.sort(flat, stable=True).indices)
    assert torch.equal(r["inv"].long()[r["perm"].long()], torch.arange(T * k, device="cuda"))


@pytest.mark.parametrize("name,tid", [("Q4_0", 2), ("Q8_0", 8), ("Q4K", 12), ("Q6K", 14)])
def test_gguf_dequant_kernel_matches_host(name, tid):
    nat = _nat()
    from pmetal_b200.gguf import native as host
    from pmetal_b200.gguf.types import GgmlType
    x = (np.random.default_rng(3).standard_normal(256 * 40) * 0.1).astype(np.float32)
    raw = host.quantize(x, GgmlType(tid))
    ref = host.dequantize(raw, GgmlType(tid), x.size)
    out = nat.gguf_dequant_bf16(torch.from_numpy(raw).cuda(), tid, (40, 256))
    want = torch.from_numpy(ref).reshape(40, 256).bfloat16()
    assert torch.equal(out.cpu(), want)


def test_fp8_block_quant_round_trip():
    nat = _nat()
    torch.manual_seed(4)
    x = (torch.randn(64, 512, device="cuda") * 3).bfloat16()
    x[0, :128] = 0
    q, sc = nat.fp8_quant(x)
    amax = x.float().reshape(-1, 128).abs().amax(-1)
    assert torch.allclose(sc, torch.where(amax > 0, amax / 448, torch.ones_like(amax)), rtol=1e-6)
    y = nat.fp8_dequant(q, sc)
    ref = (x.float().reshape(-1, 128) / sc[:, None]).to(torch.float8_e4m3fn).float() * sc[:, None]
    close = torch.isclose(y.float().reshape(-1, 128), ref.bfloat16().float(), atol=1e-6, rtol=1e-2)
    assert close.float().mean().item() > 0.995       # x * (1/scale) vs x / scale can differ on exact rounding ties
    assert (y.float() - x.float()).abs().max() <= 0.07 * x.float().abs().max()


@pytest.mark.parametrize("kind", ["kl", "reverse_kl", "js", "soft_ce", "tvd"])
def test_distill_kernel_loss_and_grad(kind):
    nat = _nat()
    torch.manual_seed(5)
    rows, V, temp, beta = 6, 3001, 2.0, 0.3
    s0 = (torch.randn(rows, V, device="cuda") * 2).bfloat16()
    t0 = (torch.randn(rows, V, device="cuda") * 2).bfloat16()
    scale = torch.tensor([1.0, 0.5, 0.0, 1.0, 2.0, 1.0], device="cuda")
    s = s0.float().requires_grad_(True)
    ls, lt = torch.log_softmax(s / temp, -1), torch.log_softmax(t0.float() / temp, -1)
    ps, pt = ls.exp(), lt.exp()
    if kind == "kl":
        loss = (pt * (lt - ls)).sum(-1)
    elif kind == "reverse_kl":
        loss = (ps * (ls - lt)).sum(-1)
    elif kind == "js":
        m = beta * pt + (1 - beta) * ps
        loss = (beta * pt * (lt - m.log()) + (1 - beta) * ps * (ls - m.log())).sum(-1)
    elif kind == "soft_ce":
        loss = -(pt * ls).sum(-1)
    else:
        loss = 0.5 * (pt - ps).abs().sum(-1)
    (loss * scale).sum().backward()
    sg = s0.clone()
    row_loss = nat.kd_fwd_bwd(sg, t0, temp, kind, beta, row_scale=scale)
    want = torch.where(scale > 0, loss.detach(), torch.zeros_like(loss))
    assert torch.allclose(row_loss, want, atol=2e-3, rtol=2e-3)
    g = s.grad
    assert (sg.float() - g).abs().max() <= 0.02 * g.abs().max() + 1e-6


def test_merge_kernels_match_torch_methods():
    nat = _nat()
    from pmetal_b200.merge import methods as M
    torch.manual_seed(6)
    n = 100_003
    base = torch.randn(n, device="cuda")
    models = [base + 0.1 * torch.randn(n, device="cuda") for _ in range(3)]
    w = [0.5, 0.3, 0.2]
    out = nat.merge_fused(models, base, w, lam=0.8)
    assert torch.allclose(out, M.task_arithmetic(models, base, w, 0.8), atol=1e-5)
    out = nat.merge_fused(models, None, w)
    assert torch.allclose(out, M.linear(models, w, normalize=False), atol=1e-5)
    dens = [0.3, 0.5, 0.7]
    thr = []
    for m, d in zip(models, dens):
        flat = (m - base).abs()
        kk = min(int(math.ceil((1 - d) * n)), n - 1)
        thr.append(torch.kthvalue(flat, kk + 1).values.item())
    out = nat.merge_fused(models, base, w, thresholds=thr, consensus=True, lam=1.0)
    assert torch.allclose(out, M.ties(models, base, w, dens, 1.0), atol=1e-5)
    # DARE on one model: a `density` fraction survives and survivors are rescaled by 1/density
    one = nat.merge_fused(models[:1], base, [1.0], densities=[0.3], rescale=True, seed=9) - base
    tau = models[0] - base
    kept = one != 0
    assert abs(kept.float().mean().item() - 0.3) < 0.01
    assert torch.allclose(one[kept], tau[kept] / 0.3, rtol=1e-5, atol=1e-6)
    again = nat.merge_fused(models[:1], base, [1.0], densities=[0.3], rescale=True, seed=9) - base
    assert torch.equal(one, again)                                  # same seed, same mask
    other = nat.merge_fused(models[:1], base, [1.0], densities=[0.3], rescale=True, seed=10) - base
    assert not torch.equal(one != 0, other != 0)
    # three models: unbiased estimate of task arithmetic
    out = nat.merge_fused(models, base, w, densities=dens, rescale=True, seed=9)
    diff = (out - base) - (M.task_arithmetic(models, base, w, 1.0) - base)
    assert abs(diff.mean().item()) < 5 * diff.std().item() / math.sqrt(n)
    d3 = nat.dot_norms(models[0], models[1])
    assert torch.allclose(d3, torch.stack([(models[0] * models[1]).sum(), models[0].pow(2).sum(), models[1].pow(2).sum()]),
                          rtol=1e-3)
    ob = nat.merge_fused([m.bfloat16() for m in models], base.bfloat16(), w, out_dtype=torch.bfloat16)
    assert ob.dtype == torch.bfloat16 and (ob.float() - M.task_arithmetic(models, base, w, 1.0)).abs().max() < 0.05


def test_local_grouped_moe_engine_matches_dense_reference():
    nat = _nat()
    from pmetal_b200.parallel.ep import FusedExpertMoE
    torch.manual_seed(8)
    E, k, H, I, T = 8, 2, 256, 384, 1000
    gate_up = (torch.randn(E, 2 * I, H, device="cuda") * 0.05).bfloat16()
    down = (torch.randn(E, H, I, device="cuda") * 0.05).bfloat16()
    eng = FusedExpertMoE(gate_up, down, E, k, max_tokens=1024)
    for _ in range(2):
        x = torch.randn(T, H, device="cuda").bfloat16()
        logits = torch.randn(T, E, device="cuda")
        y = eng.forward(x, logits)
        torch.cuda.synchronize()
        nat.check_status()
        p = torch.softmax(logits, -1)
        w, idx = p.topk(k, -1)
        w = w / w.sum(-1, keepdim=True)
        ref = torch.zeros(T, H, device="cuda")
        for e in range(E):
            tok, slot = (idx == e).nonzero(as_tuple=True)
            h = x[tok].float() @ gate_up[e].float().t()
            h = (torch.nn.functional.silu(h[:, :I]) * h[:, I:]).bfloat16().float()
            ref.index_add_(0, tok, (h @ down[e].float().t()).bfloat16().float() * w[tok, slot][:, None])
        assert (y.float() - ref).abs().max().item() < 0.03 * ref.abs().max().item() + 2e-3


@pytest.mark.parametrize("M,N,K", [(1, 4096, 1024), (4, 1024, 3072), (7, 6144, 1024), (16, 1000, 2048), (3, 151936, 1024)])
def test_gemv_plain_norm_residual(M, N, K):
    nat = _nat()
    torch.manual_seed(M + N)
    x = (torch.randn(M, K, device="cuda")).bfloat16()
    w = (torch.randn(N, K, device="cuda") * K ** -0.5).bfloat16()
    nw = (1 + 0.1 * torch.randn(K, device="cuda")).bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16()
    y = nat.gemv(x, w)
    ref = x.float() @ w.float().t()
    assert (y.float() - ref).abs().max() <= 0.02 * ref.abs().max() + 1e-2
    y = nat.gemv(x, w, norm_w=nw, eps=1e-6, residual=res, alpha=0.5)
    xn = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)
    ref = 0.5 * ((xn.bfloat16().float() * nw.float()).bfloat16().float() @ w.float().t()) + res.float()
    assert (y.float() - ref).abs().max() <= 0.02 * ref.abs().max() + 2e-2


def test_gemv_swiglu_and_lora():
    nat = _nat()
    torch.manual_seed(9)
    M, K, I, r = 5, 1024, 3072, 16
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(2 * I, K, device="cuda") * K ** -0.5).bfloat16()
    a = (torch.randn(2 * r, K, device="cuda") * K ** -0.5).bfloat16()
    b = torch.randn(2 * I, r, device="cuda") * 0.1
    scale = 2.0
    t = nat.gemv(x, a, alpha=scale)
    assert (t.float() - scale * (x.float() @ a.float().t())).abs().max() < 0.05
    y = nat.gemv(x, w, swiglu=True, t=t, lora_b=b, r=r, seg_sizes=(I, I))
    full = x.float() @ w.float().t()
    full[:, :I] += t.float()[:, :r] @ b[:I].t()
    full[:, I:] += t.float()[:, r:2 * r] @ b[I:].t()
    ref = torch.nn.functional.silu(full[:, :I]) * full[:, I:]
    assert (y.float() - ref).abs().max() <= 0.03 * ref.abs().max() + 2e-2
    # stacked q/k/v style segments without swiglu
    segs = (2048, 1024, 1024)
    w3 = (torch.randn(sum(segs), K, device="cuda") * K ** -0.5).bfloat16()
    a3 = (torch.randn(3 * r, K, device="cuda") * K ** -0.5).bfloat16()
    b3 = torch.randn(sum(segs), r, device="cuda") * 0.1
    t3 = nat.gemv(x, a3, alpha=scale)
    y3 = nat.gemv(x, w3, t=t3, lora_b=b3, r=r, seg_sizes=segs)
    ref3 = x.float() @ w3.float().t()
    o = 0
    for i, sz in enumerate(segs):
        ref3[:, o:o + sz] += t3.float()[:, i * r:(i + 1) * r] @ b3[o:o + sz].t()
        o += sz
    assert (y3.float() - ref3).abs().max() <= 0.03 * ref3.abs().max() + 2e-2


@pytest.mark.parametrize("M,K,I", [(1, 1024, 3072), (11, 2048, 768), (16, 1024, 1000)])
def test_gemv_tensor_core_swiglu(M, K, I):
    """SwiGLU epilogue of the tensor-core mat-vec (no LoRA term): gate rows [0, I), up rows [I, 2I)."""
    nat = _nat()
    torch.manual_seed(M)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(2 * I, K, device="cuda") * K ** -0.5).bfloat16()
    nw = (1 + 0.1 * torch.randn(K, device="cuda")).bfloat16()
    y = nat.gemv(x, w, norm_w=nw, eps=1e-6, swiglu=True)
    xn = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)
    full = (xn.bfloat16().float() * nw.float()).bfloat16().float() @ w.float().t()
    ref = torch.nn.functional.silu(full[:, :I]) * full[:, I:]
    assert y.shape == (M, I)
    assert (y.float() - ref).abs().max() <= 0.03 * ref.abs().max() + 2e-2


@pytest.mark.parametrize("scheme,double_quant,M,N,K,swiglu", [("nf4", False, 1, 512, 1024, False), ("nf4", True, 7, 1000, 2560, False),
                                                             ("fp4", False, 16, 384, 1024, True), ("nf4", True, 3, 768, 3072, True)])
def test_gemv_4bit_weights_match_dequantised_reference(scheme, double_quant, M, N, K, swiglu):
    """The fused 4-bit mat-vec (codes expanded in registers) against dequantise-then-multiply, with norm, residual and
    a LoRA term."""
    from pmetal_b200.lora.nf4 import dequantize, quantize
    nat = _nat()
    torch.manual_seed(N + K)
    rows = 2 * N if swiglu else N
    w = (torch.randn(rows, K, device="cuda") * K ** -0.5)
    q = quantize(w, scheme, 64, double_quant)
    wd = dequantize(q, torch.float32).bfloat16().float()
    x = torch.randn(M, K, device="cuda").bfloat16()
    nw = (1 + 0.1 * torch.randn(K, device="cuda")).bfloat16()
    r = 8
    a = (torch.randn(r, K, device="cuda") * K ** -0.5).bfloat16()
    b = torch.randn(rows, r, device="cuda") * 0.1
    xn = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)
    xn = (xn.bfloat16().float() * nw.float()).bfloat16()
    t = nat.gemv(x, a, norm_w=nw, eps=1e-6, alpha=2.0)
    full = xn.float() @ wd.t() + t.float() @ b.t()
    if swiglu:
        y = nat.gemv_q4(x, q, norm_w=nw, eps=1e-6, swiglu=True, t=t, lora_b=b, r=r)
        ref = torch.nn.functional.silu(full[:, :N]) * full[:, N:]
    else:
        res = torch.randn(M, N, device="cuda").bfloat16()
        y = nat.gemv_q4(x, q, norm_w=nw, eps=1e-6, residual=res, t=t, lora_b=b, r=r)
        ref = full + res.float()
    assert y.shape == (M, N)
    assert (y.float() - ref).abs().max() <= 0.03 * ref.abs().max() + 2e-2
    # the bf16 tensor-core path with a LoRA term agrees too
    y2 = nat.gemv(x, wd.bfloat16(), norm_w=nw, eps=1e-6, swiglu=swiglu, t=t, lora_b=b, r=r)
    ref2 = ref if swiglu else full
    assert (y2.float() - ref2).abs().max() <= 0.03 * ref2.abs().max() + 2e-2


@pytest.mark.parametrize("dk,dv,T", [(128, 128, 1), (128, 128, 37), (64, 64, 20), (128, 64, 9), (64, 128, 5)])
def test_gated_delta_rule_scan_kernel(dk, dv, T):
    from pmetal_b200.models.gdn import gdn_recurrent
    nat = _nat()
    torch.manual_seed(dk + T)
    B, H = 2, 3
    q = torch.nn.functional.normalize(torch.randn(B, T, H, dk, device="cuda"), dim=-1) * dk ** -0.5
    k = torch.nn.functional.normalize(torch.randn(B, T, H, dk, device="cuda"), dim=-1)
    v = torch.randn(B, T, H, dv, device="cuda")
    g = torch.rand(B, T, H, device="cuda") * 0.3 + 0.7
    beta = torch.rand(B, T, H, device="cuda")
    S0 = torch.randn(B, H, dk, dv, device="cuda") * 0.1
    y, S = nat.gdn_scan(q, k, v, g, beta, S0)
    for b in range(B):
        yr, Sr = gdn_recurrent(q[b], k[b], v[b], g[b], beta[b], S0[b])
        assert torch.allclose(y[b], yr, atol=1e-4, rtol=1e-4), float((y[b] - yr).abs().max())
        assert torch.allclose(S[b], Sr, atol=1e-4, rtol=1e-4)
    y0, _ = nat.gdn_scan(q, k, v, g, beta)                     # zero initial state
    yr0, _ = gdn_recurrent(q[0], k[0], v[0], g[0], beta[0])
    assert torch.allclose(y0[0], yr0, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("E,N,K,counts,cap", [(4, 256, 128, [3, 0, 40, 1], 32), (16, 768, 2048, [5, 0, 1, 9, 64, 2, 3, 0, 7, 1, 1, 4, 8, 6, 2, 30], 64),
                                              (3, 200, 136, [10, 70, 33], 32), (16, 2048, 768, [4] * 16, 128)])
def test_grouped_gemm_few_rows_per_expert(E, N, K, counts, cap):
    """Swapped-operand expert GEMM (weights in the 128-row operand, a few token rows in the narrow one) against a
    per-row fp32 product: unpadded slabs, experts without rows, experts with more rows than one token tile, widths that
    are not a multiple of the tile; then the gate / up variant with SwiGLU in the epilogue. Garbage in the rows that
    belong to no expert must not leak into the result."""
    nat = _nat()
    torch.manual_seed(5)
    off = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device="cuda")
    n = int(off[-1])
    e_of = torch.cat([torch.full((c,), e, dtype=torch.int64) for e, c in enumerate(counts)]).cuda()
    rows = n + 37
    x = torch.full((rows, K), float("nan"), dtype=torch.bfloat16, device="cuda")
    x[:n] = torch.randn(n, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(E, N, K, device="cuda") * K ** -0.5).to(torch.bfloat16)
    for _ in range(2):              # twice: barriers and accumulator buffers start over cleanly
        y = nat.grouped_gemm_skinny(x, w, off, max_rows_per_expert=cap)
    nat.check_status()
    ref = torch.einsum("rk,rnk->rn", x[:n].float(), w.float()[e_of])
    _close(y[:n], ref, what="few-rows grouped")
    w2 = (torch.randn(E, 2 * N, K, device="cuda") * K ** -0.5).to(torch.bfloat16)
    act = nat.grouped_gemm_skinny(x, w2, off, swiglu=True, max_rows_per_expert=cap)
    nat.check_status()
    gu = torch.einsum("rk,rnk->rn", x[:n].float(), w2.float()[e_of])
    ref_act = torch.nn.functional.silu(gu[:, :N]) * gu[:, N:]
    _close(act[:n], ref_act, what="few-rows grouped swiglu")


@pytest.mark.parametrize("E,N,K,counts", [(4, 256, 128, [130, 0, 257, 64]), (8, 1536, 2048, [300, 5, 0, 129, 1000, 64, 128, 1]),
                                          (3, 200, 136, [10, 20, 30])])
def test_grouped_gemm_forward_dx_dw(E, N, K, counts):
    """Expert-grouped GEMMs in the padded sorted layout against a per-expert fp32 loop: forward, input gradient,
    weight gradient (an expert without rows keeps a zero gradient)."""
    nat = _nat()
    from pmetal_b200.ops import functional as F
    torch.manual_seed(21)
    idx = torch.cat([torch.full((c,), e, dtype=torch.int64) for e, c in enumerate(counts)])
    idx = idx[torch.randperm(idx.numel())].cuda().reshape(-1, 1)
    dest, off, cap = F.padded_expert_layout(idx, E)
    o = off.tolist()
    assert all(x % 128 == 0 for x in o) and o[-1] <= cap and [b - a >= c for a, b, c in zip(o, o[1:], counts)]
    assert dest.unique().numel() == idx.numel()
    n = idx.numel()
    x = (torch.randn(n, K, device="cuda")).to(torch.bfloat16)
    w = (torch.randn(E, N, K, device="cuda") * K ** -0.5).to(torch.bfloat16)
    xs = torch.zeros(cap, K, dtype=torch.bfloat16, device="cuda").index_copy(0, dest, x)
    y = nat.grouped_gemm(0, xs, w, off, N, K)
    nat.check_status()
    e_of = idx.reshape(-1)
    ref_y = torch.einsum("rk,rnk->rn", x.float(), w.float()[e_of])
    _close(y[dest], ref_y, what="grouped fwd")
    pad = torch.ones(cap, dtype=torch.bool, device="cuda")
    pad[dest] = False
    assert float(y[pad].float().abs().max()) == 0.0                                # padding rows stay zero
    dy = (torch.randn(n, N, device="cuda")).to(torch.bfloat16)
    dys = torch.zeros(cap, N, dtype=torch.bfloat16, device="cuda").index_copy(0, dest, dy)
    dx = nat.grouped_gemm(1, dys, w, off, N, K)
    _close(dx[dest], torch.einsum("rn,rnk->rk", dy.float(), w.float()[e_of]), what="grouped dx")
    dw = nat.grouped_gemm(2, dys, xs, off, N, K)
    nat.check_status()
    ref_dw = torch.zeros(E, N, K, device="cuda")
    for e in range(E):
        sel = e_of == e
        if bool(sel.any()):
            ref_dw[e] = dy[sel].float().t() @ x[sel].float()
    _close(dw, ref_dw, rtol=2e-2, atol=2e-2 * max(1.0, float(ref_dw.abs().max())), what="grouped dw")
    for e, c in enumerate(counts):
        if c == 0:
            assert float(dw[e].abs().max()) == 0.0


def test_fused_dp_step_gives_up_on_a_silent_peer_and_recovers():
    """The fused data-parallel kernel is launched as rank 0 of a world of two whose second rank never shows up (its
    signal pad is a local buffer that nothing writes). The bounded wait must run out after the 20 ms limit, the status
    word must carry the peer-timeout code, the process must stay usable, and the next, ordinary step on the same signal
    pad must give the AdamW result."""
    import ctypes
    nat = _nat()
    from pmetal_b200.ops import reference as ref
    lib = nat.lib()
    lib.pm_dp_reduce_adamw.restype = ctypes.c_int
    dev = "cuda"
    n = 8 * 1024
    torch.manual_seed(5)
    g0, g1 = torch.randn(n, device=dev), torch.zeros(n, device=dev)
    p0, p1 = torch.randn(n, device=dev), torch.zeros(n, device=dev)
    s0, s1 = torch.zeros(n, device=dev, dtype=torch.bfloat16), torch.zeros(n, device=dev, dtype=torch.bfloat16)
    pad0, pad1 = torch.zeros(32, dtype=torch.int32, device=dev), torch.zeros(32, dtype=torch.int32, device=dev)
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    lr_mult, wd = torch.ones(n // 1024, device=dev), torch.zeros(n // 1024, device=dev)
    gn = torch.zeros(1, device=dev)
    nat.sumsq(g0, gn)
    arr = ctypes.c_ulonglong * 2

    def launch(world, timeout_s, step):
        ptr = lambda a, b: arr(a.data_ptr(), b.data_ptr())       # noqa: E731
        return lib.pm_dp_reduce_adamw(ptr(g0, g1), ptr(p0, p1), ptr(s0, s1), ptr(pad0, pad1), nat._p(m), nat._p(v),
                                      nat._p(lr_mult), nat._p(wd), nat._p(gn), nat._p(None), ctypes.c_longlong(n),
                                      ctypes.c_int(0), ctypes.c_int(world), ctypes.c_float(1e-2), ctypes.c_float(0.9),
                                      ctypes.c_float(0.999), ctypes.c_float(1e-8), ctypes.c_int(step), ctypes.c_float(1.0),
                                      ctypes.c_float(0.0), ctypes.c_double(timeout_s), ctypes.c_int(16),
                                      nat._p(nat.status_word()), nat._stream())
    before = p0.clone()
    assert launch(2, 0.02, 1) == 0
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="104"):
        nat.check_status()
    assert torch.equal(p0, before)                       # nothing was updated by the abandoned step
    assert int(pad0[25]) == 0 and int(pad0[24]) == 1     # arrival counter cleared, epoch closed
    # the same pad, now as a world of one: an ordinary step
    assert launch(1, 5.0, 1) == 0
    torch.cuda.synchronize()
    nat.check_status()
    pr, mr, vr = before.clone(), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    ref.adamw_step(pr, g0.clone(), mr, vr, 1, 1e-2, 0.9, 0.999, 1e-8, 0.0)
    assert torch.allclose(p0, pr, rtol=1e-5, atol=1e-6) and int(pad0[24]) == 2
    assert torch.allclose(s0.float(), pr, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("T", [40, 700])
def test_batched_lora_rows_pick_their_adapter(T):
    """Multi-adapter LoRA on the grouped kernels (few rows: swapped operands; many rows: 128-row tiles) against the
    per-adapter loop in fp32."""
    _nat()
    from pmetal_b200.lora.batched import NO_ADAPTER, BatchedLoraAdapters, batched_lora_linear
    torch.manual_seed(31)
    K, segs, r, n = 256, (256, 128, 128), 16, 5
    st = BatchedLoraAdapters(n, K, segs, r, torch.bfloat16, "cuda")
    facs = []
    for i in range(n - 1):                      # the last slot stays empty
        a = (torch.randn(len(segs) * r, K, device="cuda") * 0.1).bfloat16()
        b = (torch.randn(sum(segs), r, device="cuda") * 0.1).bfloat16()
        st.load_adapter(i, a, b, 1.0 + 0.5 * i)
        facs.append((a, b, 1.0 + 0.5 * i))
    x = (torch.randn(T, K, device="cuda")).bfloat16()
    w = (torch.randn(sum(segs), K, device="cuda") * K ** -0.5).bfloat16()
    ids = torch.randint(-1, n - 1, (T,), device="cuda")
    y = batched_lora_linear(x, w, st, ids)
    ref = x.float() @ w.float().t()
    for i, (a, b, sc) in enumerate(facs):
        rows = (ids == i).nonzero().flatten()
        t = (x[rows].float() @ a.float().t()).bfloat16().float()
        o = 0
        for s, sz in enumerate(segs):
            ref[rows, o:o + sz] += sc * (t[:, s * r:(s + 1) * r] @ b[o:o + sz].float().t())
            o += sz
    _close(y, ref, what=f"batched lora T={T}")
    assert bool((ids == NO_ADAPTER).any())


@pytest.mark.parametrize("n,C", [(4, 256), (2, 1024), (8, 64)])
def test_hyper_connection_kernels(n, C):
    """Per-token hyper-connection mappings, the two stream applications and all their gradients (including the one
    through the Sinkhorn iterations) against the PyTorch formulation in fp32."""
    _nat()
    from pmetal_b200.models import mhc
    torch.manual_seed(17)
    T, iters = 300, 12
    out_dim = n * n + 2 * n
    x = (torch.randn(T, n, C, device="cuda")).bfloat16()
    phi = (torch.randn(n * C, out_dim, device="cuda") * (n * C) ** -0.5).bfloat16().float()
    bias = torch.randn(out_dim, device="cuda") * 0.5
    alpha = torch.tensor([0.7, 1.3, 0.9], device="cuda")
    w = (torch.randn(C, C, device="cuda") * C ** -0.5)

    def run(native):
        xs = x.clone().requires_grad_(True) if native else x.float().requires_grad_(True)
        p, b, a = (t.clone().requires_grad_(True) for t in (phi, bias, alpha))
        if native:
            pre, post, res = mhc.compute_mappings(xs, p, b, a, iters)
            h_in = mhc.apply_pre(xs, pre)
            h_out = torch.tanh(h_in.float() @ w).to(h_in.dtype)
            y = mhc.apply_post_res(xs, h_out, res, post)
        else:
            pre, post, res = mhc.mappings_reference(xs, p, b, a, iters)
            h_in = torch.einsum("tn,tnc->tc", pre, xs)
            h_out = torch.tanh(h_in @ w)
            y = torch.einsum("tmn,tnc->tmc", res, xs) + post[:, :, None] * h_out[:, None, :]
        g = torch.Generator(device="cuda").manual_seed(5)
        dy = torch.randn(T, n, C, device="cuda", generator=g)
        (y.float() * dy).sum().backward()
        return y.float(), pre, post, res, xs.grad.float(), p.grad, b.grad, a.grad
    got, want = run(True), run(False)
    names = ["y", "H_pre", "H_post", "H_res", "dx", "dphi", "dbias", "dalpha"]
    for name, a, b in zip(names, got, want):
        _close(a, b, rtol=4e-2, atol=4e-2 * max(1.0, float(b.abs().max())) if name.startswith("d") else 3e-2, what=name)
    fr, fc = mhc.amax_gain(got[3])
    assert abs(float(fr) - float(want[3].abs().sum(-1).max())) < 1e-3
    xe = (torch.randn(50, C, device="cuda")).bfloat16()
    assert torch.equal(mhc.expand_streams(xe, n)[:, n - 1], xe)
    _close(mhc.collapse_streams(x), x.float().mean(1), what="collapse")
