"""Kernel corpus benchmark (the analogue of the reference's ``pmetal bench-corpus``,
crates/pmetal/src/commands/bench.rs:498-600): fixed kernel cases at the shapes of the
Qwen3-0.6B packed LoRA step, timed with CUDA events after warm-up, reported as
min/median ms, achieved TFLOP/s or GB/s, and fraction of the measured device peak.

    python -m pmetal_b200.bench.kernels [--case NAME ...] [--iters 20] [--json out.json]

Between timed iterations a 256 MB buffer is written so every iteration starts with a cold L2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch


def peaks() -> dict:
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as fh:
            d = json.load(fh)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def timeit(fn, iters: int, warmup: int = 3):
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return min(ts), statistics.median(ts)


def _r(*s, scale=1.0):
    return (torch.randn(*s, device="cuda") * scale).to(torch.bfloat16)


def make_cases(T: int = 16384):
    from pmetal_b200.ops import native as nat
    from pmetal_b200.ops import reference as ref
    cases = {}

    def gemm_case(M, N, K, segs=None, r=16, bn=0):
        x, w = _r(M, K), _r(N, K, scale=K ** -0.5)
        if segs:
            a, b = _r(len(segs) * r, K, scale=K ** -0.5), _r(N, r, scale=0.1)
            t = nat.lora_t(x, a, 2.0)
            return (lambda: nat.gemm_lora(x, w, t, b, segs, r, None, bn)), 2.0 * M * N * (K + r), \
                2.0 * (M * K + N * K + M * N)
        return (lambda: nat.gemm(x, w, bn=bn)), 2.0 * M * N * K, 2.0 * (M * K + N * K + M * N)

    cases["gemm_qkv_lora"] = lambda: gemm_case(T, 4096, 1024, (2048, 1024, 1024))
    cases["gemm_qkv_lora_bn128"] = lambda: gemm_case(T, 4096, 1024, (2048, 1024, 1024), bn=128)
    cases["gemm_gate_up_lora"] = lambda: gemm_case(T, 6144, 1024, (3072, 3072))
    cases["gemm_down_lora"] = lambda: gemm_case(T, 1024, 3072, (1024,))
    cases["gemm_o_lora"] = lambda: gemm_case(T, 1024, 2048, (1024,))
    cases["gemm_lm_head_chunk"] = lambda: gemm_case(4096, 151936, 1024)
    cases["gemm_square_8192"] = lambda: gemm_case(8192, 8192, 8192)

    def lora_side(which):
        """The narrow products of the LoRA path at the q|k|v projection shape (K_in 1024, N 4096, r 16 x 3 segments)."""
        segs, r, K, N = (2048, 1024, 1024), 16, 1024, 4096
        x, dy = _r(T, K), _r(T, N)
        a, b = _r(len(segs) * r, K, scale=K ** -0.5), _r(N, r, scale=0.1)
        t = nat.lora_t(x, a, 2.0)
        dt = nat.lora_dt(dy, b, segs, r, 2.0)
        ga = torch.zeros(len(segs) * r, K, device="cuda")
        gb = torch.zeros(N, r, device="cuda")
        if which == "t":
            return (lambda: nat.lora_t(x, a, 2.0)), 0.0, 2.0 * (T * K + T * 64)
        if which == "dt":
            return (lambda: nat.lora_dt(dy, b, segs, r, 2.0)), 0.0, 2.0 * (T * N + T * 64)
        if which == "da":
            return (lambda: nat.lora_da(dt, x, len(segs) * r, ga)), 0.0, 2.0 * (T * K + T * 64)
        return (lambda: nat.lora_db(dy, t, segs, r, gb)), 0.0, 2.0 * (T * N + T * 64)

    for w_ in ("t", "dt", "da", "db"):
        cases["lora_" + w_] = (lambda w_=w_: lora_side(w_))

    def attn(which, one_doc=False):
        hq, hkv, d = 16, 8, 128
        g = torch.Generator().manual_seed(0)
        lens, tot = [], 0
        while tot < T:
            n = T if one_doc else int(torch.randint(64, 2049, (1,), generator=g))
            n = min(n, T - tot)
            lens.append(n)
            tot += n
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
        ss = ref.seq_starts_from_cu(cu, T)
        q, k, v = _r(T, hq, d), _r(T, hkv, d), _r(T, hkv, d)
        o, lse = nat.attn_fwd(q, k, v, ss, d ** -0.5, 0)
        do = _r(T, hq, d)
        pairs = sum(n * (n + 1) / 2 for n in lens)
        fl = 4.0 * pairs * d * hq
        if which == "fwd":
            return (lambda: nat.attn_fwd(q, k, v, ss, d ** -0.5, 0)), fl, 2.0 * T * d * (2 * hq + 2 * hkv)
        return (lambda: nat.attn_bwd(do, q, k, v, o, lse, ss, d ** -0.5, 0)), 2.5 * fl, 2.0 * T * d * (4 * hq + 4 * hkv)

    cases["attn_varlen_fwd"] = lambda: attn("fwd")
    cases["attn_varlen_bwd"] = lambda: attn("bwd")
    cases["attn_onedoc_fwd"] = lambda: attn("fwd", True)
    cases["attn_onedoc_bwd"] = lambda: attn("bwd", True)

    def rms():
        x, res, w = _r(T, 1024), _r(T, 1024), _r(1024)
        return (lambda: nat.rmsnorm_fwd(x, w, 1e-6, res)), 0.0, 2.0 * T * 1024 * 4

    def swi():
        gu = _r(T, 6144)
        return (lambda: nat.swiglu_fwd(gu)), 0.0, 2.0 * T * (6144 + 3072)

    def ce():
        V = 151936
        lg = _r(2048, V)
        lab = torch.randint(0, V, (2048,), device="cuda")
        loss = torch.zeros(1, device="cuda")
        inv = torch.ones(1, device="cuda")
        from ctypes import c_int, c_longlong
        L = nat.lib()
        return (lambda: L.pm_ce_fwd_bwd(nat._p(lg), c_longlong(V), nat._p(lab), nat._p(loss), nat._p(inv), nat._p(None),
                                        nat._p(None), c_int(2048), c_int(V), c_longlong(-100), c_int(1),
                                        nat._stream())), 0.0, 2.0 * 2048 * V * 3

    def adam():
        n = 10 * 1024 * 1024
        p, g, m, v = (torch.randn(n, device="cuda") for _ in range(4))
        sh = torch.empty(n, device="cuda", dtype=torch.bfloat16)
        lm, wd = torch.ones(n // 1024, device="cuda"), torch.zeros(n // 1024, device="cuda")
        gn = torch.ones(1, device="cuda")
        return (lambda: nat.adamw_flat(p, g, m, v, sh, lm, wd, gn, 1e-4, .9, .999, 1e-8, 3, 1.0, 1.0)), 0.0, n * (7 * 4 + 2)

    def rms_bwd():
        dy, h, w, dh = _r(T, 1024), _r(T, 1024), _r(1024), _r(T, 1024)
        rstd = torch.rand(T, device="cuda") + 0.5
        return (lambda: nat.rmsnorm_bwd(dy, h, w, rstd, dh, False)), 0.0, 2.0 * T * 1024 * 4

    def qk(which):
        hq, hkv = 16, 8
        qkv, qw, kw = _r(T, (hq + 2 * hkv) * 128), _r(128), _r(128)
        cs, sn = nat.rope_table(torch.arange(T, device="cuda", dtype=torch.int32), 128, 1e6, 1.0)
        if which == "fwd":
            return (lambda: nat.qknorm_rope_fwd(qkv, qw, kw, cs, sn, hq, hkv, 1e-6)), 0.0, 2.0 * T * 128 * (hq + hkv) * 2
        dq, dk, dqkv = _r(T, hq, 128), _r(T, hkv, 128), torch.zeros_like(qkv)
        return (lambda: nat.qknorm_rope_bwd(dq, dk, qkv, qw, kw, cs, sn, hq, hkv, 1e-6, dqkv)), 0.0, \
            2.0 * T * 128 * (hq + hkv) * 3

    cases["rmsnorm_add_fwd"] = rms
    cases["rmsnorm_bwd"] = rms_bwd
    cases["qknorm_rope_fwd"] = lambda: qk("fwd")
    cases["qknorm_rope_bwd"] = lambda: qk("bwd")
    cases["swiglu_fwd"] = swi
    cases["ce_fwd_bwd"] = ce
    cases["adamw_flat_10M"] = adam
    return cases


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", nargs="*", default=None)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--json", default=None)
    a = ap.parse_args(argv)
    from pmetal_b200.ops import native
    if not native.available():
        raise SystemExit(f"native library missing: {native.load_error()}")
    pk = peaks()
    cases = make_cases(a.tokens)
    names = a.case or list(cases)
    rows = []
    for n in names:
        fn, flops, nbytes = cases[n]()
        mn, med = timeit(fn, a.iters)
        row = {"case": n, "min_ms": round(mn, 4), "median_ms": round(med, 4)}
        if flops:
            row["tflops"] = round(flops / (med * 1e-3) / 1e12, 1)
            row["frac_of_bf16_peak"] = round(row["tflops"] / pk["bf16_tflops"], 3)
        row["gbs"] = round(nbytes / (med * 1e-3) / 1e9, 1)
        row["frac_of_hbm_peak"] = round(row["gbs"] / pk["hbm_gbs"], 3)
        row["peaks"] = pk["source"]
        rows.append(row)
        print(json.dumps(row), flush=True)
    native.check_status()
    if a.json:
        with open(a.json, "w") as fh:
            json.dump(rows, fh, indent=1)


if __name__ == "__main__":
    main()
