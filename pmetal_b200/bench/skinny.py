"""Few-row linear layers: this repository's mat-vec and GEMM kernels against cuBLAS, weights streamed from HBM.

    python -m pmetal_b200.bench.skinny                       tensor-core mat-vec
    PMETAL_GEMV_TC=0 python -m pmetal_b200.bench.skinny      CUDA-core mat-vec

One JSON line per (weight shape, rows): microseconds (median of 20, CUDA events) for ``torch.matmul`` (cuBLAS), the
tcgen05 GEMM with 32 / 64 / 128-wide tiles, and the mat-vec kernel called once per 16 rows. A 256 MB buffer is rewritten
before every timed call so that nothing is served from L2."""
import json


def main(argv=None, args=None) -> int:
    """Also reachable as ``pmetal bench-skinny``."""
    import torch

    from ..ops import native
    dev = torch.device("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timeit(fn, iters=20):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        ts.sort()
        return round(ts[len(ts) // 2], 1)
    for (N, K) in [(5120, 2048), (2048, 4096), (4096, 1024), (1024, 2048), (6144, 1024), (1024, 3072)]:
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        for M in (16, 32, 64, 128):
            x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
            r = {"N": N, "K": K, "M": M, "cublas": timeit(lambda: x @ w.t())}
            for bn in (32, 64, 128):
                r[f"gemm_bn{bn}"] = timeit(lambda: native.gemm(x, w, bn=bn))

            def chunked():
                for a in range(0, M, 16):
                    native.gemv(x[a:a + 16], w)
            if M <= 64:
                r["matvec16"] = timeit(chunked)
            ref = x.float() @ w.float().t()
            r["max_err"] = round(float((native.gemv(x[:16], w).float() - ref[:16]).abs().max()), 4)
            print(json.dumps(r), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
