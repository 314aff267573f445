"""Builds the native libraries in-tree with nvcc / g++ (sm_100a only).

    python -m pmetal_b200.build [--force]

``libpmetal_b200.so`` holds the CUDA kernels (``pmetal_b200/csrc/*.cu``);
``libpmetal_host.so`` holds host-side C++ (``pmetal_b200/csrc/host/*.cpp``: GGUF
quantisers, packing helpers). Objects are compiled in parallel and cached by mtime.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(ROOT, "csrc")
LIBDIR = os.path.join(ROOT, "lib")
OBJDIR = os.path.join(LIBDIR, "obj")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-ffp-contract=off", "-pthread"]   # no FMA contraction: byte-exact quantisers


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found")


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd, log):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    log.append(" ".join(cmd) + "\n" + r.stdout)
    if r.returncode != 0:
        raise RuntimeError("build failed:\n" + " ".join(cmd) + "\n" + r.stdout)


def build_native(force: bool = False, verbose: bool = False) -> dict:
    os.makedirs(OBJDIR, exist_ok=True)
    log = []
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + \
        glob.glob(os.path.join(CSRC, "host", "*.h"))
    out = {}
    # ---- CUDA
    cu = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    nvcc = _nvcc()
    jobs = []
    objs = []
    for src in cu:
        obj = os.path.join(OBJDIR, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            jobs.append([nvcc] + NVCC_FLAGS + ["-c", src, "-o", obj])
    so = os.path.join(LIBDIR, "libpmetal_b200.so")
    with ThreadPoolExecutor(max_workers=min(8, max(len(jobs), 1))) as ex:
        list(ex.map(lambda c: _run(c, log), jobs))
    if jobs or not os.path.exists(so):
        _run([nvcc, "-shared", "-o", so] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"], log)
    out["cuda"] = so
    # ---- host C++
    cpp = sorted(glob.glob(os.path.join(CSRC, "host", "*.cpp")))
    if cpp:
        hso = os.path.join(LIBDIR, "libpmetal_host.so")
        if force or _stale(hso, cpp + headers):
            _run(["g++"] + CXX_FLAGS + ["-shared", "-o", hso] + cpp, log)
        out["host"] = hso
    if verbose:
        print("\n".join(log))
    out["log"] = "\n".join(log)
    return out


if __name__ == "__main__":
    res = build_native(force="--force" in sys.argv, verbose=True)
    print({k: v for k, v in res.items() if k != "log"})
