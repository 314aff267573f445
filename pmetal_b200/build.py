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


ABI_HEADER_TOP = '''// C interface of libpmetal_b200.so: every launcher of the sm_100a kernel library.
//
// All functions take raw device pointers and a CUDA stream, allocate nothing unless their comment says so, and return
// 0 on success, a negative value for an argument or descriptor error, or the CUDA error code of the launch. `status`
// arguments point at a device int that a kernel sets when one of its bounded waits runs out (codes 101-109); the
// caller reads it after synchronising the stream. Pointers and the stream must belong to the current device.
// The no-allocation paged-attention entry point is declared in paged_attn_static.h.
//
// This file is written by pmetal_b200/build.py from the definitions in csrc/*.cu; every source includes it, so a
// declaration that drifts from its definition fails to compile.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif
'''


def write_abi_header() -> str:
    """Collect every ``extern "C" ... pm_*`` definition (with the comment block above it) into csrc/pmetal_b200.h."""
    import re
    decls = []
    for src in sorted(glob.glob(os.path.join(CSRC, "*.cu"))):
        with open(src, "r", encoding="utf-8") as fh:
            text = fh.read()
        for m in re.finditer(r'((?:^//[^\n]*\n)*)^extern "C" ([\w \*]+?)\b(pm_\w+)\(([^{;]*?)\)\s*\{', text, re.M | re.S):
            decls.append((os.path.basename(src), m.group(1), m.group(2).strip(), m.group(3), " ".join(m.group(4).split())))
    out, cur = ABI_HEADER_TOP, None
    for fname, comment, ret, name, args in decls:
        if name == "pm_paged_attn_static":
            continue
        if fname != cur:
            out += f"\n// ---------------------------------------------------------------- {fname}\n"
            cur = fname
        out += comment
        line, piece = "", ""
        for tok in f"{ret} {name}({args});".split(" "):
            if len(piece) + len(tok) + 1 > 116:
                line += piece.rstrip() + "\n"
                piece = "    "
            piece += tok + " "
        out += line + piece.rstrip() + "\n"
    out += "\n#ifdef __cplusplus\n}\n#endif\n"
    path = os.path.join(CSRC, "pmetal_b200.h")
    old = open(path, "r", encoding="utf-8").read() if os.path.exists(path) else None
    if old != out:
        with open(path, "w", encoding="utf-8") as fh:
            fh.write(out)
    return path


def build_native(force: bool = False, verbose: bool = False) -> dict:
    os.makedirs(OBJDIR, exist_ok=True)
    log = []
    write_abi_header()
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
