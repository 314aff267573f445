"""Loader of the host C++ library (``csrc/host/*.cpp`` -> ``lib/libpmetal_host.so``).

The library is rebuilt with g++ (a few seconds) when it is missing or older than any of its sources; bindings elsewhere
in the package call :func:`load` and declare their own argument types."""
from __future__ import annotations

import ctypes
import glob
import os
import subprocess
import threading

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC_DIR = os.path.join(_ROOT, "csrc", "host")
SO = os.path.join(_ROOT, "lib", "libpmetal_host.so")
# -ffp-contract=off: a fused multiply-add would change block-codec results in the last bit
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-ffp-contract=off", "-pthread"]
_LOCK = threading.Lock()
_LIB = None


def sources():
    return sorted(glob.glob(os.path.join(SRC_DIR, "*.cpp")))


def build(force: bool = False) -> str:
    os.makedirs(os.path.dirname(SO), exist_ok=True)
    srcs = sources()
    deps = srcs + glob.glob(os.path.join(SRC_DIR, "*.h"))
    stale = force or not os.path.exists(SO) or any(os.path.getmtime(SO) < os.path.getmtime(s) for s in deps)
    if stale:
        tmp = SO + f".{os.getpid()}.tmp"
        r = subprocess.run(["g++"] + CXX_FLAGS + ["-shared", "-o", tmp] + srcs, stdout=subprocess.PIPE,
                           stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError("host library build failed:\n" + r.stdout)
        os.replace(tmp, SO)
    return SO


def build_instrumented(out_path: str, sanitizers: str = "address,undefined") -> str:
    """The same sources with compiler sanitisers, for test runs (``PMETAL_HOST_LIB`` then points the package at it and
    the interpreter is started with the sanitiser runtime preloaded)."""
    r = subprocess.run(["g++", "-O1", "-g", "-std=c++17", "-fPIC", "-ffp-contract=off", "-pthread", f"-fsanitize={sanitizers}",
                        "-fno-omit-frame-pointer", "-fno-sanitize-recover=all", "-shared", "-o", out_path] + sources(),
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("instrumented host library build failed:\n" + r.stdout)
    return out_path


def load() -> ctypes.CDLL:
    global _LIB
    with _LOCK:
        if _LIB is None:
            override = os.environ.get("PMETAL_HOST_LIB")        # an alternative build (sanitisers) for test runs
            _LIB = ctypes.CDLL(override if override else build())
    return _LIB
