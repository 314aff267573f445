"""The host C++ library under AddressSanitizer and UndefinedBehaviorSanitizer.

An instrumented build of ``csrc/host/*.cpp`` is loaded by a child interpreter that has the sanitiser runtimes preloaded,
and the tests that drive the block codecs, the integer dot products, the packer / collation code, the threaded shard
reader and the KV block pool run against it. Any out-of-bounds access, use after free, misaligned or overflowing
arithmetic aborts the child."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TARGETS = ["tests/test_gguf.py", "tests/test_fastpack.py", "tests/test_small_parts.py::test_gguf_reader_survives_mutated_files"]


def _runtime(name: str) -> str:
    p = subprocess.run(["gcc", f"-print-file-name={name}"], stdout=subprocess.PIPE, text=True).stdout.strip()
    return p if os.path.isabs(p) and os.path.exists(p) else ""


@pytest.mark.timeout(900)
def test_host_library_is_clean_under_asan_and_ubsan(tmp_path):
    asan, ubsan = _runtime("libasan.so"), _runtime("libubsan.so")
    if not asan or not ubsan:
        pytest.skip("sanitiser runtimes are not installed with this compiler")
    from pmetal_b200.utils import hostlib
    so = hostlib.build_instrumented(str(tmp_path / "libpmetal_host_san.so"))
    env = dict(os.environ, LD_PRELOAD=f"{asan}:{ubsan}", PMETAL_HOST_LIB=so,
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=1:halt_on_error=1", UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1")
    existing = [t for t in TARGETS if os.path.exists(os.path.join(ROOT, t.split("::")[0]))]
    r = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider"] + existing, cwd=ROOT, env=env,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=850)
    assert r.returncode == 0, r.stdout[-4000:]
    assert "passed" in r.stdout and "AddressSanitizer" not in r.stdout and "runtime error" not in r.stdout, r.stdout[-4000:]
    # the child really ran on the instrumented build
    probe = subprocess.run([sys.executable, "-c", "from pmetal_b200.utils import hostlib; print(hostlib.load()._name)"], cwd=ROOT,
                           env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=120)
    assert so in probe.stdout, probe.stdout[-1000:]


THREADED_DRIVER = r"""
import numpy as np, os, tempfile, torch
from pmetal_b200.gguf import native
from pmetal_b200.gguf.types import GgmlType as T
rng = np.random.default_rng(0)
x = rng.standard_normal(64 * 1024).astype(np.float32)
for t in (T.Q4_0, T.Q8_0, T.Q4K, T.Q6K):
    q = native.quantize(x, t, threads=4)
    y = native.dequantize(q, t, x.size, threads=4)
    assert np.isfinite(y).all()
w = rng.standard_normal((64, 1024)).astype(np.float32)
out = native.matvec_q8k(native.quantize(w, T.Q5K, threads=3), T.Q5K, 64, 1024, x[:1024], threads=4)
assert out.shape == (64,)
from pmetal_b200.utils.safetensors_io import load_file, load_file_parallel, save_file
path = os.path.join(tempfile.mkdtemp(), "m.safetensors")
tensors = {f"w{j}": torch.randn(256, 300 + j) for j in range(12)}
save_file(tensors, path)
a, b = load_file(path), load_file_parallel(path, threads=4)
assert all(torch.equal(a[k], b[k]) for k in tensors)
print("THREADED_OK")
"""


@pytest.mark.timeout(900)
def test_threaded_host_paths_are_race_free_under_tsan(tmp_path):
    """Block codecs split over threads, the row-parallel quantised mat-vec and the multi-threaded shard reader under
    ThreadSanitizer."""
    tsan = _runtime("libtsan.so")
    if not tsan:
        pytest.skip("the thread sanitiser runtime is not installed with this compiler")
    from pmetal_b200.utils import hostlib
    so = hostlib.build_instrumented(str(tmp_path / "libpmetal_host_tsan.so"), sanitizers="thread")
    env = dict(os.environ, LD_PRELOAD=tsan, PMETAL_HOST_LIB=so, PMETAL_READ_THREADS="4",
               TSAN_OPTIONS="halt_on_error=1:report_signal_unsafe=0:exitcode=66")
    r = subprocess.run([sys.executable, "-c", THREADED_DRIVER], cwd=ROOT, env=env, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT, text=True, timeout=850)
    assert r.returncode == 0 and "THREADED_OK" in r.stdout and "ThreadSanitizer" not in r.stdout, r.stdout[-4000:]
