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
