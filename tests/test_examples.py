"""The scripts under examples/ run as written (tiny random models on the CPU)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(script, *args, timeout=300):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, os.path.join(ROOT, "examples", script), *args], cwd=ROOT, env=env,
                       stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=timeout)
    assert r.returncode == 0, r.stderr[-3000:]
    return [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")], r.stdout


@pytest.mark.timeout(600)
def test_finetune_example():
    lines, out = _run("finetune_lora.py", "--model", "random:tiny-qwen3", "--steps", "3", "--device", "cpu")
    assert lines[0]["steps"] == 3 and lines[0]["adapter"].endswith(".safetensors")
    assert len(out.strip().splitlines()) >= 2                    # the summary and the generated text


@pytest.mark.timeout(600)
def test_grpo_example():
    lines, _ = _run("grpo_custom_reward.py", "--model", "random:tiny-qwen3", "--steps", "2", "--device", "cpu")
    assert [l["step"] for l in lines] == [1, 2] and all(0.0 <= l["mean_reward"] <= 1.0 for l in lines)


@pytest.mark.timeout(600)
def test_serve_client_example():
    lines, _ = _run("serve_client.py", "--model", "random:tiny-qwen3", "--device", "cpu", "--port", "18557")
    assert lines[0]["address"].endswith(":18557") and isinstance(lines[0]["text"], str)
