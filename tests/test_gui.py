"""Browser front end: API over the job runner, forms from the job specifications, and the page itself."""
import sys
import time

import pytest

pytest.importorskip("fastapi")
from fastapi.testclient import TestClient  # noqa: E402

from pmetal_b200.gui import create_app  # noqa: E402
from pmetal_b200.tui.runner import JobRunner  # noqa: E402

def _fake_cli() -> str:
    """The stand-in command line of the terminal-application tests (same directory), loaded by path."""
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location("_tui_tests", os.path.join(os.path.dirname(os.path.abspath(__file__)), "test_tui.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.FAKE_CLI


FAKE_CLI = _fake_cli()


@pytest.fixture
def client(tmp_path, monkeypatch):
    pkg = tmp_path / "fakecli"
    pkg.mkdir()
    (pkg / "__init__.py").write_text("")
    (pkg / "__main__.py").write_text(FAKE_CLI)
    monkeypatch.setenv("PYTHONPATH", str(tmp_path))
    (tmp_path / "d.jsonl").write_text('{"text": "x"}\n')
    runner = JobRunner(workdir=str(tmp_path / "jobs") if (tmp_path / "jobs").mkdir() is None else None, python=sys.executable,
                       module="fakecli")
    with TestClient(create_app(runner, model_roots=[], dataset_roots=[str(tmp_path)])) as c:
        yield c


def test_page_specs_and_listings(client):
    page = client.get("/").text
    assert "<nav" in page and "/api/specs" in page and "polyline" in page
    s = client.get("/api/specs").json()
    assert s["tabs"]["Training"] == "train" and "grpo" in s["specs"] and "serve" in s["specs"]
    names = [f["name"] for f in s["specs"]["train"]["fields"]]
    assert "model" in names and "max_steps" in names and "func" not in names
    assert s["specs"]["train"]["schema"]["properties"]["max_steps"]["type"] == "integer"
    assert any(m["id"] == "random:tiny-qwen3" for m in client.get("/api/models").json())
    assert client.get("/api/datasets").json()[0]["path"].endswith("d.jsonl")
    assert "torch" in client.get("/api/system").json()


def test_jobs_start_follow_fail_and_cancel(client):
    r = client.post("/api/jobs", json={"command": "train", "values": {"model": "m", "dataset": "d", "max_steps": 5}})
    assert r.status_code == 200 and r.json()["argv"][:1] == ["train"]
    jid = r.json()["id"]
    end = time.time() + 30
    while client.get(f"/api/jobs/{jid}").json()["state"] == "running" and time.time() < end:
        time.sleep(0.1)
    d = client.get(f"/api/jobs/{jid}").json()
    assert d["state"] == "finished" and d["metrics"]["step"] == 5 and len(d["history"]["loss"]) == 5 and d["log"][-1] == "step 5"
    assert client.post("/api/jobs", json={"command": "nope", "values": {}}).status_code == 400
    assert client.post("/api/jobs", json={"command": "quantize", "values": {}}).status_code == 422       # missing required fields
    assert client.post("/api/jobs", json={"command": "train", "values": {"max_steps": "many"}}).status_code == 422
    assert client.get("/api/jobs/99").status_code == 404
    assert [j["id"] for j in client.get("/api/jobs").json()] == [jid]
    assert client.post(f"/api/jobs/{jid}/cancel").json()["state"] == "finished"          # nothing left to cancel
