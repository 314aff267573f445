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


def test_settings_directories_and_dashboard(client, tmp_path):
    cfg = client.get("/api/config").json()
    assert cfg["model_directories"] == [] and cfg["default_lora_r"] == 16
    assert client.put("/api/config", json={"default_lora_r": 32, "default_learning_rate": 1}).json()["default_lora_r"] == 32
    assert client.get("/api/config").json()["default_learning_rate"] == 1.0
    assert client.put("/api/config", json={"nonsense": 1}).status_code == 422
    assert client.put("/api/config", json={"default_lora_r": "many"}).status_code == 422
    lib = tmp_path / "lib"
    (lib / "m1").mkdir(parents=True)
    (lib / "m1" / "config.json").write_text('{"model_type": "qwen3", "hidden_size": 64, "num_hidden_layers": 2, "vocab_size": 100}')
    assert client.post("/api/model-directories", json={"path": str(lib / "absent")}).status_code == 404
    assert client.post("/api/model-directories", json={"path": str(lib)}).json() == [str(lib)]
    assert client.post("/api/model-directories", json={"path": str(lib)}).json() == [str(lib)]          # no duplicates
    ids = [m["id"] for m in client.get("/api/library/models").json()]
    assert str(lib / "m1") in ids
    d = client.get("/api/dashboard").json()
    assert d["models"] >= 1 and d["presets"] > 0 and d["datasets"] >= 1 and d["jobs_total"] == 0
    info = client.get("/api/models/info", params={"path": str(lib / "m1")}).json()
    assert info["model_type"] == "qwen3" and info["num_layers"] == 2 and info["parameters"] is None and info["bytes"] > 0
    assert client.get("/api/models/info", params={"path": str(lib / "nothing")}).status_code == 404
    assert client.get("/api/models/info", params={"path": "random:tiny-qwen3"}).json()["model_type"] == "qwen3"
    dft = client.get("/api/models/defaults", params={"path": str(lib / "m1")}).json()
    assert "temperature" in dft["sampling"] and dft["training"]["lora_r"] == 16
    # deletion: only direct children of registered directories
    assert client.delete("/api/models", params={"path": str(tmp_path / "jobs")}).status_code == 403
    assert client.delete("/api/models", params={"path": str(lib)}).status_code == 403
    gone = client.delete("/api/models", params={"path": str(lib / "m1")}).json()
    assert gone["deleted"] == str(lib / "m1") and not (lib / "m1").exists()
    assert client.delete("/api/model-directories", params={"path": str(lib)}).json() == []


def test_parameter_count_comes_from_the_file_headers(tmp_path):
    import torch

    from pmetal_b200.gui.library import model_info
    from pmetal_b200.utils import safetensors_io as st
    (tmp_path / "config.json").write_text('{"model_type": "llama"}')
    st.save_file({"a": torch.zeros(3, 5), "b": torch.zeros(7)}, str(tmp_path / "model.safetensors"))
    assert model_info(str(tmp_path))["parameters"] == 22


def test_dataset_columns_adapters_and_merge_methods(client, tmp_path):
    (tmp_path / "qa.jsonl").write_text('{"question": "why", "answer": "so", "meta": {"k": 1}}\n{"question": "how", "extra": 3}\n')
    c = client.get("/api/datasets/columns", params={"path": str(tmp_path / "qa.jsonl")}).json()
    assert [x["name"] for x in c["columns"]] == ["question", "answer", "meta", "extra"] and c["rows_read"] == 2
    assert c["suggested_text_column"] == "question"
    (tmp_path / "t.csv").write_text("text,label\nhello,1\n")
    c = client.get("/api/datasets/columns", params={"path": str(tmp_path / "t.csv")}).json()
    assert c["suggested_text_column"] == "text" and c["columns"][1]["sample"] == "1"
    assert client.get("/api/datasets/columns", params={"path": str(tmp_path / "none.jsonl")}).status_code == 404
    run = tmp_path / "jobs" / "run1"
    run.mkdir()
    (run / "adapter_config.json").write_text('{"r": 8, "lora_alpha": 16, "base_model_name_or_path": "random:tiny-qwen3"}')
    ad = client.get("/api/adapters").json()
    assert ad and ad[0]["path"] == str(run) and ad[0]["r"] == 8
    methods = client.get("/api/merge-strategies").json()
    assert "ties" in methods and "slerp" in methods and len(methods) >= 16


def test_hub_routes_answer_without_a_network(client, monkeypatch):
    monkeypatch.setenv("HF_ENDPOINT", "http://127.0.0.1:9")            # nothing listens there
    assert client.get("/api/hub/models", params={"query": "qwen"}).status_code == 503
    r = client.post("/api/hub/download", json={"model": "org/name", "revision": "main"}).json()
    assert r["command"] == "download" and r["argv"] == ["download", "org/name", "--revision", "main"]
    assert client.post("/api/hub/download", json={}).status_code == 422
