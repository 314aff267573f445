"""Terminal application: key decoding, form editing from the job specifications, job runner and monitor drawing."""
import json
import os
import sys
import time

import pytest

from pmetal_b200.tui.app import TuiApp, run, scan_datasets, sparkline
from pmetal_b200.tui.runner import JobRunner
from pmetal_b200.tui.term import decode_keys


def _text(app, width=160, height=44):
    from rich.console import Console
    c = Console(record=True, width=width, height=height, force_terminal=False)
    c.print(app.render(height))
    return c.export_text()


def test_decode_keys():
    assert decode_keys("a\x1b[A\x1b[B\t\x1b[Z\r\x7f\x1bq\x03") == \
        ["a", "up", "down", "tab", "backtab", "enter", "backspace", "esc", "q", "ctrl-c"]
    assert decode_keys("\x1b[5~\x1bOC") == ["pageup", "right"]


def test_sparkline_scales_and_buckets():
    s = sparkline([float(i) for i in range(200)], width=20)
    assert len(s) == 20 and s[0] == "▁" and s[-1] == "█"
    assert sparkline([]) == "" and sparkline([float("nan")]) == ""


def test_forms_follow_the_job_specs_and_edit(tmp_path):
    (tmp_path / "data").mkdir()
    (tmp_path / "data" / "train.jsonl").write_text(json.dumps({"text": "hello"}) + "\n")
    app = TuiApp(runner=JobRunner(workdir=str(tmp_path)), model_roots=[], dataset_roots=[str(tmp_path)], system_info={})
    assert app.tabs[:3] == ["System", "Models", "Datasets"] and app.tabs[-2:] == ["Monitor", "Jobs"]
    assert {"Training", "Pretrain", "GRPO", "Inference", "Serve", "Quantize", "Merge"} <= set(app.forms)
    # pick a model and a dataset: they land in the forms
    app.goto("Models")
    assert any(m["id"] == "random:tiny-qwen3" for m in app.models)
    app.cursor["Models"] = next(i for i, m in enumerate(app.models) if m["id"] == "random:tiny-qwen3")
    app.handle_key("enter")
    app.goto("Datasets")
    assert "train.jsonl" in _text(app) and "hello" in _text(app)
    app.handle_key("enter")
    form = app.forms["Training"]
    assert form.values["model"] == "random:tiny-qwen3" and form.values["dataset"].endswith("train.jsonl")
    # edit an integer field by typing, reject a bad value, toggle a switch, cycle a choice
    app.goto("Training")
    names = [f.name for f in form.fields()]
    form.cursor = names.index("max_steps")
    for k in ["enter", "backspace", "backspace", "backspace", "7", "enter"]:
        app.handle_key(k)
    assert form.values["max_steps"] == 7
    for k in ["enter", "x", "enter"]:
        app.handle_key(k)
    assert form.values["max_steps"] == 7 and "rejected" in app.status
    form.cursor = names.index("use_rslora")
    app.handle_key("enter")
    assert form.values["use_rslora"] is True
    form.cursor = names.index("quantization")
    first = form.current().default
    app.handle_key("enter")
    assert form.values["quantization"] in form.current().choices and form.values["quantization"] != first
    argv = form.argv()
    assert argv[0] == "train" and "--max-steps" in argv and "--use-rslora" in argv
    txt = _text(app)
    assert "pmetal train" in txt and "--max-steps" in txt
    app.handle_key("?")
    assert "cancel the selected job" in _text(app)
    app.handle_key("x")                      # any key closes the help
    assert not app.show_help
    app.handle_key("q")
    assert app.quit


def test_missing_required_field_is_reported(tmp_path):
    app = TuiApp(runner=JobRunner(workdir=str(tmp_path)), model_roots=[], dataset_roots=[], system_info={})
    app.goto("Quantize")
    app.handle_key("r")
    assert app.status.startswith("cannot run") and not app.runner.jobs


FAKE_CLI = r'''
import json, sys, time
ev = sys.argv[sys.argv.index("--log-events") + 1]
with open(ev, "w") as fh:
    fh.write(json.dumps({"event": "started", "job_id": "j", "kind": "train"}) + "\n")
    for s in range(1, 6):
        fh.write(json.dumps({"event": "metric", "job_id": "j", "payload": {"step": s, "loss": 3.0 / s, "lr": 1e-4}}) + "\n")
        fh.flush()
        print("step", s, flush=True)
    if "--hang" in sys.argv:
        time.sleep(60)
sys.exit(3 if "--fail" in sys.argv else 0)
'''


@pytest.fixture
def fake_runner(tmp_path):
    pkg = tmp_path / "fakecli"
    pkg.mkdir()
    (pkg / "__init__.py").write_text("")
    (pkg / "__main__.py").write_text(FAKE_CLI)
    old = os.environ.get("PYTHONPATH")
    os.environ["PYTHONPATH"] = str(tmp_path) + (os.pathsep + old if old else "")
    yield JobRunner(workdir=str(tmp_path / "jobs-out") if (tmp_path / "jobs-out").mkdir() is None else None,
                    python=sys.executable, module="fakecli")
    if old is None:
        os.environ.pop("PYTHONPATH")
    else:
        os.environ["PYTHONPATH"] = old


def _wait(runner, timeout=30.0):
    end = time.time() + timeout
    while runner.running() and time.time() < end:
        time.sleep(0.05)
        runner.poll()
    runner.poll()


def test_runner_follows_events_and_exit_codes(fake_runner):
    ok = fake_runner.start("train", ["train", "--max-steps", "5"])
    bad = fake_runner.start("train", ["train", "--fail"])
    _wait(fake_runner)
    assert ok.state == "finished" and ok.metrics["step"] == 5 and ok.history["loss"] == [3.0 / s for s in range(1, 6)]
    assert bad.state == "failed" and bad.returncode == 3
    assert ok.tail(2) == ["step 4", "step 5"]


def test_runner_cancels_only_its_own_process_group(fake_runner):
    job = fake_runner.start("train", ["train", "--hang"])
    end = time.time() + 30
    while job.metrics.get("step") != 5 and time.time() < end:
        time.sleep(0.05)
        fake_runner.poll()
    fake_runner.cancel(job, grace=5.0)
    assert job.state == "cancelled" and job.proc.poll() is not None


def test_run_form_monitor_and_jobs_tab(fake_runner, tmp_path):
    app = TuiApp(runner=fake_runner, model_roots=[], dataset_roots=[], system_info={"torch": "x", "devices": []})
    form = app.forms["Training"]
    form.values.update(model="random:tiny-qwen3", dataset="d.jsonl", max_steps=5)
    app.goto("Training")
    app.handle_key("r")
    assert app.tab_name == "Monitor" and len(fake_runner.jobs) == 1
    _wait(fake_runner)
    txt = _text(app)
    assert "finished" in txt and "5/5" in txt and "loss" in txt and "step 5" in txt
    app.goto("Jobs")
    assert "finished" in _text(app) and "train" in _text(app)
    app.handle_key("enter")
    assert app.tab_name == "Monitor"


def test_scripted_run_prints_a_frame(tmp_path, capsys):
    from rich.console import Console
    app = TuiApp(runner=JobRunner(workdir=str(tmp_path)), model_roots=[], dataset_roots=[], system_info={"torch": "t"})
    c = Console(record=True, width=140, height=40)
    assert run(app, keys=["tab", "tab", "tab"], console=c) == 0
    assert app.tab_name == "Tokenize" and "Tokenize" in c.export_text()


def test_scan_datasets_respects_depth(tmp_path):
    d = tmp_path / "a" / "b" / "c"
    d.mkdir(parents=True)
    (tmp_path / "top.jsonl").write_text("{}\n")
    (d / "deep.jsonl").write_text("{}\n")
    found = [os.path.basename(x["path"]) for x in scan_datasets([str(tmp_path)], depth=2)]
    assert "top.jsonl" in found and "deep.jsonl" not in found


def test_training_job_through_the_real_command_line(tmp_path):
    """A form launches the actual command line as a child process and the monitor shows its per-step metric events."""
    data = tmp_path / "d.jsonl"
    data.write_text("".join(json.dumps({"text": "hello world " * 8}) + "\n" for _ in range(16)))
    app = TuiApp(runner=JobRunner(workdir=str(tmp_path)), model_roots=[], dataset_roots=[str(tmp_path)], system_info={})
    app.forms["Training"].values.update(model="random:tiny-llama", dataset=str(data), max_steps=3,
                                        output=str(tmp_path / "out"), device="cpu", dtype="float32")
    app.goto("Training")
    app.handle_key("r")
    _wait(app.runner, timeout=240.0)
    job = app.runner.jobs[0]
    assert job.state == "finished", "\n".join(job.tail(30))
    assert job.metrics["step"] == 3 and job.metrics["total_steps"] == 3 and len(job.history["loss"]) == 3
    txt = _text(app)
    assert "3/3" in txt and "grad_norm" in txt and os.path.exists(tmp_path / "out" / "lora_weights.safetensors")


def test_interactive_loop_on_a_pseudo_terminal(tmp_path):
    """The real loop: raw-mode key reading and full-screen drawing on a pty; tab twice, open and close the help, quit."""
    import pty
    import select
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    master, slave = pty.openpty()
    env = dict(os.environ, TERM="xterm-256color", COLUMNS="140", LINES="40")
    p = subprocess.Popen([sys.executable, "-m", "pmetal_b200.cli.main", "tui", "--workdir", str(tmp_path)], cwd=root,
                         stdin=slave, stdout=slave, stderr=subprocess.PIPE, env=env, start_new_session=True)
    os.close(slave)
    seen = b""

    def pump(seconds):
        nonlocal seen
        end = time.time() + seconds
        while time.time() < end:
            r, _, _ = select.select([master], [], [], 0.2)
            if r:
                try:
                    chunk = os.read(master, 65536)
                except OSError:
                    return
                if not chunk:
                    return
                seen += chunk

    try:
        deadline = time.time() + 90
        while b"System" not in seen and time.time() < deadline and p.poll() is None:
            pump(0.5)
        assert b"System" in seen and b"Training" in seen, (seen[-500:], p.stderr.read()[-2000:] if p.poll() is not None else b"")
        for key in (b"\t", b"\t", b"?"):
            os.write(master, key)
            pump(0.8)
        assert b"cancel the selected job" in seen              # the help page was drawn
        os.write(master, b"x")                                  # any key closes it
        pump(0.5)
        os.write(master, b"q")
        end = time.time() + 30
        while p.poll() is None and time.time() < end:
            pump(0.3)
        assert p.poll() == 0, p.stderr.read()[-2000:]
    finally:
        if p.poll() is None:
            p.kill()
            p.wait()
        os.close(master)
