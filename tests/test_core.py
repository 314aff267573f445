import json
import math
import os

import pytest
import torch

from pmetal_b200.core.config import FullTrainingConfig, LoraConfig, TrainingConfig
from pmetal_b200.core.events import JobEvent, JobStatus, JsonlSink
from pmetal_b200.core.scheduler import LearningRateScheduler


def test_config_defaults_match_reference():
    t, l = TrainingConfig(), LoraConfig()
    assert (t.learning_rate, t.batch_size, t.gradient_accumulation_steps, t.num_epochs) == (2e-4, 1, 4, 3)
    assert (t.warmup_steps, t.weight_decay, t.max_grad_norm, t.lr_scheduler, t.seed) == (100, 0.01, 1.0, "cosine", 42)
    assert (l.r, l.alpha, l.target_modules) == (16, 32.0, ["q_proj", "k_proj", "v_proj", "o_proj"])
    assert l.scaling() == 2.0
    assert LoraConfig(r=16, alpha=32, use_rslora=True).scaling() == 8.0
    assert LoraConfig(r=0).scaling() == 0.0


def test_yaml_roundtrip(tmp_path):
    p = tmp_path / "c.yaml"
    p.write_text("model:\n  model_id: m\nlora:\n  r: 8\ntraining:\n  learning_rate: 0.001\ndataset:\n  dataset_id: d.jsonl\n")
    c = FullTrainingConfig.from_yaml(str(p))
    assert c.model.model_id == "m" and c.lora.r == 8 and c.training.learning_rate == 1e-3
    assert c.dataset.dataset_id == "d.jsonl" and c.training.warmup_steps == 100


def test_scheduler_shapes():
    s = LearningRateScheduler(1.0, 100, 10, "cosine")
    assert s.get_lr(0) == 0.0 and s.get_lr(5) == 0.5 and s.get_lr(10) == 1.0
    assert abs(s.get_lr(55) - 0.5) < 1e-12 and s.get_lr(100) < 1e-12 and s.get_lr(1000) < 1e-12
    lin = LearningRateScheduler(1.0, 100, 0, "linear", min_lr=0.1)
    assert abs(lin.get_lr(50) - 0.55) < 1e-12
    wsd = LearningRateScheduler(1.0, 110, 10, "wsd", stable_ratio=0.7)
    assert wsd.get_lr(10 + 69) == 1.0 and wsd.get_lr(10 + 70) == 1.0 and abs(wsd.get_lr(10 + 85) - 0.5) < 1e-12
    rs = LearningRateScheduler(1.0, 100, 0, "cosine_with_restarts", num_restarts=2)
    assert rs.get_lr(0) == 1.0 and rs.get_lr(50) == 1.0 and rs.get_lr(25) == 0.5
    poly = LearningRateScheduler(1.0, 100, 0, "polynomial", polynomial_power=2.0)
    assert abs(poly.get_lr(50) - 0.25) < 1e-12
    assert LearningRateScheduler(0.3, 10, 0, "constant").get_lr(7) == 0.3


def test_job_events(tmp_path):
    p = tmp_path / "ev.jsonl"
    sink = JsonlSink(str(p))
    evs = [JobEvent.started("j", "train"), JobEvent.phase("j", "training"),
           JobEvent.metric("j", "step", step=1, loss=2.0), JobEvent.completed("j", steps=1)]
    for e in evs:
        sink.emit(e)
    sink.close()
    lines = [JobEvent.from_json(l) for l in p.read_text().splitlines()]
    assert lines[0]["event"] == "started" and lines[0]["kind"] == "train"
    assert lines[1]["phase"] == {"phase": "training"}
    st = JobStatus.fold(lines)
    assert st.state == "completed" and st.phase == "training" and st.last_metric["loss"] == 2.0
    assert JobStatus.fold([JobEvent.started("j", "train"), JobEvent.failed("j", "boom")]).error == "boom"


def test_tensorboard_callback_writes_event_file(tmp_path):
    import os

    import pytest
    pytest.importorskip("tensorboard")
    from pmetal_b200.core.callbacks import StepMetrics, TensorBoardCallback
    cb = TensorBoardCallback(str(tmp_path / "tb"))
    for i in range(3):
        cb.on_step_end_with_metrics(StepMetrics(step=i + 1, total_steps=3, loss=2.0 - i * 0.1, lr=1e-4, tok_sec=100.0, grad_norm=0.5))
    cb.on_eval({"loss": 1.5, "perplexity": 4.48})
    cb.on_train_end()
    files = os.listdir(tmp_path / "tb")
    assert any(f.startswith("events.out.tfevents") for f in files)
    assert os.path.getsize(os.path.join(tmp_path / "tb", files[0])) > 100


def test_job_specs_describe_every_command_and_round_trip():
    from pmetal_b200.cli.main import build_parser
    from pmetal_b200.core.jobs import job_spec, job_specs
    specs = job_specs()
    for cmd in ("train", "infer", "serve", "grpo", "distill", "quantize", "merge", "fuse", "pretrain", "embed-train", "eval",
                "tokenize", "dflash", "rlkd", "pack-experts", "bench", "dataset filter", "dataset prepare"):
        assert cmd in specs and specs[cmd].fields, cmd
    t = job_spec("train")
    f = t.field("lora_r")
    assert (f.kind, f.default, f.flags) == ("integer", 16, ["--lora-r"]) and t.field("use_dora").kind == "boolean"
    assert t.json_schema()["properties"]["quantization"]["enum"] == ["none", "nf4", "fp4", "int8"]
    vals = {"model": "m", "dataset": "d.jsonl", "lora_r": 8, "use_dora": True, "learning_rate": 1e-4, "max_steps": 3}
    ns = build_parser().parse_args(t.to_argv(vals))
    for k, v in vals.items():
        assert getattr(ns, k) == v
    g = job_spec("dataset merge")
    ns = build_parser().parse_args(g.to_argv({"inputs": ["a", "b"], "output": "o", "shuffle": True}))
    assert ns.inputs == ["a", "b"] and ns.output == "o" and ns.shuffle
    for bad in ({"model": "m", "dataset": "d", "lora_r": "eight"}, {"model": "m", "dataset": "d", "quantization": "q3"},
                {"model": "m", "dataset": "d", "bogus": 1}, {"model": "m", "dataset": "d", "use_dora": "yes"}):
        with pytest.raises(ValueError):
            t.validate(bad)
    with pytest.raises(ValueError):
        job_spec("fuse").validate({"model": "m"})                       # --lora and --output are required
    with pytest.raises(KeyError):
        job_spec("nope")


def test_cli_log_file_with_rotation(tmp_path, monkeypatch):
    import logging

    from pmetal_b200.cli.main import setup_logging
    log = tmp_path / "logs" / "cli.log"
    monkeypatch.setenv("PMETAL_LOG_FILE", str(log))
    assert setup_logging() == str(log)
    logging.getLogger("pmetal").info("first run")
    log_size = os.path.getsize(log)
    assert log_size > 0
    with open(log, "ab") as fh:
        fh.write(b"x" * (9 << 20))
    assert setup_logging() == str(log)                                    # re-initialising rotates the oversized file
    logging.getLogger("pmetal").info("second run")
    assert os.path.getsize(str(log) + ".1") > 9 << 20 and b"second run" in open(log, "rb").read()
    monkeypatch.setenv("PMETAL_LOG_FILE", "off")
    assert setup_logging() is None
    monkeypatch.setenv("PMETAL_LOG_FILE", "/proc/definitely/not/writable/cli.log")
    assert setup_logging() is None
    monkeypatch.setenv("PMETAL_LOG_FILE", "off")
    setup_logging()


def test_nvtx_ranges_are_inert_without_a_device():
    from pmetal_b200.utils import nvtx
    nvtx.set_enabled(False)
    with nvtx.range("phase"):
        nvtx.mark("point")
    assert not nvtx.enabled()
