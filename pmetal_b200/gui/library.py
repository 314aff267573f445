"""Library side of the browser front end: settings, model and dataset directories, model details, hub search and
downloads, dataset columns, merge methods and trained adapters.

The reference's desktop application answers these through window commands (crates/pmetal-gui/src-tauri/src/commands.rs:
get_config / set_config, get_dashboard_stats, get_model_info / get_model_defaults / delete_model,
add / remove / list_model_directories, search_hub_models, get_trending_models, get_model_fit, download_model,
search_hub_datasets, download_dataset, peek_dataset_columns, get_merge_strategies, list_trained_adapters). Here they are
HTTP routes registered on the job-runner application; job starts and stops of every kind go through ``/api/jobs``."""
from __future__ import annotations

import json
import os
import shutil
import threading
from typing import Any, Dict, List, Optional

DEFAULT_CONFIG = {"model_directories": [], "dataset_directories": [], "output_directory": "./output",
                  "default_lora_r": 16, "default_learning_rate": 2e-4, "default_max_seq_len": 2048, "theme": "dark"}


class Settings:
    """The application's settings as one JSON file; unknown keys are refused, missing ones take their defaults."""

    def __init__(self, path: str):
        self.path = path
        self._lock = threading.Lock()

    def load(self) -> Dict[str, Any]:
        cfg = dict(DEFAULT_CONFIG)
        try:
            with open(self.path, "r", encoding="utf-8") as fh:
                cfg.update({k: v for k, v in json.load(fh).items() if k in DEFAULT_CONFIG})
        except (OSError, ValueError):
            pass
        return cfg

    def update(self, patch: Dict[str, Any]) -> Dict[str, Any]:
        bad = [k for k in patch if k not in DEFAULT_CONFIG]
        if bad:
            raise KeyError(f"unknown settings: {', '.join(sorted(bad))}")
        for k, v in patch.items():
            want = type(DEFAULT_CONFIG[k])
            if want is float and isinstance(v, int) and not isinstance(v, bool):
                v = patch[k] = float(v)
            if not isinstance(v, want) or (want is not bool and isinstance(v, bool)):
                raise TypeError(f"{k}: {want.__name__} expected")
        with self._lock:
            cfg = self.load()
            cfg.update(patch)
            os.makedirs(os.path.dirname(os.path.abspath(self.path)), exist_ok=True)
            tmp = self.path + ".tmp"
            with open(tmp, "w", encoding="utf-8") as fh:
                json.dump(cfg, fh, indent=1)
            os.replace(tmp, self.path)
        return cfg


def dir_bytes(path: str) -> int:
    total = 0
    for dp, _, files in os.walk(path):
        for f in files:
            try:
                total += os.path.getsize(os.path.join(dp, f))       # follows the cache's links to the blobs
            except OSError:
                pass
    return total


def resolve_snapshot(path: str) -> str:
    """A hub cache entry (``models--org--name``) holds its files under ``snapshots/<revision>``."""
    snaps = os.path.join(path, "snapshots")
    if os.path.isdir(snaps):
        revs = sorted(os.listdir(snaps))
        if revs:
            return os.path.join(snaps, revs[-1])
    return path


def model_info(path: str) -> Dict[str, Any]:
    """Architecture, sizes and the parameter count of a model directory (or ``random:<preset>``)."""
    if path.startswith("random:"):
        from ..models.config import preset
        cfg = preset(path.split(":", 1)[1]).to_hf_dict()
        root, size = "", 0
    else:
        root = resolve_snapshot(path)
        with open(os.path.join(root, "config.json"), "r", encoding="utf-8") as fh:
            cfg = json.load(fh)
        size = dir_bytes(root)
    t = cfg.get("text_config") or cfg
    info = {"path": path, "model_type": cfg.get("model_type"), "architectures": cfg.get("architectures") or [],
            "hidden_size": t.get("hidden_size"), "num_layers": t.get("num_hidden_layers"),
            "num_attention_heads": t.get("num_attention_heads"), "num_key_value_heads": t.get("num_key_value_heads"),
            "vocab_size": t.get("vocab_size"), "max_position_embeddings": t.get("max_position_embeddings"),
            "num_experts": t.get("num_experts") or t.get("num_local_experts"), "bytes": size,
            "quantization": cfg.get("quantization") or cfg.get("quantization_config"),
            "has_tokenizer": bool(root) and os.path.exists(os.path.join(root, "tokenizer.json")),
            "has_chat_template": bool(root) and (os.path.exists(os.path.join(root, "chat_template.jinja")) or _has_template(root))}
    info["parameters"] = _count_parameters(root) if root else None
    return info


def _has_template(root: str) -> bool:
    try:
        with open(os.path.join(root, "tokenizer_config.json"), "r", encoding="utf-8") as fh:
            return bool(json.load(fh).get("chat_template"))
    except (OSError, ValueError):
        return False


def _count_parameters(root: str) -> Optional[int]:
    """From the safetensors headers only (no tensor is read)."""
    import struct
    total, seen = 0, False
    for f in sorted(os.listdir(root)):
        if not f.endswith(".safetensors") or "lora" in f or "adapter" in f:
            continue
        try:
            with open(os.path.join(root, f), "rb") as fh:
                n = struct.unpack("<Q", fh.read(8))[0]
                if n > (256 << 20):
                    continue
                head = json.loads(fh.read(n))
        except (OSError, ValueError, struct.error):
            continue
        for k, v in head.items():
            if k != "__metadata__":
                cnt = 1
                for d in v.get("shape", []):
                    cnt *= d
                total += cnt
                seen = True
    return total if seen else None


def model_defaults(path: str) -> Dict[str, Any]:
    """Sampling defaults of the model family / its generation_config.json, and the training defaults the forms start from."""
    from ..data.chat_templates import ChatTemplate
    from ..data.inference_config import load_sampling_defaults
    root = None if path.startswith("random:") else resolve_snapshot(path)
    ttype = None
    if root:
        try:
            ttype = ChatTemplate.from_model_dir(root).template_type
        except Exception:
            ttype = None
    d = load_sampling_defaults(root, ttype, "auto", False, use_preset=root is not None)
    return {"sampling": {k: getattr(d, k) for k in ("temperature", "top_k", "top_p", "min_p") if hasattr(d, k)},
            "chat_template": ttype,
            "training": {"lora_r": 16, "lora_alpha": 32.0, "learning_rate": 2e-4, "max_seq_len": 2048, "batch_size": 4}}


def peek_columns(path: str, rows: int = 20) -> Dict[str, Any]:
    """Column names (with a sample value each) from the head of a dataset file."""
    cols: Dict[str, Any] = {}
    n = 0
    if path.endswith(".parquet"):
        import pyarrow.parquet as pq
        t = pq.read_table(path).slice(0, rows)
        n = t.num_rows
        for name in t.column_names:
            vals = t.column(name).to_pylist()
            cols[name] = next((v for v in vals if v is not None), None)
    elif path.endswith(".csv"):
        import csv
        with open(path, "r", encoding="utf-8", newline="") as fh:
            for rec in csv.DictReader(fh):
                n += 1
                for k, v in rec.items():
                    cols.setdefault(k, v)
                if n >= rows:
                    break
    else:
        with open(path, "r", encoding="utf-8") as fh:
            head = fh.read(1)
            fh.seek(0)
            if head == "[":
                records = json.load(fh)[:rows]
            else:
                records = []
                for line in fh:
                    line = line.strip()
                    if line:
                        try:
                            records.append(json.loads(line))
                        except ValueError:
                            records.append({"text": line})
                    if len(records) >= rows:
                        break
        for rec in records:
            n += 1
            if isinstance(rec, dict):
                for k, v in rec.items():
                    cols.setdefault(k, v)
    short = lambda v: (v[:120] + "...") if isinstance(v, str) and len(v) > 120 else v
    guess = next((k for k in ("text", "prompt", "instruction", "question", "messages", "conversations") if k in cols), None)
    return {"path": path, "rows_read": n, "columns": [{"name": k, "type": type(v).__name__, "sample": short(v) if not isinstance(v, (list, dict)) else json.dumps(v)[:120]}
                                                      for k, v in cols.items()], "suggested_text_column": guess}


def list_adapters(roots: List[str], depth: int = 3) -> List[Dict[str, Any]]:
    """Directories with an ``adapter_config.json`` under the given roots (outputs of train / grpo / distill runs)."""
    out = []
    for root in roots:
        if not os.path.isdir(root):
            continue
        base = root.rstrip(os.sep).count(os.sep)
        for dp, dirnames, files in os.walk(root):
            if dp.count(os.sep) - base >= depth:
                dirnames[:] = []
            dirnames[:] = [d for d in dirnames if not d.startswith(".") and d != "__pycache__"]
            if "adapter_config.json" in files:
                try:
                    with open(os.path.join(dp, "adapter_config.json"), "r", encoding="utf-8") as fh:
                        c = json.load(fh)
                except (OSError, ValueError):
                    c = {}
                out.append({"path": dp, "base_model": c.get("base_model_name_or_path") or c.get("base_model"),
                            "r": c.get("r"), "alpha": c.get("lora_alpha") or c.get("alpha"),
                            "modified": os.path.getmtime(os.path.join(dp, "adapter_config.json"))})
    return sorted(out, key=lambda a: -a["modified"])


def register(app, runner, settings: Settings, model_roots: Optional[List[str]], dataset_roots: Optional[List[str]]) -> None:
    from fastapi import HTTPException

    from ..tui.app import scan_datasets, scan_models

    def roots() -> List[str]:
        return list(model_roots if model_roots is not None else [os.getcwd()]) + settings.load()["model_directories"]

    def managed(path: str) -> bool:
        """Only entries of the hub cache and of registered directories may be deleted."""
        real = os.path.realpath(path)
        hub = os.path.realpath(os.path.join(os.environ.get("HF_HOME", os.path.expanduser("~/.cache/huggingface")), "hub"))
        for base in [hub] + [os.path.realpath(r) for r in roots()]:
            if real != base and os.path.commonpath([real, base]) == base and os.path.dirname(real) == base:
                return True
        return False

    @app.get("/api/config")
    def get_config():
        return settings.load()

    @app.put("/api/config")
    def set_config(body: dict):
        try:
            return settings.update(body)
        except (KeyError, TypeError) as e:
            raise HTTPException(422, str(e).strip("'\"")) from None

    @app.get("/api/dashboard")
    def dashboard():
        runner.poll()
        states: Dict[str, int] = {}
        for j in runner.jobs:
            states[j.state] = states.get(j.state, 0) + 1
        models = scan_models(roots())
        return {"models": sum(1 for m in models if m["source"] != "preset"), "presets": sum(1 for m in models if m["source"] == "preset"),
                "datasets": len(scan_datasets(dataset_roots)), "adapters": len(list_adapters(roots() + [runner.workdir])),
                "jobs": states, "jobs_total": len(runner.jobs)}

    @app.get("/api/model-directories")
    def list_dirs():
        return settings.load()["model_directories"]

    @app.post("/api/model-directories")
    def add_dir(body: dict):
        path = os.path.abspath(os.path.expanduser(str(body.get("path") or "")))
        if not os.path.isdir(path):
            raise HTTPException(404, f"{path} is not a directory")
        dirs = settings.load()["model_directories"]
        if path not in dirs:
            dirs = settings.update({"model_directories": dirs + [path]})["model_directories"]
        return dirs

    @app.delete("/api/model-directories")
    def remove_dir(path: str):
        path = os.path.abspath(os.path.expanduser(path))
        dirs = [d for d in settings.load()["model_directories"] if d != path]
        return settings.update({"model_directories": dirs})["model_directories"]

    @app.get("/api/library/models")
    def library_models():
        return scan_models(roots())

    @app.get("/api/models/info")
    def info(path: str):
        try:
            return model_info(path)
        except (OSError, KeyError, ValueError) as e:
            raise HTTPException(404, f"{path}: {e}") from None

    @app.get("/api/models/defaults")
    def defaults(path: str):
        try:
            return model_defaults(path)
        except (OSError, KeyError, ValueError) as e:
            raise HTTPException(404, f"{path}: {e}") from None

    @app.get("/api/models/fit")
    def fit(model: str, seq_len: int = 2048, batch: int = 1, lora_r: int = 16, quantization: str = "none"):
        from ..utils.sysinfo import estimate_fit
        try:
            return estimate_fit(model, seq_len, batch, lora_r, quantization)
        except Exception as e:
            raise HTTPException(404, f"{model}: {e}") from None

    @app.delete("/api/models")
    def delete_model(path: str):
        if not os.path.isdir(path):
            raise HTTPException(404, f"{path} is not a directory")
        if not managed(path):
            raise HTTPException(403, "only entries of the hub cache and of registered model directories can be deleted")
        size = dir_bytes(path)
        shutil.rmtree(path)
        return {"deleted": path, "bytes": size}

    def _hub(fn, *a, **kw):
        from .. import hub
        try:
            return fn(hub, *a, **kw)
        except Exception as e:                       # no route to the hub is the normal case on an isolated machine
            raise HTTPException(503, f"hub not reachable: {e}") from None

    @app.get("/api/hub/models")
    def hub_models(query: str = "", limit: int = 20, tag: Optional[str] = None):
        rows = _hub(lambda h: h.search_models(query, limit, tag))
        return [r.__dict__ if hasattr(r, "__dict__") else r for r in rows]

    @app.get("/api/hub/trending")
    def hub_trending(limit: int = 20):
        rows = _hub(lambda h: h.search_models("", limit, None))        # the listing is sorted by downloads
        return [r.__dict__ if hasattr(r, "__dict__") else r for r in rows]

    @app.post("/api/hub/download")
    def hub_download(body: dict):
        repo = str(body.get("model") or "")
        if not repo:
            raise HTTPException(422, "model missing")
        argv = ["download", repo] + (["--revision", str(body["revision"])] if body.get("revision") else [])
        j = runner.start("download", argv)
        return {"id": j.job_id, "command": j.command, "argv": j.argv, "state": j.state}

    @app.get("/api/datasets/columns")
    def columns(path: str, rows: int = 20):
        try:
            return peek_columns(path, max(1, min(rows, 1000)))
        except (OSError, ValueError) as e:
            raise HTTPException(404, f"{path}: {e}") from None

    @app.get("/api/merge-strategies")
    def merge_strategies():
        from ..merge.methods import METHODS
        return list(METHODS)

    @app.get("/api/adapters")
    def adapters():
        return list_adapters(roots() + [runner.workdir, settings.load()["output_directory"]])
