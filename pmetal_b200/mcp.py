"""Model Context Protocol server over stdio exposing the framework as tools (crates/pmetal-mcp/src/lib.rs, jobs.rs).

JSON-RPC 2.0, one message per line: ``initialize``, ``tools/list``, ``tools/call``. Long-running tools (train, grpo,
distill, quantize, merge, serve) run as background jobs of the CLI in a subprocess: ``start_*`` returns a job id, and
``job_status`` / ``job_logs`` / ``job_cancel`` / ``list_jobs`` manage them; quick tools (info, memory, tokenize, eval,
infer, dataset_analyze, lr control) run inline. ``set_learning_rate`` and friends write the ``.lr_control.json`` file that
the training loop polls (crates/pmetal-trainer/src/adaptive_lr.rs:276-292)."""
from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile
import time
from typing import Any, Callable, Dict, List, Optional

PROTOCOL_VERSION = "2024-11-05"


class Job:
    def __init__(self, kind: str, argv: List[str]):
        self.id = f"{kind}-{int(time.time() * 1000) % 10 ** 10}"
        self.kind, self.argv = kind, argv
        self.log_path = os.path.join(tempfile.gettempdir(), f"pmetal-job-{self.id}.log")
        self._log = open(self.log_path, "w")
        self.proc = subprocess.Popen([sys.executable, "-m", "pmetal_b200.cli.main"] + argv, stdout=self._log,
                                     stderr=subprocess.STDOUT)
        self.started = time.time()

    def status(self) -> dict:
        rc = self.proc.poll()
        return {"id": self.id, "kind": self.kind, "state": "running" if rc is None else ("completed" if rc == 0 else "failed"),
                "exit_code": rc, "elapsed_s": round(time.time() - self.started, 1), "argv": self.argv}

    def logs(self, tail: int = 50) -> str:
        self._log.flush()
        with open(self.log_path, "r", errors="replace") as fh:
            return "".join(fh.readlines()[-tail:])

    def cancel(self) -> None:
        if self.proc.poll() is None:
            self.proc.terminate()


def _args_to_argv(args: Dict[str, Any]) -> List[str]:
    out: List[str] = []
    for k, v in args.items():
        flag = "--" + k.replace("_", "-")
        if isinstance(v, bool):
            if v:
                out.append(flag)
        elif isinstance(v, list):
            out.append(flag)
            out.extend(str(x) for x in v)
        elif v is not None:
            out.extend([flag, str(v)])
    return out


class McpServer:
    def __init__(self):
        self.jobs: Dict[str, Job] = {}
        self.tools: Dict[str, dict] = {}
        self._register()

    def tool(self, name: str, description: str, properties: Dict[str, dict], required: List[str], fn: Callable):
        self.tools[name] = {"description": description, "fn": fn,
                            "schema": {"type": "object", "properties": properties, "required": required}}

    def _job_tool(self, kind: str, description: str, required: List[str]):
        # the tool's input schema is the command's job specification (every flag with its type, default and help)
        from .core.jobs import job_specs
        if not hasattr(self, "_specs"):
            self._specs = job_specs()
        spec = self._specs.get(kind)
        props = dict(spec.json_schema()["properties"]) if spec else {}
        for r in required:
            props.setdefault(r, {"type": "string"})
        props["extra"] = {"type": "object", "description": "additional CLI flags, e.g. {\"max_steps\": 10}"}

        def start(args):
            flags = {k: v for k, v in args.items() if k != "extra"}
            flags.update(args.get("extra") or {})
            if spec is not None:
                try:
                    spec.validate(flags)
                except ValueError as e:
                    if "unknown field" not in str(e):      # unknown flags go through as they are; bad values are refused
                        raise
            job = Job(kind, [kind] + _args_to_argv(flags))
            self.jobs[job.id] = job
            return job.status()
        self.tool(f"start_{kind}", description, props, required, start)

    def _cli_inline(self, argv: List[str]) -> Any:
        r = subprocess.run([sys.executable, "-m", "pmetal_b200.cli.main"] + argv, stdout=subprocess.PIPE,
                           stderr=subprocess.PIPE, text=True)
        if r.returncode != 0:
            raise RuntimeError(r.stderr[-2000:] or f"exit code {r.returncode}")
        text = r.stdout.strip()
        for cand in (text, text.splitlines()[-1] if text else ""):      # one (possibly indented) document, or a last line
            try:
                return json.loads(cand)
            except json.JSONDecodeError:
                continue
        return {"output": r.stdout[-4000:]}

    def _register(self):
        s = {"type": "string"}
        self._job_tool("train", "LoRA / QLoRA / DoRA fine-tuning job", ["model", "dataset"])
        self._job_tool("grpo", "GRPO / DAPO reinforcement-learning job", ["model", "dataset"])
        self._job_tool("distill", "knowledge-distillation job", ["teacher", "student", "dataset"])
        self._job_tool("quantize", "GGUF / FP8 export job", ["model", "output"])
        self._job_tool("merge", "model-merge job", ["output"])
        self._job_tool("fuse", "merge a LoRA adapter into its base", ["model", "lora", "output"])
        self._job_tool("serve", "start the OpenAI-compatible server", ["model"])
        self.tool("list_jobs", "all jobs started by this server", {}, [], lambda a: [j.status() for j in self.jobs.values()])
        self.tool("job_status", "state of one job", {"id": s}, ["id"], lambda a: self.jobs[a["id"]].status())
        self.tool("job_logs", "tail of a job's log", {"id": s, "tail": {"type": "integer"}}, ["id"],
                  lambda a: {"log": self.jobs[a["id"]].logs(int(a.get("tail", 50)))})
        self.tool("job_cancel", "terminate a job", {"id": s}, ["id"],
                  lambda a: (self.jobs[a["id"]].cancel(), self.jobs[a["id"]].status())[1])
        self.tool("system_info", "devices, interconnect, library status", {}, [], lambda a: self._cli_inline(["info"]))
        self.tool("estimate_memory", "memory-fit estimate for a training configuration",
                  {"model": s, "seq_len": {"type": "integer"}, "batch_size": {"type": "integer"}}, ["model"],
                  lambda a: self._cli_inline(["memory", "-m", a["model"]] + _args_to_argv({k: v for k, v in a.items() if k != "model"})))
        self.tool("infer", "generate text", {"model": s, "prompt": s, "max_tokens": {"type": "integer"}, "lora": s},
                  ["model", "prompt"],
                  lambda a: self._cli_inline(["infer", "--json"] + _args_to_argv(a)))
        self.tool("evaluate", "loss / perplexity on a dataset", {"model": s, "dataset": s}, ["model", "dataset"],
                  lambda a: self._cli_inline(["eval"] + _args_to_argv(a)))
        self.tool("tokenize", "token ids of a text", {"model": s, "text": s}, ["model", "text"],
                  lambda a: self._cli_inline(["tokenize", "-m", a["model"], "--text", a["text"]]))
        self.tool("dataset_analyze", "format detection and length statistics", {"path": s}, ["path"],
                  lambda a: self._cli_inline(["dataset", "analyze", a["path"]]))

        def lr_cmd(cmd):
            def fn(a):
                path = os.path.join(a["output_dir"], ".lr_control.json")
                body = {"command": cmd, **{k: v for k, v in a.items() if k != "output_dir"}}
                with open(path, "w", encoding="utf-8") as fh:
                    json.dump(body, fh)
                return {"written": path, **body}
            return fn
        od = {"output_dir": s}
        self.tool("set_learning_rate", "set the LR of a running job", {**od, "lr": {"type": "number"}}, ["output_dir", "lr"], lr_cmd("set_lr"))
        self.tool("reduce_learning_rate", "multiply the LR of a running job", {**od, "factor": {"type": "number"}},
                  ["output_dir", "factor"], lr_cmd("reduce_lr"))
        self.tool("reset_learning_rate", "return to the schedule", od, ["output_dir"], lr_cmd("reset_lr"))
        self.tool("save_checkpoint_now", "ask a running job to checkpoint", od, ["output_dir"], lr_cmd("save_checkpoint"))
        self.tool("graceful_stop", "ask a running job to stop after the current step", od, ["output_dir"], lr_cmd("graceful_stop"))

        self._register_more()

    def _register_more(self):
        """The rest of the reference server's tool list (crates/pmetal-mcp/src/lib.rs:187-1400): model discovery,
        further job kinds, the dataset actions, benchmarks, packaging helpers and generic CLI access, under the
        reference's tool names; a few earlier tools are also reachable by the name the reference gives them."""
        s, i, b = {"type": "string"}, {"type": "integer"}, {"type": "boolean"}
        extra = {"extra": {"type": "object", "description": "additional CLI flags"}}

        def cli(name, description, argv_prefix, props, required, positional=()):
            def fn(a):
                flags = {k: v for k, v in a.items() if k not in positional and k != "extra"}
                flags.update(a.get("extra") or {})
                return self._cli_inline(list(argv_prefix) + [str(a[k]) for k in positional if k in a] + _args_to_argv(flags))
            self.tool(name, description, {**props, **extra}, required, fn)

        for alias, target in (("device_info", "system_info"), ("memory", "estimate_memory"), ("generate", "infer"),
                              ("stop_job", "job_cancel"), ("eval_perplexity", "evaluate"), ("quantize", "start_quantize"),
                              ("fuse_lora", "start_fuse"), ("merge_models", "start_merge"), ("train", "start_train"),
                              ("distill", "start_distill"), ("grpo", "start_grpo"), ("job_set_lr", "set_learning_rate"),
                              ("job_reduce_lr", "reduce_learning_rate"), ("job_reset_lr", "reset_learning_rate"),
                              ("job_save_checkpoint", "save_checkpoint_now"), ("job_graceful_stop", "graceful_stop")):
            self.tools[alias] = self.tools[target]
        self._job_tool("pretrain", "full-parameter pre-training job on token shards", ["model", "dataset"])
        self._job_tool("rlkd", "GRPO with a distillation term from a teacher", ["model", "teacher", "dataset"])
        self._job_tool("embed-train", "embedding fine-tuning job (InfoNCE / triplet / CoSENT)", ["model", "dataset"])
        for kind in ("pretrain", "rlkd"):
            self.tools[kind] = self.tools[f"start_{kind}"]
        self.tools["embed_train"] = self.tools["start_embed-train"]

        def start_cli_job(a):
            argv = [str(x) for x in a["argv"]]
            job = Job(argv[0] if argv else "cli", argv)
            self.jobs[job.id] = job
            return job.status()
        arr = {"type": "array", "items": s}
        self.tool("run_cli", "run any pmetal subcommand and return its output", {"argv": arr}, ["argv"],
                  lambda a: self._cli_inline([str(x) for x in a["argv"]]))
        self.tool("start_cli_job", "start any pmetal subcommand as a background job", {"argv": arr}, ["argv"], start_cli_job)
        cli("search_models", "search the local model cache (online: the hub)", ["search"], {"query": s, "limit": i, "online": b},
            [], ("query",))
        cli("list_local_models", "models in the local cache", ["search"], {"limit": i}, [])
        cli("download_model", "download a model from the hub", ["download"], {"model": s}, ["model"], ("model",))
        cli("model_fit", "does a model fit this device, and at what speed", ["memory"], {"model": s, "seq_len": i,
                                                                                      "batch_size": i, "quantization": s}, ["model"])

        def model_info(a):
            from .models.loader import resolve_model_path
            path = resolve_model_path(a["model"])
            cfg_path = os.path.join(path, "config.json")
            if not os.path.exists(cfg_path):
                return {"model": a["model"], "path": path, "config": None}
            with open(cfg_path, "r", encoding="utf-8") as fh:
                cfg = json.load(fh)
            from .models.architectures import family_of
            files = sorted(f for f in os.listdir(path) if f.endswith((".safetensors", ".gguf")))
            keys = ("model_type", "architectures", "hidden_size", "num_hidden_layers", "num_attention_heads",
                    "num_key_value_heads", "intermediate_size", "vocab_size", "max_position_embeddings", "num_experts",
                    "num_local_experts", "torch_dtype")
            return {"model": a["model"], "path": path, "family": family_of(cfg), "weight_files": files,
                    "bytes": sum(os.path.getsize(os.path.join(path, f)) for f in files),
                    "config": {k: cfg[k] for k in keys if k in cfg}}
        self.tool("model_info", "architecture, sizes and weight files of a local model", {"model": s}, ["model"], model_info)

        def chat(a):
            argv = ["infer", "--json", "--chat", "-m", a["model"], "-p", a["message"]]
            if a.get("system"):
                argv += ["--system", a["system"]]
            rest = {k: v for k, v in a.items() if k not in ("model", "message", "system")}
            return self._cli_inline(argv + _args_to_argv(rest))
        self.tool("chat", "one chat turn through the model's chat template",
                  {"model": s, "message": s, "system": s, "max_tokens": i, "lora": s}, ["model", "message"], chat)
        # ---- dataset actions
        io = {"input": s, "output": s}
        cli("dataset_preview", "first samples of a dataset file", ["dataset", "preview"], {"dataset_id": s, "num": i},
            ["dataset_id"], ("dataset_id",))
        cli("dataset_validate", "check a JSONL dataset for training", ["dataset", "validate"],
            {"path": s, "model": s, "max_seq_len": i}, ["path"], ("path",))
        cli("dataset_download", "download a dataset from the hub", ["dataset", "download"], {"dataset_id": s, "split": s,
                                                                                            "output": s}, ["dataset_id"], ("dataset_id",))
        cli("dataset_convert", "convert a dataset to training JSONL", ["dataset", "convert"],
            {"path": s, "output": s, "to": s, "columns": s, "shuffle": b}, ["path", "output"], ("path",))
        cli("dataset_filter", "filter by token count, pattern, duplicates, completeness", ["dataset", "filter"],
            {**io, "model": s, "min_tokens": i, "max_tokens": i, "dedup": b, "pattern": s, "invert": b, "complete_only": b},
            ["input", "output"])
        cli("dataset_split", "train / validation / test split", ["dataset", "split"],
            {"input": s, "output_dir": s, "val_ratio": {"type": "number"}, "test_ratio": {"type": "number"}, "seed": i,
             "stratify": s}, ["input", "output_dir"])

        def dataset_merge(a):
            argv = ["dataset", "merge", "-i"] + [str(x) for x in a["inputs"]]
            return self._cli_inline(argv + _args_to_argv({k: v for k, v in a.items() if k != "inputs"}))
        self.tool("dataset_merge", "merge several datasets", {"inputs": arr, "output": s, "shuffle": b, "interleave": b,
                                                             "weights": s, "seed": i}, ["inputs", "output"], dataset_merge)
        cli("dataset_sample", "random sample of a dataset", ["dataset", "sample"], {**io, "num": i, "seed": i},
            ["input", "output", "num"])
        cli("dataset_template", "apply a chat template", ["dataset", "template"],
            {**io, "template": s, "system": s, "model": s, "add_generation_prompt": b, "mask_prompt": b}, ["input", "output"])
        cli("dataset_prepare", "template + de-duplicate + length filter + split", ["dataset", "prepare"],
            {"dataset": s, "output_dir": s, "model": s, "template": s, "max_seq_len": i, "val_ratio": {"type": "number"},
             "columns": s}, ["dataset", "output_dir", "model"], ("dataset",))
        # ---- benchmarks, packaging
        cli("benchmark", "kernel corpus benchmark", ["bench", "corpus"], {"iters": i, "device": s}, [])
        cli("bench_corpus", "kernel corpus benchmark", ["bench", "corpus"], {"iters": i, "device": s}, [])
        cli("bench_train", "training-step workload benchmark", ["bench", "workload"], {"model": s, "iters": i}, [])
        cli("bench_gen", "generation benchmark", ["bench", "gen"], {"model": s, "iters": i}, [])
        cli("pack_experts", "write one file per MoE expert layer", ["pack-experts"], {"model": s, "output": s}, ["model", "output"])
        cli("dflash", "speculative decoding with a block-diffusion draft", ["dflash"], {"model": s, "draft": s, "prompt": s},
            ["model", "draft", "prompt"])
        cli("ollama_modelfile", "write an Ollama Modelfile", ["ollama", "modelfile"], {"gguf": s, "output": s, "template": s,
                                                                                   "system": s}, ["gguf"])
        cli("ollama_create", "write a Modelfile and print the ollama create command", ["ollama", "create"],
            {"name": s, "gguf": s, "output": s, "template": s, "system": s, "lora": s}, ["name", "gguf"])

    # ---------------------------------------------------------------- JSON-RPC
    def handle(self, msg: dict) -> Optional[dict]:
        mid, method, params = msg.get("id"), msg.get("method"), msg.get("params") or {}
        try:
            if method == "initialize":
                res = {"protocolVersion": PROTOCOL_VERSION, "capabilities": {"tools": {}},
                       "serverInfo": {"name": "pmetal-b200", "version": "0.1.0"}}
            elif method == "notifications/initialized":
                return None
            elif method == "ping":
                res = {}
            elif method == "tools/list":
                res = {"tools": [{"name": n, "description": t["description"], "inputSchema": t["schema"]}
                                 for n, t in self.tools.items()]}
            elif method == "tools/call":
                t = self.tools.get(params.get("name"))
                if t is None:
                    raise KeyError(f"unknown tool {params.get('name')!r}")
                args = params.get("arguments") or {}
                missing = [r for r in t["schema"]["required"] if r not in args]
                if missing:
                    raise ValueError(f"missing arguments: {missing}")
                out = t["fn"](args)
                res = {"content": [{"type": "text", "text": json.dumps(out)}], "isError": False}
            else:
                return {"jsonrpc": "2.0", "id": mid, "error": {"code": -32601, "message": f"method not found: {method}"}}
        except Exception as e:        # tool errors are results, protocol errors are errors
            if method == "tools/call":
                return {"jsonrpc": "2.0", "id": mid,
                        "result": {"content": [{"type": "text", "text": f"{type(e).__name__}: {e}"}], "isError": True}}
            return {"jsonrpc": "2.0", "id": mid, "error": {"code": -32603, "message": str(e)}}
        return {"jsonrpc": "2.0", "id": mid, "result": res} if mid is not None else None

    def serve_stdio(self, fin=None, fout=None) -> None:
        fin, fout = fin or sys.stdin, fout or sys.stdout
        for line in fin:
            line = line.strip()
            if not line:
                continue
            try:
                msg = json.loads(line)
            except json.JSONDecodeError:
                fout.write(json.dumps({"jsonrpc": "2.0", "id": None, "error": {"code": -32700, "message": "parse error"}}) + "\n")
                fout.flush()
                continue
            out = self.handle(msg)
            if out is not None:
                fout.write(json.dumps(out) + "\n")
                fout.flush()
        for j in self.jobs.values():
            j.cancel()


if __name__ == "__main__":
    McpServer().serve_stdio()
