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
        props = {r: {"type": "string"} for r in required}
        props["extra"] = {"type": "object", "description": "additional CLI flags, e.g. {\"max_steps\": 10}"}

        def start(args):
            flags = {k: v for k, v in args.items() if k != "extra"}
            flags.update(args.get("extra") or {})
            job = Job(kind, [kind] + _args_to_argv(flags))
            self.jobs[job.id] = job
            return job.status()
        self.tool(f"start_{kind}", description, props, required, start)

    def _cli_inline(self, argv: List[str]) -> Any:
        r = subprocess.run([sys.executable, "-m", "pmetal_b200.cli.main"] + argv, stdout=subprocess.PIPE,
                           stderr=subprocess.PIPE, text=True)
        if r.returncode != 0:
            raise RuntimeError(r.stderr[-2000:] or f"exit code {r.returncode}")
        last = r.stdout.strip().splitlines()[-1] if r.stdout.strip() else ""
        try:
            return json.loads(last)
        except json.JSONDecodeError:
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
