"""Application state, key handling and drawing of the terminal front end.

State and rendering are separate from the terminal: ``TuiApp.handle_key`` mutates the state, ``TuiApp.render`` returns a
``rich`` renderable, and ``run`` is the only function that touches the tty. Tab set and behaviour follow the reference's
application (crates/pmetal/src/tui/tabs/mod.rs: System, Models, Datasets, one form per job kind, Monitor, Jobs); the
forms themselves come from ``core.jobs.job_specs``."""
from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .runner import Job, JobRunner

# (tab title, sub-command) of the form tabs, in display order
FORM_TABS: List[Tuple[str, str]] = [
    ("Tokenize", "tokenize"), ("Training", "train"), ("EmbedTrain", "embed-train"), ("Pretrain", "pretrain"),
    ("Distill", "distill"), ("RLKD", "rlkd"), ("GRPO", "grpo"), ("Inference", "infer"), ("DFlash", "dflash"),
    ("Serve", "serve"), ("Quantize", "quantize"), ("Merge", "merge"), ("Bench", "bench"), ("Eval", "eval"),
    ("Ollama", "ollama"),
]
TABS: List[str] = ["System", "Models", "Datasets"] + [t for t, _ in FORM_TABS] + ["Monitor", "Jobs"]
SPARK = "▁▂▃▄▅▆▇█"
HELP = [
    ("tab / shift-tab, ← →", "next / previous tab"),
    ("↑ ↓, j k, pgup pgdn", "move the selection"),
    ("enter", "edit a field, toggle a switch, cycle a choice; pick a model / dataset / job"),
    ("r", "run the form of this tab as a job (System tab: refresh)"),
    ("d", "reset the selected field to its default"),
    ("x", "cancel the selected job (Jobs tab)"),
    ("?", "this help"),
    ("q, ctrl-c", "quit (running jobs are cancelled)"),
]


def sparkline(values: List[float], width: int = 60) -> str:
    """Unicode block graph of the last ``width`` buckets of ``values`` (bucket mean), scaled to their own range."""
    vals = [v for v in values if v == v and abs(v) != float("inf")]
    if not vals:
        return ""
    if len(vals) > width:
        step = len(vals) / width
        buckets = [vals[int(i * step):max(int(i * step) + 1, int((i + 1) * step))] for i in range(width)]
        vals = [sum(b) / len(b) for b in buckets]
    lo, hi = min(vals), max(vals)
    span = (hi - lo) or 1.0
    return "".join(SPARK[min(len(SPARK) - 1, int((v - lo) / span * (len(SPARK) - 1) + 0.5))] for v in vals)


def scan_models(roots: Optional[List[str]] = None) -> List[Dict[str, str]]:
    """Models usable without a network: the built-in random presets, Hugging Face cache snapshots and local directories
    with a ``config.json``."""
    from ..models.config import PRESETS
    out = [{"id": f"random:{name}", "source": "preset", "path": ""} for name in sorted(PRESETS)]
    hub = os.path.join(os.environ.get("HF_HOME", os.path.expanduser("~/.cache/huggingface")), "hub")
    if os.path.isdir(hub):
        for d in sorted(os.listdir(hub)):
            if d.startswith("models--"):
                out.append({"id": d[len("models--"):].replace("--", "/"), "source": "cache", "path": os.path.join(hub, d)})
    for root in roots if roots is not None else [os.getcwd()]:
        if not os.path.isdir(root):
            continue
        for d in sorted(os.listdir(root)):
            p = os.path.join(root, d)
            if os.path.isfile(os.path.join(p, "config.json")):
                out.append({"id": p, "source": "local", "path": p})
    return out


def scan_datasets(roots: Optional[List[str]] = None, depth: int = 2) -> List[Dict[str, Any]]:
    """``.jsonl`` / ``.json`` / ``.parquet`` / ``.csv`` / ``.txt`` files under the given roots, at most ``depth`` levels down."""
    out: List[Dict[str, Any]] = []
    for root in roots if roots is not None else [os.getcwd(), os.path.expanduser("~/.cache/pmetal/datasets")]:
        if not os.path.isdir(root):
            continue
        base = root.rstrip(os.sep).count(os.sep)
        for dirpath, dirnames, files in os.walk(root):
            if dirpath.count(os.sep) - base >= depth:
                dirnames[:] = []
            dirnames[:] = [d for d in dirnames if not d.startswith(".") and d not in ("node_modules", "__pycache__")]
            for f in sorted(files):
                if f.endswith((".jsonl", ".parquet", ".csv")) or (f.endswith((".json", ".txt")) and "config" not in f):
                    p = os.path.join(dirpath, f)
                    try:
                        out.append({"path": p, "bytes": os.path.getsize(p)})
                    except OSError:
                        pass
    return out


def preview_dataset(path: str, limit: int = 600) -> str:
    try:
        if path.endswith(".parquet"):
            import pyarrow.parquet as pq
            t = pq.read_table(path)
            return f"{t.num_rows} rows; columns {t.column_names}\n" + json.dumps(t.slice(0, 1).to_pylist()[0], default=str)[:limit]
        with open(path, "r", encoding="utf-8", errors="replace") as fh:
            return fh.read(limit)
    except Exception as e:  # a preview never takes the application down
        return f"(cannot read: {e})"


@dataclass
class Form:
    """Editable values of one sub-command, generated from its :class:`~pmetal_b200.core.jobs.JobSpec`."""
    title: str
    spec: Any
    values: Dict[str, Any] = field(default_factory=dict)
    cursor: int = 0

    def fields(self):
        return [f for f in self.spec.fields if f.name not in ("func", "what")]

    def current(self):
        return self.fields()[self.cursor]

    def shown(self, f) -> str:
        v = self.values.get(f.name, f.default)
        if v is None:
            return ""
        if isinstance(v, (list, tuple)):
            return " ".join(str(x) for x in v)
        return str(v)

    def set_text(self, f, text: str) -> None:
        text = text.strip()
        if text == "":
            self.values.pop(f.name, None)
        elif f.kind == "integer":
            self.values[f.name] = int(text)
        elif f.kind == "number":
            self.values[f.name] = float(text)
        elif f.kind == "array":
            self.values[f.name] = text.split()
        else:
            self.values[f.name] = text

    def argv(self) -> List[str]:
        return self.spec.to_argv({k: v for k, v in self.values.items() if v is not None})


class TuiApp:
    def __init__(self, runner: Optional[JobRunner] = None, model_roots: Optional[List[str]] = None,
                 dataset_roots: Optional[List[str]] = None, system_info: Optional[dict] = None):
        from ..core.jobs import job_specs
        specs = job_specs()
        self.runner = runner or JobRunner()
        self.forms: Dict[str, Form] = {t: Form(t, specs[c]) for t, c in FORM_TABS if c in specs}
        self.tabs = [t for t in TABS if t in self.forms or t in ("System", "Models", "Datasets", "Monitor", "Jobs")]
        self.tab = 0
        self.cursor: Dict[str, int] = {"Models": 0, "Datasets": 0, "Jobs": 0}
        self.editing: Optional[str] = None           # text being edited for the form's current field
        self.status = "? for help"
        self.show_help = False
        self.quit = False
        self._model_roots, self._dataset_roots = model_roots, dataset_roots
        self.models = scan_models(model_roots)
        self.datasets = scan_datasets(dataset_roots)
        self._sysinfo = system_info
        self.monitor_job: Optional[Job] = None

    # ------------------------------------------------------------------ state helpers
    @property
    def tab_name(self) -> str:
        return self.tabs[self.tab]

    def goto(self, name: str) -> None:
        self.tab = self.tabs.index(name)

    def system_info(self) -> dict:
        if self._sysinfo is None:
            from ..utils.sysinfo import system_info
            try:
                self._sysinfo = system_info()
            except Exception as e:
                self._sysinfo = {"error": str(e)}
        return self._sysinfo

    def _fill(self, names: Tuple[str, ...], value: str) -> int:
        """Put ``value`` into the first field among ``names`` of every form that has one; returns how many were filled."""
        n = 0
        for form in self.forms.values():
            for f in form.fields():
                if f.name in names and f.kind == "string":
                    form.values[f.name] = value
                    n += 1
                    break
        return n

    def run_form(self, form: Form) -> Optional[Job]:
        try:
            argv = form.argv()
        except ValueError as e:
            self.status = f"cannot run: {e}"
            return None
        job = self.runner.start(form.spec.command, argv)
        self.monitor_job = job
        self.status = f"job {job.job_id} started: {' '.join(argv)}"
        self.goto("Monitor")
        return job

    # ------------------------------------------------------------------ keys
    def handle_key(self, key: str) -> None:
        if self.show_help:
            self.show_help = False
            return
        name = self.tab_name
        form = self.forms.get(name)
        if self.editing is not None and form is not None:
            return self._edit_key(form, key)
        if key in ("q", "ctrl-c"):
            self.quit = True
        elif key == "?":
            self.show_help = True
        elif key in ("tab", "right"):
            self.tab = (self.tab + 1) % len(self.tabs)
        elif key in ("backtab", "left"):
            self.tab = (self.tab - 1) % len(self.tabs)
        elif key in ("up", "k", "down", "j", "pageup", "pagedown", "home", "end"):
            self._move(key)
        elif form is not None:
            self._form_key(form, key)
        elif name == "System" and key == "r":
            self._sysinfo = None
            self.status = "system information refreshed"
        elif name == "Models":
            if key == "enter" and self.models:
                m = self.models[self.cursor["Models"]]
                n = self._fill(("model", "base", "base_model", "student", "target"), m["id"])
                self.status = f"model {m['id']} set in {n} forms"
            elif key == "r":
                self.models = scan_models(self._model_roots)
        elif name == "Datasets":
            if key == "enter" and self.datasets:
                d = self.datasets[self.cursor["Datasets"]]
                n = self._fill(("dataset", "data", "input"), d["path"])
                self.status = f"dataset {d['path']} set in {n} forms"
            elif key == "r":
                self.datasets = scan_datasets(self._dataset_roots)
        elif name == "Jobs" and self.runner.jobs:
            job = self.runner.jobs[min(self.cursor["Jobs"], len(self.runner.jobs) - 1)]
            if key == "enter":
                self.monitor_job = job
                self.goto("Monitor")
            elif key == "x":
                self.runner.cancel(job)
                self.status = f"job {job.job_id} cancelled"

    def _move(self, key: str) -> None:
        name = self.tab_name
        form = self.forms.get(name)
        n = len(form.fields()) if form else {"Models": len(self.models), "Datasets": len(self.datasets),
                                             "Jobs": len(self.runner.jobs)}.get(name, 0)
        if n == 0:
            return
        cur = form.cursor if form else self.cursor[name]
        cur = {"up": cur - 1, "k": cur - 1, "down": cur + 1, "j": cur + 1, "pageup": cur - 10, "pagedown": cur + 10,
               "home": 0, "end": n - 1}[key]
        cur = max(0, min(n - 1, cur))
        if form:
            form.cursor = cur
        else:
            self.cursor[name] = cur

    def _form_key(self, form: Form, key: str) -> None:
        f = form.current()
        if key == "enter":
            if f.kind == "boolean":
                form.values[f.name] = not bool(form.values.get(f.name, f.default))
            elif f.choices:
                opts = list(f.choices)
                cur = form.values.get(f.name, f.default)
                form.values[f.name] = opts[(opts.index(cur) + 1) % len(opts)] if cur in opts else opts[0]
            else:
                self.editing = form.shown(f)
        elif key == "d":
            form.values.pop(f.name, None)
        elif key == "r":
            self.run_form(form)

    def _edit_key(self, form: Form, key: str) -> None:
        f = form.current()
        if key == "enter":
            try:
                form.set_text(f, self.editing or "")
                self.status = f"{f.name} = {form.shown(f)!r}"
            except ValueError:
                self.status = f"{f.name} expects {f.kind}: {self.editing!r} rejected"
            self.editing = None
        elif key == "esc":
            self.editing = None
        elif key == "backspace":
            self.editing = (self.editing or "")[:-1]
        elif len(key) == 1:
            self.editing = (self.editing or "") + key

    def tick(self) -> None:
        """Called between key polls: follow the jobs."""
        self.runner.poll()

    # ------------------------------------------------------------------ drawing
    def render(self, height: int = 40):
        from rich.console import Group
        from rich.panel import Panel
        from rich.text import Text
        bar = Text()
        for i, t in enumerate(self.tabs):
            bar.append(f" {t} ", style="reverse bold" if i == self.tab else "dim")
        body_h = max(8, height - 6)
        if self.show_help:
            body = self._help()
        else:
            body = getattr(self, "_draw_" + ("form" if self.tab_name in self.forms else self.tab_name.lower()))(body_h)
        running = len(self.runner.running())
        foot = Text(f"{self.status}", style="bold")
        foot.append(f"   [{running} running / {len(self.runner.jobs)} jobs]", style="dim")
        return Group(bar, Panel(body, title=self.tab_name, height=body_h + 2), foot)

    def _help(self):
        from rich.table import Table
        t = Table.grid(padding=(0, 2))
        for k, what in HELP:
            t.add_row(k, what)
        return t

    @staticmethod
    def _window(cursor: int, n: int, rows: int) -> Tuple[int, int]:
        lo = max(0, min(cursor - rows // 2, n - rows))
        return lo, min(n, lo + rows)

    def _draw_form(self, rows: int):
        from rich.console import Group
        from rich.table import Table
        from rich.text import Text
        form = self.forms[self.tab_name]
        fields = form.fields()
        t = Table.grid(padding=(0, 2), expand=True)
        t.add_column(width=30)
        t.add_column(width=38)
        t.add_column(ratio=1)
        try:
            line = "pmetal " + " ".join(form.argv())
        except ValueError as e:
            line = str(e)
        head = Text("$ " + line, style="italic", no_wrap=True, overflow="ellipsis")
        lo, hi = self._window(form.cursor, len(fields), rows - 2)
        for i in range(lo, hi):
            f = fields[i]
            sel = i == form.cursor
            val = form.shown(f)
            if sel and self.editing is not None:
                val = self.editing + "▏"
            elif f.kind == "boolean":
                val = "[x]" if form.values.get(f.name, f.default) else "[ ]"
            label = ("* " if f.required else "  ") + (f.flags[-1] if f.flags else f"<{f.name}>")
            changed = f.name in form.values
            note = (f"{f.choices}  " if f.choices and sel else "") + (f.help or "")
            t.add_row(Text(label, style="reverse" if sel else "", no_wrap=True, overflow="ellipsis"),
                      Text(val, style="bold" if changed else "", no_wrap=True, overflow="ellipsis"),
                      Text(note, style="dim", no_wrap=True, overflow="ellipsis"))
        return Group(head, Text(""), t)

    def _draw_system(self, rows: int):
        from rich.table import Table
        info = self.system_info()
        t = Table.grid(padding=(0, 2))
        for k in ("torch", "cuda_available"):
            if k in info:
                t.add_row(k, str(info[k]))
        for d in info.get("devices", []):
            t.add_row(f"gpu {d['index']}", f"{d['name']}  {d['sms']} SMs  {d['memory_gib']} GiB  sm_{d['capability'].replace('.', '')}")
        if "nvlink_links_up" in info:
            t.add_row("nvlink links up", str(info["nvlink_links_up"]))
        nl = info.get("native_library") or {}
        if nl:
            t.add_row("native library", f"{nl.get('path')}  loaded={nl.get('loaded')}" + (f"  ({nl['error']})" if nl.get("error") else ""))
        for k, v in (info.get("measured_peaks") or {}).items():
            if isinstance(v, (int, float)):
                t.add_row(k, str(v))
        if "error" in info:
            t.add_row("error", info["error"])
        return t

    def _draw_list(self, items: List[str], cursor: int, rows: int):
        from rich.text import Text
        out = Text()
        lo, hi = self._window(cursor, len(items), rows)
        for i in range(lo, hi):
            out.append(items[i] + "\n", style="reverse" if i == cursor else "")
        return out

    def _draw_models(self, rows: int):
        if not self.models:
            return "no models found"
        return self._draw_list([f"{m['source']:7s} {m['id']}" for m in self.models], self.cursor["Models"], rows)

    def _draw_datasets(self, rows: int):
        from rich.console import Group
        from rich.text import Text
        if not self.datasets:
            return "no dataset files found under the working directory (r rescans)"
        half = max(3, rows // 2)
        cur = self.cursor["Datasets"]
        lst = self._draw_list([f"{d['bytes']:>12,d}  {d['path']}" for d in self.datasets], cur, half)
        return Group(lst, Text(preview_dataset(self.datasets[cur]["path"]), style="dim"))

    def _draw_jobs(self, rows: int):
        if not self.runner.jobs:
            return "no jobs yet: fill a form and press r"
        items = [f"{j.job_id:>3d}  {j.state:9s} {j.elapsed():8.1f}s  {j.command:12s} "
                 f"step {int(j.metrics.get('step', 0)):>6d}  loss {j.metrics.get('loss', float('nan')):.4f}  "
                 f"{' '.join(j.argv)[:70]}" for j in self.runner.jobs]
        return self._draw_list(items, min(self.cursor["Jobs"], len(items) - 1), rows)

    def _draw_monitor(self, rows: int):
        from rich.console import Group
        from rich.table import Table
        from rich.text import Text
        j = self.monitor_job or (self.runner.jobs[-1] if self.runner.jobs else None)
        if j is None:
            return "no job to follow: start one from a form (r), or pick one in the Jobs tab"
        t = Table.grid(padding=(0, 2))
        t.add_row("job", f"{j.job_id}  {j.command}  ({j.state})  {j.elapsed():.1f} s" +
                  (f"  exit code {j.returncode}" if j.returncode not in (None, 0) else ""))
        m = j.metrics
        total = next((int(j.argv[i + 1]) for i, a in enumerate(j.argv[:-1]) if a == "--max-steps" and j.argv[i + 1].isdigit()), 0)
        total = total or int(m.get("total_steps", 0))
        step = int(m.get("step", 0))
        if total:
            done = min(1.0, step / total)
            t.add_row("progress", f"{'█' * int(done * 40):<40s} {step}/{total}")
        elif step:
            t.add_row("step", str(step))
        for k, fmt in (("loss", "{:.4f}"), ("eval_loss", "{:.4f}"), ("lr", "{:.3e}"), ("grad_norm", "{:.3f}"),
                       ("tokens_per_s", "{:,.0f}"), ("reward", "{:.4f}"), ("kl", "{:.5f}")):
            if k in m:
                t.add_row(k, fmt.format(m[k]) + "  " + sparkline(j.history.get(k, []), 50))
        log = Text("\n".join(j.tail(max(3, rows - 12))), style="dim")
        return Group(t, Text(""), log)


def run(app: Optional[TuiApp] = None, refresh: float = 0.25, keys: Optional[List[str]] = None, console=None) -> int:
    """Interactive loop. With ``keys`` (a scripted key list) no terminal is needed: the keys are applied, jobs are followed
    until they end and the last frame is printed; this is what runs when stdin is not a tty."""
    from rich.console import Console
    from rich.live import Live
    from .term import RawTerminal, is_interactive
    app = app or TuiApp()
    console = console or Console()
    if keys is not None or not is_interactive():
        for k in keys or []:
            app.handle_key(k)
            app.tick()
        deadline = time.time() + 3600
        while app.runner.running() and time.time() < deadline:
            time.sleep(0.1)
            app.tick()
        console.print(app.render(console.size.height))
        return 0
    try:
        with RawTerminal() as term, Live(app.render(console.size.height), console=console, screen=True,
                                         auto_refresh=False) as live:
            while not app.quit:
                for k in term.read_keys(refresh):
                    app.handle_key(k)
                app.tick()
                live.update(app.render(console.size.height), refresh=True)
    finally:
        app.runner.shutdown()
    return 0
