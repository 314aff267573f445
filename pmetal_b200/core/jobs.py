"""Job specifications: one description of every sub-command's inputs, shared by the command line, the MCP server and any
form-based front end.

The reference derives per-field metadata from its ``*Spec`` structs with a proc-macro (``#[derive(JobSpec)]``,
crates/pmetal-core-derive/src/lib.rs:1-948; specs in crates/pmetal-core/src/jobs/*.rs) and generates ``to_argv()`` and
validation from it. Here the argparse definitions are the single source of truth: :func:`job_specs` introspects the
parser built by ``cli.main.build_parser`` and yields, per command, the field descriptors (name, flags, kind, default,
choices, help, required), a JSON schema, ``to_argv(values)`` and ``validate(values)``; ``parse(to_argv(v))`` gives back
``v`` (tested)."""
from __future__ import annotations

import argparse
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class FieldDescriptor:
    name: str                       # attribute name in the parsed namespace
    flags: List[str]                # option strings; empty for a positional
    kind: str                       # string | integer | number | boolean | array
    default: Any = None
    required: bool = False
    choices: Optional[List[Any]] = None
    help: str = ""
    label: str = ""

    def schema(self) -> dict:
        s: Dict[str, Any] = {"type": self.kind}
        if self.kind == "array":
            s["items"] = {"type": "string"}
        if self.choices:
            s["enum"] = list(self.choices)
        if self.help:
            s["description"] = self.help
        if self.default is not None and self.kind != "array":
            s["default"] = self.default
        return s


@dataclass
class JobSpec:
    command: str
    help: str = ""
    fields: List[FieldDescriptor] = field(default_factory=list)

    def field(self, name: str) -> FieldDescriptor:
        for f in self.fields:
            if f.name == name:
                return f
        raise KeyError(name)

    def json_schema(self) -> dict:
        return {"type": "object", "properties": {f.name: f.schema() for f in self.fields},
                "required": [f.name for f in self.fields if f.required]}

    def defaults(self) -> Dict[str, Any]:
        return {f.name: f.default for f in self.fields}

    def validate(self, values: Dict[str, Any]) -> Dict[str, Any]:
        """Type-coerced copy of ``values``; raises ``ValueError`` for unknown fields, missing required fields, values
        outside ``choices`` or of the wrong type."""
        out: Dict[str, Any] = {}
        known = {f.name: f for f in self.fields}
        for k, v in values.items():
            k = k.replace("-", "_")
            if k not in known:
                raise ValueError(f"{self.command}: unknown field {k!r}")
            f = known[k]
            if v is None:
                continue
            try:
                if f.kind == "integer":
                    if isinstance(v, bool) or (isinstance(v, float) and v != int(v)):
                        raise ValueError
                    v = int(v)
                elif f.kind == "number":
                    v = float(v)
                elif f.kind == "boolean":
                    if not isinstance(v, bool):
                        raise ValueError
                elif f.kind == "array":
                    v = [str(x) for x in (v if isinstance(v, (list, tuple)) else [v])]
                else:
                    v = str(v)
            except (TypeError, ValueError):
                raise ValueError(f"{self.command}: field {k!r} expects {f.kind}, got {v!r}") from None
            if f.choices and v not in f.choices:
                raise ValueError(f"{self.command}: field {k!r} must be one of {f.choices}, got {v!r}")
            out[k] = v
        missing = [f.name for f in self.fields if f.required and f.name not in out]
        if missing:
            raise ValueError(f"{self.command}: missing required field(s) {missing}")
        return out

    def to_argv(self, values: Dict[str, Any]) -> List[str]:
        """``[command, positionals..., --flag value ...]`` for validated values; defaults and false booleans are left out."""
        vals = self.validate(values)
        argv = self.command.split()
        tail: List[str] = []
        for f in self.fields:
            if f.name not in vals:
                continue
            v = vals[f.name]
            if not f.flags:
                argv.extend(v if isinstance(v, list) else [str(v)])
            elif f.kind == "boolean":
                if v:
                    tail.append(f.flags[-1])
            elif f.kind == "array":
                tail.append(f.flags[-1])
                tail.extend(v)
            elif v != f.default:
                tail.extend([f.flags[-1], str(v)])
        return argv + tail


def _kind(action: argparse.Action) -> str:
    if isinstance(action, (argparse._StoreTrueAction, argparse._StoreFalseAction)):
        return "boolean"
    if action.nargs in ("*", "+") or (isinstance(action.nargs, int) and action.nargs > 1):
        return "array"
    if action.type is int:
        return "integer"
    if action.type is float:
        return "number"
    return "string"


def _spec_of(command: str, parser: argparse.ArgumentParser, help_text: str) -> JobSpec:
    spec = JobSpec(command, help_text)
    for a in parser._actions:
        if isinstance(a, (argparse._HelpAction, argparse._SubParsersAction)) or a.nargs == argparse.REMAINDER:
            continue
        flags = sorted(a.option_strings, key=len)
        required = bool(a.required) if flags else a.nargs not in ("?", "*")
        spec.fields.append(FieldDescriptor(a.dest, flags, _kind(a), a.default if a.default is not argparse.SUPPRESS else None,
                                           required, list(a.choices) if a.choices else None, a.help or "",
                                           a.dest.replace("_", " ")))
    return spec


def job_specs() -> Dict[str, JobSpec]:
    """Command name (``"train"``, ``"dataset filter"``, ...) -> :class:`JobSpec`."""
    from ..cli.main import build_parser
    root = build_parser()
    out: Dict[str, JobSpec] = {}

    def walk(prefix: str, parser: argparse.ArgumentParser):
        subs = [a for a in parser._actions if isinstance(a, argparse._SubParsersAction)]
        if not subs:
            return
        helps = {c.dest: c.help for c in subs[0]._choices_actions}
        for name, sub in subs[0].choices.items():
            cmd = (prefix + " " + name).strip()
            out[cmd] = _spec_of(cmd, sub, helps.get(name) or "")
            walk(cmd, sub)
    walk("", root)
    return out


def job_spec(command: str) -> JobSpec:
    specs = job_specs()
    if command not in specs:
        raise KeyError(f"unknown command {command!r}; known: {sorted(specs)}")
    return specs[command]
