"""Ollama Modelfile generation (crates/pmetal-models/src/ollama.rs, crates/pmetal/src/commands/ollama.rs:35-310; CLI
``ollama modelfile|create|templates``)."""
from __future__ import annotations

import os
from typing import Optional

TEMPLATES = {
    "chatml": "{{ if .System }}<|im_start|>system\n{{ .System }}<|im_end|>\n{{ end }}{{ if .Prompt }}<|im_start|>user\n"
              "{{ .Prompt }}<|im_end|>\n{{ end }}<|im_start|>assistant\n{{ .Response }}<|im_end|>\n",
    "llama3": "{{ if .System }}<|start_header_id|>system<|end_header_id|>\n\n{{ .System }}<|eot_id|>{{ end }}"
              "{{ if .Prompt }}<|start_header_id|>user<|end_header_id|>\n\n{{ .Prompt }}<|eot_id|>{{ end }}"
              "<|start_header_id|>assistant<|end_header_id|>\n\n{{ .Response }}<|eot_id|>",
    "mistral": "[INST] {{ if .System }}{{ .System }} {{ end }}{{ .Prompt }} [/INST]{{ .Response }}</s>",
    "gemma": "<start_of_turn>user\n{{ if .System }}{{ .System }} {{ end }}{{ .Prompt }}<end_of_turn>\n<start_of_turn>model\n"
             "{{ .Response }}<end_of_turn>\n",
    "phi3": "{{ if .System }}<|system|>\n{{ .System }}<|end|>\n{{ end }}<|user|>\n{{ .Prompt }}<|end|>\n<|assistant|>\n"
            "{{ .Response }}<|end|>\n",
    "alpaca": "{{ if .System }}{{ .System }}\n\n{{ end }}### Instruction:\n{{ .Prompt }}\n\n### Response:\n{{ .Response }}",
}
STOPS = {"chatml": ["<|im_end|>", "<|im_start|>"], "llama3": ["<|eot_id|>", "<|start_header_id|>"], "mistral": ["</s>", "[INST]"],
         "gemma": ["<end_of_turn>"], "phi3": ["<|end|>", "<|user|>"], "alpaca": ["### Instruction:"]}


TEMPLATES["qwen3"] = TEMPLATES["chatml"]
TEMPLATES["deepseek"] = ("{{ if .System }}{{ .System }}\n\n{{ end }}{{ if .Prompt }}User: {{ .Prompt }}\n\n{{ end }}"
                         "Assistant: {{ .Response }}<｜end▁of▁sentence｜>")
STOPS["qwen3"] = STOPS["chatml"]
STOPS["deepseek"] = ["<｜end▁of▁sentence｜>", "User:"]


def detect_template(model_name: str) -> str:
    """Template by model name (llama / qwen / gemma / mistral / phi / deepseek), ChatML otherwise."""
    n = model_name.lower()
    for key, tpl in (("llama", "llama3"), ("qwen", "qwen3"), ("gemma", "gemma"), ("mistral", "mistral"),
                     ("mixtral", "mistral"), ("phi", "phi3"), ("deepseek", "deepseek")):
        if key in n:
            return tpl
    return "chatml"


def validate_model_name(name: str) -> str:
    """Ollama model names: ``[namespace/]model[:tag]`` of letters, digits, ``._-``; anything else is refused so the
    printed ``ollama create`` command cannot be turned into another command."""
    import re
    if not name or len(name) > 128 or not re.fullmatch(r"[A-Za-z0-9][A-Za-z0-9._-]*(/[A-Za-z0-9][A-Za-z0-9._-]*)?(:[A-Za-z0-9._-]+)?", name):
        raise ValueError(f"invalid Ollama model name {name!r}")
    return name


def modelfile_text(gguf_path: str, template: str = "chatml", system: Optional[str] = None, adapter: Optional[str] = None,
                   license: Optional[str] = None, **params) -> str:
    if template not in TEMPLATES:
        raise ValueError(f"unknown template {template!r}; choose from {sorted(TEMPLATES)}")
    lines = [f"FROM {gguf_path}"]
    if adapter:
        lines.append(f"ADAPTER {adapter}")
    lines.append(f'TEMPLATE """{TEMPLATES[template]}"""')
    if system:
        lines.append(f'SYSTEM """{system}"""')
    for k, v in params.items():
        if v is not None:
            lines.append(f"PARAMETER {k} {v}")
    lines.extend(f'PARAMETER stop "{s}"' for s in STOPS[template])
    if license:
        lines.append(f'LICENSE """{license}"""')
    return "\n".join(lines) + "\n"


def write_modelfile(gguf_path: str, out_path: str = "Modelfile", template: str = "chatml", system: Optional[str] = None,
                    adapter: Optional[str] = None, license: Optional[str] = None, **params) -> str:
    with open(out_path, "w", encoding="utf-8") as fh:
        fh.write(modelfile_text(os.path.abspath(gguf_path), template, system,
                                os.path.abspath(adapter) if adapter else None, license, **params))
    return out_path
