"""Chat templates: hard-coded formats for the common model families plus execution of a
model's own Jinja template from ``tokenizer_config.json``.

Mirrors crates/pmetal-data/src/chat_templates.rs:247-600 (17 template types with per-type end
tokens; ``apply`` returns the text and the offset where the last assistant response begins so
SFT can mask the prompt) and jinja_chat.rs:110 (Jinja rendering, tools passed through).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

TEMPLATE_TYPES = ("chatml", "llama2", "llama3", "llama4", "mistral", "gemma", "gemma4", "phi3", "phi4", "qwen",
                  "alpaca", "vicuna", "zephyr", "gpt_oss", "deepseek", "cohere", "custom")

EOS = {
    "chatml": "<|im_end|>", "qwen": "<|im_end|>", "custom": "<|im_end|>", "llama2": "</s>", "llama3": "<|eot_id|>",
    "llama4": "<|eot|>", "mistral": "</s>", "gemma": "<end_of_turn>", "gemma4": "<turn|>", "phi3": "<|end|>",
    "phi4": "<|im_end|>", "alpaca": "</s>", "vicuna": "</s>", "zephyr": "</s>", "gpt_oss": "<|return|>",
    "deepseek": "<｜end▁of▁sentence｜>", "cohere": "<|END_OF_TURN_TOKEN|>",
}


@dataclass
class Message:
    role: str
    content: str
    tool_calls: Optional[list] = None
    tool_call_id: Optional[str] = None
    name: Optional[str] = None


@dataclass
class FormattedChat:
    text: str
    response_start: int
    template_type: str

    def prompt(self) -> str:
        return self.text[:self.response_start]

    def response(self) -> str:
        return self.text[self.response_start:]


def _tools_block(tools) -> str:
    return ("\n\n# Tools\n\nYou may call one or more functions to assist with the user query.\n\n"
            "You are provided with function signatures within <tools></tools> XML tags:\n<tools>\n"
            + "\n".join(json.dumps(t, ensure_ascii=False) for t in tools)
            + "\n</tools>\n\nFor each function call, return a json object with function name and arguments within "
              "<tool_call></tool_call> XML tags:\n<tool_call>\n{\"name\": <function-name>, \"arguments\": "
              "<args-json-object>}\n</tool_call>")


class ChatTemplate:
    def __init__(self, template_type: str = "chatml", jinja_source: Optional[str] = None,
                 bos_token: str = "", eos_token: str = "", add_generation_prompt: bool = True):
        if template_type not in TEMPLATE_TYPES:
            raise ValueError(f"unknown chat template {template_type!r}")
        self.template_type = template_type
        self.jinja_source = jinja_source
        self.bos_token, self.eos_token = bos_token, eos_token
        self.add_generation_prompt = add_generation_prompt

    # ---------------------------------------------------------------- detection
    @classmethod
    def detect(cls, model_name: str) -> str:
        n = model_name.lower()
        rules = [("gpt-oss", "gpt_oss"), ("gpt_oss", "gpt_oss"), ("llama-4", "llama4"), ("llama4", "llama4"),
                 ("llama-3", "llama3"), ("llama3", "llama3"), ("llama-2", "llama2"), ("llama2", "llama2"),
                 ("gemma-4", "gemma4"), ("gemma4", "gemma4"), ("gemma", "gemma"), ("qwen", "qwen"),
                 ("mistral", "mistral"), ("mixtral", "mistral"), ("phi-4", "phi4"), ("phi4", "phi4"),
                 ("phi-3", "phi3"), ("phi3", "phi3"), ("deepseek", "deepseek"), ("command", "cohere"),
                 ("cohere", "cohere"), ("vicuna", "vicuna"), ("zephyr", "zephyr"), ("alpaca", "alpaca")]
        for key, t in rules:
            if key in n:
                return t
        return "chatml"

    @classmethod
    def from_model_dir(cls, model_dir: str, model_name: Optional[str] = None) -> "ChatTemplate":
        src = bos = eos = None
        p = os.path.join(model_dir, "tokenizer_config.json")
        if os.path.exists(p):
            with open(p, "r", encoding="utf-8") as fh:
                tc = json.load(fh)
            src = tc.get("chat_template")
            if isinstance(src, list):
                src = next((x.get("template") for x in src if x.get("name") == "default"), None)

            def tok(v):
                return v.get("content") if isinstance(v, dict) else v
            bos, eos = tok(tc.get("bos_token")), tok(tc.get("eos_token"))
        j = os.path.join(model_dir, "chat_template.jinja")
        if src is None and os.path.exists(j):
            with open(j, "r", encoding="utf-8") as fh:
                src = fh.read()
        return cls(cls.detect(model_name or os.path.basename(os.path.normpath(model_dir))), src, bos or "", eos or "")

    def eos(self) -> str:
        return self.eos_token or EOS[self.template_type]

    # ---------------------------------------------------------------- training-time formatting
    def apply(self, messages: List[Message], tools: Optional[list] = None) -> FormattedChat:
        f = getattr(self, "_fmt_" + ("chatml" if self.template_type in ("chatml", "qwen", "custom")
                                     else self.template_type))
        parts = f(messages, tools)
        text, start = "", 0
        last_asst = max((i for i, (is_a, _) in enumerate(parts) if is_a), default=None)
        for i, (is_a, s) in enumerate(parts):
            if i == last_asst:
                start = len(text)
            text += s
        if last_asst is None:
            start = len(text)
        return FormattedChat(text, start, self.template_type)

    # each formatter returns [(is_assistant_content, string)], where the assistant string is the part to train on
    def _fmt_chatml(self, msgs, tools):
        out = []
        msgs = list(msgs)
        if tools:
            if msgs and msgs[0].role == "system":
                msgs[0] = Message("system", msgs[0].content + _tools_block(tools))
            else:
                msgs.insert(0, Message("system", "You are a helpful assistant." + _tools_block(tools)))
        for m in msgs:
            if m.role == "assistant":
                out.append((False, "<|im_start|>assistant\n"))
                body = m.content
                for tc in m.tool_calls or []:
                    body += ("\n" if body else "") + "<tool_call>\n" + json.dumps(tc, ensure_ascii=False) + "\n</tool_call>"
                out.append((True, body + "<|im_end|>\n"))
            elif m.role == "tool":
                out.append((False, f"<|im_start|>user\n<tool_response>\n{m.content}\n</tool_response><|im_end|>\n"))
            else:
                out.append((False, f"<|im_start|>{m.role}\n{m.content}<|im_end|>\n"))
        return out

    def _fmt_llama3(self, msgs, tools):
        out = [(False, "<|begin_of_text|>")]
        for m in msgs:
            head = f"<|start_header_id|>{'ipython' if m.role == 'tool' else m.role}<|end_header_id|>\n\n"
            if m.role == "assistant":
                out += [(False, head), (True, m.content + "<|eot_id|>")]
            else:
                extra = _tools_block(tools) if (tools and m.role == "system") else ""
                out.append((False, head + m.content + extra + "<|eot_id|>"))
        return out

    def _fmt_llama4(self, msgs, tools):
        out = [(False, "<|begin_of_text|>")]
        for m in msgs:
            head = f"<|header_start|>{m.role}<|header_end|>\n\n"
            if m.role == "assistant":
                out += [(False, head), (True, m.content + "<|eot|>")]
            else:
                out.append((False, head + m.content + "<|eot|>"))
        return out

    def _fmt_llama2(self, msgs, tools):
        out, sys_txt = [], ""
        for m in msgs:
            if m.role == "system":
                sys_txt = f"<<SYS>>\n{m.content}\n<</SYS>>\n\n"
            elif m.role == "user":
                out.append((False, f"<s>[INST] {sys_txt}{m.content} [/INST]"))
                sys_txt = ""
            elif m.role == "assistant":
                out.append((True, f" {m.content} </s>"))
        return out

    def _fmt_mistral(self, msgs, tools):
        out, sys_txt = [(False, "<s>")], ""
        for m in msgs:
            if m.role == "system":
                sys_txt = m.content + "\n\n"
            elif m.role == "user":
                pre = f"[AVAILABLE_TOOLS] {json.dumps(tools)}[/AVAILABLE_TOOLS]" if tools else ""
                out.append((False, f"{pre}[INST] {sys_txt}{m.content} [/INST]"))
                sys_txt, tools = "", None
            elif m.role == "assistant":
                out.append((True, f" {m.content}</s>"))
            elif m.role == "tool":
                out.append((False, f"[TOOL_RESULTS] {m.content}[/TOOL_RESULTS]"))
        return out

    def _fmt_gemma(self, msgs, tools):
        out, sys_txt = [(False, "<bos>")], ""
        for m in msgs:
            if m.role == "system":
                sys_txt = m.content + "\n\n"
            elif m.role == "assistant":
                out += [(False, "<start_of_turn>model\n"), (True, m.content + "<end_of_turn>\n")]
            else:
                out.append((False, f"<start_of_turn>user\n{sys_txt}{m.content}<end_of_turn>\n"))
                sys_txt = ""
        return out

    def _fmt_gemma4(self, msgs, tools):
        out = [(False, "<bos>")]
        for m in msgs:
            if m.role == "assistant":
                out += [(False, "<|turn>model\n"), (True, m.content + "<turn|>\n")]
            else:
                out.append((False, f"<|turn>{m.role}\n{m.content}<turn|>\n"))
        return out

    def _fmt_phi3(self, msgs, tools):
        out = []
        for m in msgs:
            if m.role == "assistant":
                out += [(False, "<|assistant|>\n"), (True, m.content + "<|end|>\n")]
            else:
                out.append((False, f"<|{m.role}|>\n{m.content}<|end|>\n"))
        return out

    def _fmt_phi4(self, msgs, tools):
        out = []
        for m in msgs:
            if m.role == "assistant":
                out += [(False, "<|im_start|>assistant<|im_sep|>"), (True, m.content + "<|im_end|>")]
            else:
                out.append((False, f"<|im_start|>{m.role}<|im_sep|>{m.content}<|im_end|>"))
        return out

    def _fmt_alpaca(self, msgs, tools):
        out = []
        for m in msgs:
            if m.role == "system":
                out.append((False, m.content + "\n\n"))
            elif m.role == "user":
                out.append((False, f"### Instruction:\n{m.content}\n\n### Response:\n"))
            elif m.role == "assistant":
                out.append((True, m.content + "\n\n"))
        return out

    def _fmt_vicuna(self, msgs, tools):
        out = []
        for m in msgs:
            if m.role == "system":
                out.append((False, m.content + " "))
            elif m.role == "user":
                out.append((False, f"USER: {m.content} ASSISTANT:"))
            elif m.role == "assistant":
                out.append((True, f" {m.content}</s>"))
        return out

    def _fmt_zephyr(self, msgs, tools):
        out = []
        for m in msgs:
            if m.role == "assistant":
                out += [(False, "<|assistant|>\n"), (True, m.content + "</s>\n")]
            else:
                out.append((False, f"<|{m.role}|>\n{m.content}</s>\n"))
        return out

    def _fmt_gpt_oss(self, msgs, tools):
        out = []
        for m in msgs:
            if m.role == "assistant":
                out += [(False, "<|start|>assistant<|channel|>final<|message|>"), (True, m.content + "<|return|>")]
            else:
                role = "developer" if m.role == "system" else m.role
                out.append((False, f"<|start|>{role}<|message|>{m.content}<|end|>"))
        return out

    def _fmt_deepseek(self, msgs, tools):
        out = [(False, "<｜begin▁of▁sentence｜>")]
        for m in msgs:
            if m.role == "system":
                out.append((False, m.content))
            elif m.role == "user":
                out.append((False, f"<｜User｜>{m.content}"))
            elif m.role == "assistant":
                out += [(False, "<｜Assistant｜>"), (True, m.content + "<｜end▁of▁sentence｜>")]
        return out

    def _fmt_cohere(self, msgs, tools):
        out = [(False, "<BOS_TOKEN>")]
        tag = {"system": "<|SYSTEM_TOKEN|>", "user": "<|USER_TOKEN|>", "assistant": "<|CHATBOT_TOKEN|>"}
        for m in msgs:
            head = f"<|START_OF_TURN_TOKEN|>{tag.get(m.role, '<|USER_TOKEN|>')}"
            if m.role == "assistant":
                out += [(False, head), (True, m.content + "<|END_OF_TURN_TOKEN|>")]
            else:
                out.append((False, head + m.content + "<|END_OF_TURN_TOKEN|>"))
        return out

    # ---------------------------------------------------------------- inference-time formatting
    def generation_prefix(self) -> str:
        return {"chatml": "<|im_start|>assistant\n", "qwen": "<|im_start|>assistant\n",
                "custom": "<|im_start|>assistant\n",
                "llama3": "<|start_header_id|>assistant<|end_header_id|>\n\n",
                "llama4": "<|header_start|>assistant<|header_end|>\n\n", "gemma": "<start_of_turn>model\n",
                "gemma4": "<|turn>model\n", "phi3": "<|assistant|>\n", "phi4": "<|im_start|>assistant<|im_sep|>",
                "zephyr": "<|assistant|>\n", "gpt_oss": "<|start|>assistant", "deepseek": "<｜Assistant｜>",
                "cohere": "<|START_OF_TURN_TOKEN|><|CHATBOT_TOKEN|>"}.get(self.template_type, "")

    def render_jinja(self, messages: List[Message], no_thinking: bool = False, tools: Optional[list] = None,
                     add_generation_prompt: bool = True) -> Optional[str]:
        if not self.jinja_source:
            return None
        try:
            from jinja2.sandbox import ImmutableSandboxedEnvironment
            env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
            env.filters["tojson"] = lambda v, **kw: json.dumps(v, ensure_ascii=False, **{k: kw[k] for k in kw if k == "indent"})
            env.globals["raise_exception"] = lambda msg: (_ for _ in ()).throw(ValueError(msg))
            import datetime
            env.globals["strftime_now"] = lambda fmt: datetime.datetime.now().strftime(fmt)
            tpl = env.from_string(self.jinja_source)
            ms = []
            for m in messages:
                d = {"role": m.role, "content": m.content}
                if m.tool_calls:
                    d["tool_calls"] = m.tool_calls
                if m.tool_call_id:
                    d["tool_call_id"] = m.tool_call_id
                if m.name:
                    d["name"] = m.name
                ms.append(d)
            return tpl.render(messages=ms, tools=tools, add_generation_prompt=add_generation_prompt,
                              bos_token=self.bos_token, eos_token=self.eos_token,
                              enable_thinking=not no_thinking)
        except Exception:
            return None

    def apply_inference(self, messages: List[Message], no_thinking: bool = False, tools: Optional[list] = None) -> str:
        """Prompt for generation: the model's own Jinja template when available, else the hard-coded format
        plus the assistant prefix (Qwen: an empty think block when thinking is disabled)."""
        r = self.render_jinja(messages, no_thinking, tools, True)
        if r is not None:
            return r
        text = self.apply(messages, tools).text + self.generation_prefix()
        if self.template_type == "qwen" and no_thinking:
            text += "<think>\n\n</think>\n\n"
        return text
