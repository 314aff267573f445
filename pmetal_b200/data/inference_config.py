"""Shared inference settings: stop tokens, sampling defaults and per-family sampling presets.

Resolution order of the sampling parameters (crates/pmetal-data/src/inference_config.rs:11-16, :475-501):
explicit caller value > ``--mode`` preset of the model family > the model's ``generation_config.json`` > global fallback
(temperature 0.7, top-k 20, top-p 0.8). Stop tokens are the union of every source that names one (:34-113): the
generation config, the chat template's end token, the tokenizer's eos id and the well-known end-of-turn tokens that
exist in the vocabulary as single tokens, so a fine-tuned model stops whether it emits the base model's or the chat
template's terminator."""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass
from typing import Dict, List, Optional

WELL_KNOWN_STOP_TOKENS = ("<|im_end|>", "<|eot_id|>", "<|eot|>", "<|endoftext|>", "<|end_of_text|>", "<end_of_turn>",
                          "<turn|>", "<|end|>", "<|return|>", "<|END_OF_TURN_TOKEN|>", "<｜end▁of▁sentence｜>", "</s>")

MODES = ("auto", "thinking-general", "thinking-coding", "instruct-general", "instruct-reasoning")
_MODE_ALIASES = {"general-thinking": "thinking-general", "thinking": "thinking-general", "coding": "thinking-coding",
                 "general-instruct": "instruct-general", "instruct": "instruct-general", "reasoning": "instruct-reasoning"}


@dataclass
class SamplingDefaults:
    temperature: float = 0.7
    top_k: int = 20
    top_p: float = 0.8
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0


# Model-card recommendations of the Qwen 3 family. The thinking modes carry no presence penalty: during long reasoning
# chains it penalises function words and provokes an early end of sequence.
_QWEN_PRESETS: Dict[str, SamplingDefaults] = {
    "thinking-general": SamplingDefaults(1.0, 20, 0.95, 0.0, 1.0, 0.0, 0.0),
    "thinking-coding": SamplingDefaults(0.6, 20, 0.95, 0.0, 1.0, 0.0, 0.0),
    "instruct-general": SamplingDefaults(0.7, 20, 0.8, 0.0, 1.0, 0.0, 1.5),
    "instruct-reasoning": SamplingDefaults(1.0, 40, 1.0, 0.0, 1.0, 0.0, 2.0),
}
_QWEN_TEMPLATES = ("chatml", "qwen")


def parse_mode(name: str) -> str:
    n = _MODE_ALIASES.get(name, name)
    if n not in MODES:
        raise ValueError(f"unknown mode {name!r}: expected one of {', '.join(MODES)}")
    return n


def available_modes(template_type: Optional[str]) -> List[str]:
    return list(_QWEN_PRESETS) if template_type in _QWEN_TEMPLATES else []


def resolve_auto_mode(mode: str, thinking: bool) -> str:
    if mode != "auto":
        return mode
    return "thinking-general" if thinking else "instruct-general"


def model_preset(template_type: Optional[str], mode: str) -> Optional[SamplingDefaults]:
    if template_type in _QWEN_TEMPLATES and mode in _QWEN_PRESETS:
        return dataclasses.replace(_QWEN_PRESETS[mode])
    return None


def _generation_config(model_dir: Optional[str]) -> dict:
    if not model_dir:
        return {}
    path = os.path.join(model_dir, "generation_config.json")
    try:
        with open(path, "r", encoding="utf-8") as fh:
            cfg = json.load(fh)
        return cfg if isinstance(cfg, dict) else {}
    except (OSError, ValueError):
        return {}


def load_sampling_from_generation_config(model_dir: Optional[str]) -> SamplingDefaults:
    d = SamplingDefaults()
    cfg = _generation_config(model_dir)
    for f in dataclasses.fields(d):
        v = cfg.get(f.name)
        if isinstance(v, (int, float)) and not isinstance(v, bool):
            setattr(d, f.name, int(v) if f.name == "top_k" else float(v))
    return d


def load_sampling_defaults(model_dir: Optional[str], template_type: Optional[str], mode: str = "auto",
                           thinking: bool = False, use_preset: bool = True) -> SamplingDefaults:
    """generation_config.json values, replaced as a whole by the family preset of the (resolved) mode when one exists."""
    d = load_sampling_from_generation_config(model_dir)
    if use_preset:
        p = model_preset(template_type, resolve_auto_mode(parse_mode(mode), thinking))
        if p is not None:
            d = p
    return d


def collect_all_stop_tokens(model_dir: Optional[str], tokenizer, template_eos: Optional[str] = None) -> List[int]:
    """Sorted, de-duplicated stop ids; ``[2]`` when no source yields one."""
    out = set()
    eos = _generation_config(model_dir).get("eos_token_id")
    if isinstance(eos, list):
        out.update(int(v) for v in eos if isinstance(v, int) and not isinstance(v, bool))
    elif isinstance(eos, int) and not isinstance(eos, bool):
        out.add(eos)

    def single(text: str) -> Optional[int]:
        i = tokenizer.token_to_id(text)
        if i is not None:
            return int(i)
        try:
            ids = tokenizer.encode_with_special_tokens(text)
        except Exception:
            return None
        return int(ids[0]) if len(ids) == 1 else None

    if template_eos:
        i = single(template_eos)
        if i is not None:
            out.add(i)
    if getattr(tokenizer, "eos_token_id", None) is not None:
        out.add(int(tokenizer.eos_token_id))
    for cand in WELL_KNOWN_STOP_TOKENS:
        i = tokenizer.token_to_id(cand)
        if i is not None:
            out.add(int(i))
    return sorted(out) or [2]
