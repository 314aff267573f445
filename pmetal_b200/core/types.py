"""Metric records passed to callbacks (reference: crates/pmetal-core/src/types.rs:170-290)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class StepMetrics:
    step: int = 0
    epoch: int = 0
    total_epochs: int = 0
    total_steps: int = 0
    loss: float = 0.0
    lr: float = 0.0
    tok_sec: float = 0.0
    # The four Apple-Neural-Engine timing fields of the reference record are kept
    # (always 0.0 here) so that consumers of the JSONL stream see the same keys.
    ane_fwd_ms: float = 0.0
    ane_bwd_ms: float = 0.0
    rmsnorm_ms: float = 0.0
    cblas_ms: float = 0.0
    adam_ms: float = 0.0
    total_ms: float = 0.0
    tokens: int = 0
    grad_norm: Optional[float] = None


@dataclass
class EvalMetrics:
    loss: float = 0.0
    perplexity: float = 0.0
    accuracy: Optional[float] = None


# ---------------------------------------------------------------------------------------------- enumerations
# String-valued, so that ``TrainingConfig(lr_scheduler=LrSchedulerType.COSINE)`` and ``lr_scheduler="cosine"`` are the
# same thing (crates/pmetal-core/src/types.rs:8-130, crates/pmetal-core/src/config.rs:66-355).
import enum as _enum


class _StrEnum(str, _enum.Enum):
    def __str__(self) -> str:
        return self.value


class Dtype(_StrEnum):
    FLOAT32 = "float32"
    FLOAT16 = "float16"
    BFLOAT16 = "bfloat16"
    FLOAT8_E4M3 = "float8_e4m3fn"
    FLOAT8_E5M2 = "float8_e5m2"
    INT32 = "int32"
    INT64 = "int64"
    UINT8 = "uint8"

    def torch(self):
        import torch
        return getattr(torch, self.value)


class Device(_StrEnum):
    CPU = "cpu"
    GPU = "cuda"


class Quantization(_StrEnum):
    NONE = "none"
    NF4 = "nf4"
    FP4 = "fp4"
    INT8 = "int8"
    FP8 = "fp8"


class LoraBias(_StrEnum):
    NONE = "none"
    ALL = "all"
    LORA_ONLY = "lora_only"


class LrSchedulerType(_StrEnum):
    CONSTANT = "constant"
    LINEAR = "linear"
    COSINE = "cosine"
    COSINE_WITH_RESTARTS = "cosine_with_restarts"
    POLYNOMIAL = "polynomial"
    WSD = "wsd"


class OptimizerType(_StrEnum):
    ADAMW = "adamw"
    SGD = "sgd"
    ADAFACTOR = "adafactor"
    LION = "lion"


class CheckpointStrategy(_StrEnum):
    NONE = "none"
    EVERY_N = "every_n"
    SMART = "smart"
    SELECTIVE_ATTENTION = "selective_attention"


class DistributedCompression(_StrEnum):
    NONE = "none"
    TOPK = "topk"
    FP16 = "fp16"
    RANDOM = "random"


class DatasetFormat(_StrEnum):
    AUTO = "auto"
    TEXT = "text"
    ALPACA = "alpaca"
    SHAREGPT = "sharegpt"
    MESSAGES = "messages"
    REASONING = "reasoning"
    CUSTOM = "custom"


class ModelArchitecture(_StrEnum):
    LLAMA = "llama"
    LLAMA4 = "llama4"
    QWEN2 = "qwen2"
    QWEN3 = "qwen3"
    QWEN3_MOE = "qwen3_moe"
    QWEN3_NEXT = "qwen3_next"
    MISTRAL = "mistral"
    MIXTRAL = "mixtral"
    GEMMA = "gemma"
    GEMMA4 = "gemma4"
    PHI = "phi"
    COHERE = "cohere"
    GRANITE = "granite"
    DEEPSEEK = "deepseek"
    GPT_OSS = "gpt_oss"
    NEMOTRON_H = "nemotron_h"
    MLLAMA = "mllama"
    PIXTRAL = "pixtral"
    QWEN2_VL = "qwen2_vl"
    BERT = "bert"
    T5 = "t5"
    CLIP = "clip"
    WHISPER = "whisper"
    FLUX = "flux"

    @classmethod
    def from_config(cls, config: dict) -> "ModelArchitecture":
        """Family of a Hugging Face ``config.json`` (first enumeration value contained in its ``model_type``)."""
        mt = str(config.get("model_type", "")).lower().replace("-", "_")
        for m in sorted(cls, key=lambda m: -len(m.value)):
            if mt.startswith(m.value) or m.value in mt:
                return m
        raise ValueError(f"unknown architecture {mt!r}")
