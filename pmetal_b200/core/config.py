"""Configuration dataclasses.

Field names and default values follow the reference's serde structs
(crates/pmetal-core/src/config.rs:8-446) so that the same YAML files load
unchanged: ``{model: {model_id,...}, lora: {...}, training: {...}, dataset: {dataset_id,...}}``.
"""
from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass, field
from typing import Any, List, Optional

LR_SCHEDULERS = ("constant", "linear", "cosine", "cosine_with_restarts", "polynomial", "wsd")
OPTIMIZERS = ("adam_w", "sgd", "adafactor", "lion")
COMPRESSIONS = ("none", "top_k", "fp16", "random")
DTYPES = ("float32", "float16", "bfloat16")


def _from_dict(cls, d: Optional[dict]):
    """Build ``cls`` from a mapping, ignoring unknown keys (serde default behaviour)."""
    if d is None:
        return cls()
    names = {f.name for f in dataclasses.fields(cls)}
    return cls(**{k: v for k, v in d.items() if k in names})


@dataclass
class ModelConfig:
    model_id: str = ""
    dtype: str = "bfloat16"
    quantization: str = "none"
    device: str = "cuda"
    max_seq_len: int = 8192
    use_flash_attention: bool = True
    trust_remote_code: bool = False
    revision: Optional[str] = None
    hf_token: Optional["SecretString"] = None      # never serialised, never printed (core/secrets.py)

    from_dict = classmethod(_from_dict)

    def __post_init__(self):
        from .secrets import SecretString
        if self.hf_token is not None and not isinstance(self.hf_token, SecretString):
            self.hf_token = SecretString(self.hf_token)


@dataclass
class LoraConfig:
    """LoRA hyper-parameters (reference: config.rs:78-152)."""

    r: int = 16
    alpha: float = 32.0
    dropout: float = 0.0
    target_modules: List[str] = field(default_factory=lambda: ["q_proj", "k_proj", "v_proj", "o_proj"])
    use_rslora: bool = False
    use_dora: bool = False
    bias: str = "none"
    init_lora_weights: bool = True
    loraplus_lr_ratio: Optional[float] = None

    from_dict = classmethod(_from_dict)

    def scaling(self) -> float:
        if self.r == 0:
            return 0.0
        if self.use_rslora:
            return self.alpha / math.sqrt(self.r)
        return self.alpha / self.r


@dataclass
class TrainingConfig:
    """Training hyper-parameters (reference: config.rs:156-286)."""

    learning_rate: float = 2e-4
    embedding_learning_rate: Optional[float] = None
    batch_size: int = 1
    gradient_accumulation_steps: int = 4
    num_epochs: int = 3
    max_steps: Optional[int] = None
    warmup_steps: int = 100
    warmup_ratio: Optional[float] = None
    weight_decay: float = 0.01
    max_grad_norm: float = 1.0
    lr_scheduler: str = "cosine"
    min_lr: Optional[float] = None
    wsd_stable_ratio: Optional[float] = None
    cosine_num_restarts: Optional[int] = None
    polynomial_power: Optional[float] = None
    gradient_checkpointing: Any = "none"
    optimizer: str = "adam_w"
    seed: int = 42
    logging_steps: int = 10
    eval_steps: Optional[int] = None
    save_steps: Optional[int] = None
    output_dir: str = "./output"
    use_packing: bool = True
    max_seq_len: int = 8192

    from_dict = classmethod(_from_dict)


@dataclass
class DistributedTrainingConfig:
    """reference: config.rs:359-396."""

    peers: List[str] = field(default_factory=list)
    auto_discover: bool = False
    gradient_port: int = 52416
    compression: str = "none"
    topk_ratio: float = 0.01
    error_feedback: bool = True

    from_dict = classmethod(_from_dict)


@dataclass
class DatasetConfig:
    dataset_id: str = ""
    split: str = "train"
    text_column: str = "text"
    max_samples: Optional[int] = None
    shuffle: bool = True
    seed: int = 42

    from_dict = classmethod(_from_dict)


@dataclass
class FullTrainingConfig:
    """The YAML document accepted by ``pmetal train --config`` (orchestrator.rs:2000-2021)."""

    model: ModelConfig = field(default_factory=ModelConfig)
    lora: LoraConfig = field(default_factory=LoraConfig)
    training: TrainingConfig = field(default_factory=TrainingConfig)
    dataset: DatasetConfig = field(default_factory=DatasetConfig)
    distributed: Optional[DistributedTrainingConfig] = None

    @classmethod
    def from_dict(cls, d: dict) -> "FullTrainingConfig":
        return cls(
            model=ModelConfig.from_dict(d.get("model")),
            lora=LoraConfig.from_dict(d.get("lora")),
            training=TrainingConfig.from_dict(d.get("training")),
            dataset=DatasetConfig.from_dict(d.get("dataset")),
            distributed=DistributedTrainingConfig.from_dict(d["distributed"]) if d.get("distributed") else None,
        )

    @classmethod
    def from_yaml(cls, path: str) -> "FullTrainingConfig":
        import yaml

        with open(path, "r", encoding="utf-8") as fh:
            return cls.from_dict(yaml.safe_load(fh) or {})

    def to_dict(self) -> dict:
        d = dataclasses.asdict(self)
        d["model"].pop("hf_token", None)  # skip_serializing in the reference
        return d


def merge_overrides(base, explicit: dict):
    """Apply CLI values over a YAML-loaded dataclass.

    The reference lets an *explicit* CLI value win over YAML by comparing the
    CLI value against the struct default (orchestrator.rs:186-300); here the
    caller passes only the options the user typed.
    """
    for k, v in explicit.items():
        if v is not None and hasattr(base, k):
            setattr(base, k, v)
    return base
