"""pmetal_b200 — LLM fine-tuning, RL and serving on NVIDIA B200 (sm_100a).

PyTorch is the framework layer; the hot operators are hand-written CUDA kernels in
``pmetal_b200/csrc`` (tcgen05/TMEM GEMMs fed by TMA, flash attention, fused
normalisation/activation/loss/optimizer kernels and peer-memory collectives).
"""
__version__ = "0.1.0"


_API = ("finetune", "infer", "Model", "Trainer", "GenerationConfig", "DataLoaderConfig", "download_model", "download_file",
        "DFlashGenerator")
_LAZY = {"LoraConfig": "core.config", "TrainingConfig": "core.config", "ModelConfig": "core.config",
         "DatasetConfig": "core.config", "Dtype": "core.types", "Quantization": "core.types", "LoraBias": "core.types",
         "LrSchedulerType": "core.types", "OptimizerType": "core.types", "DatasetFormat": "core.types",
         "ModelArchitecture": "core.types", "ProgressCallback": "core.callbacks", "LoggingCallback": "core.callbacks",
         "MetricsJsonCallback": "core.callbacks", "TensorBoardCallback": "core.callbacks", "Tokenizer": "data.tokenizer"}
__all__ = ["__version__", *_API, *_LAZY]


def __getattr__(name):          # lazy: importing the package must not import torch-heavy modules
    import importlib
    if name in _API:
        return getattr(importlib.import_module(".api", __name__), name)
    if name in _LAZY:
        return getattr(importlib.import_module("." + _LAZY[name], __name__), name)
    raise AttributeError(name)
