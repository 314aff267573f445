"""pmetal_b200 — LLM fine-tuning, RL and serving on NVIDIA B200 (sm_100a).

PyTorch is the framework layer; the hot operators are hand-written CUDA kernels in
``pmetal_b200/csrc`` (tcgen05/TMEM GEMMs fed by TMA, flash attention, fused
normalisation/activation/loss/optimizer kernels and peer-memory collectives).
"""
__version__ = "0.1.0"


def __getattr__(name):          # lazy: importing the package must not import torch-heavy modules
    if name in ("finetune", "infer", "Model"):
        from . import api
        return getattr(api, name)
    raise AttributeError(name)
