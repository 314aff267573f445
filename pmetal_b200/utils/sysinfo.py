"""Device / interconnect inventory and memory-fit estimates (``pmetal info``, ``pmetal memory``).

Replaces the reference's Apple-silicon probes (crates/pmetal-hub/src/fit.rs, bandwidth_probe.metal)
with CUDA device properties, NVML NVLink state where available, and analytic estimates.
"""
from __future__ import annotations

import json
import os
from typing import Dict


def system_info() -> Dict:
    import torch
    info: Dict = {"torch": torch.__version__, "cuda_available": torch.cuda.is_available(), "devices": []}
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            pr = torch.cuda.get_device_properties(i)
            info["devices"].append({"index": i, "name": pr.name, "sms": pr.multi_processor_count,
                                    "memory_gib": round(pr.total_memory / 2 ** 30, 1),
                                    "capability": f"{pr.major}.{pr.minor}"})
        n = torch.cuda.device_count()
        info["p2p"] = [[(i == j) or torch.cuda.can_device_access_peer(i, j) for j in range(n)] for i in range(n)]
        try:
            import pynvml
            pynvml.nvmlInit()
            links = []
            for i in range(n):
                h = pynvml.nvmlDeviceGetHandleByIndex(i)
                up = 0
                for l in range(18):
                    try:
                        up += int(pynvml.nvmlDeviceGetNvLinkState(h, l) == 1)
                    except pynvml.NVMLError:
                        break
                links.append(up)
            info["nvlink_links_up"] = links
        except Exception as e:  # NVML optional
            info["nvlink_links_up"] = f"unavailable ({type(e).__name__})"
    from ..ops import native
    info["native_library"] = {"path": native.LIB_PATH, "loaded": native.available(), "error": native.load_error()}
    peaks = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                         "MEASURED_PEAKS.json")
    if os.path.exists(peaks):
        with open(peaks) as fh:
            info["measured_peaks"] = json.load(fh)
    return info


def estimate_fit(model: str, seq_len: int, batch: int, lora_r: int, quantization: str = "none") -> Dict:
    from ..models.config import PRESETS, ModelArgs, preset
    from ..models.loader import resolve_model_path
    if model.startswith("random:"):
        cfg = preset(model.split(":", 1)[1])
    elif model.lower() in PRESETS:
        cfg = preset(model)
    else:
        cfg = ModelArgs.from_pretrained(resolve_model_path(model))
    H, I, L, V = cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers, cfg.vocab_size
    attn = H * (cfg.q_size + 2 * cfg.kv_size) + cfg.q_size * H
    if cfg.num_experts:
        mlp = cfg.num_experts * 3 * H * cfg.moe_intermediate_size + cfg.num_experts * H
    else:
        mlp = 3 * H * I
    params = L * (attn + mlp + 2 * H) + V * H * (1 if cfg.tie_word_embeddings else 2) + H
    bpw = {"none": 2.0, "nf4": 0.5 + 4.0 / 64 + 0.002, "fp4": 0.5 + 4.0 / 64, "int8": 1.0 + 4.0 / 64}[quantization]
    weights = params * bpw
    transposed = (params - V * H) * 2.0 if quantization == "none" else 0.0
    lora = L * lora_r * (H + cfg.q_size + 2 * (H + cfg.kv_size) + cfg.q_size + H + 2 * (H + I) + I + H)
    tokens = seq_len * batch
    act = tokens * L * (6 * H + 2 * (cfg.q_size + 2 * cfg.kv_size) + 2 * cfg.q_size + 3 * I) * 2.0
    total = weights + transposed + lora * 16 + act + tokens * 4096 * 2
    flops = 4.0 * (params - V * H) * tokens + 4.0 * V * H * tokens
    return {"parameters": int(params), "lora_parameters": int(lora), "weights_gib": round(weights / 2 ** 30, 2),
            "activations_gib": round(act / 2 ** 30, 2), "total_gib": round(total / 2 ** 30, 2),
            "fits_180gib": total < 170 * 2 ** 30, "step_tflop": round(flops / 1e12, 2),
            "est_tokens_per_s_at_1pflops": int(tokens / (flops / 1e15))}
