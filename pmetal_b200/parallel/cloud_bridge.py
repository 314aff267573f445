"""Run bundle for moving a training run between machines: ``model.safetensors`` (trainable parameters),
``optimizer.safetensors`` (moments), ``rng_state.bin``, ``metadata.json`` and a ``bootstrap_cluster.py`` launcher
(crates/pmetal-distributed/src/cloud_bridge.rs:55-260). ``export_bundle`` writes one, ``import_bundle`` reads one back
into a model / optimiser pair on this node."""
from __future__ import annotations

import json
import os
import time
from typing import Dict, Optional

import torch

from ..utils.safetensors_io import load_file, save_file

BOOTSTRAP = '''#!/usr/bin/env python3
"""Resume this bundle on every GPU of one node."""
import os, subprocess, sys
here = os.path.dirname(os.path.abspath(__file__))
n = int(os.environ.get("NGPU", "8"))
cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
       "--master-port", "29700", "-m", "pmetal_b200.cli.main", "train", "--resume-bundle", here] + sys.argv[1:]
raise SystemExit(subprocess.call(cmd))
'''


def export_bundle(out_dir: str, params: Dict[str, torch.Tensor], optimizer_state: Dict[str, torch.Tensor], step: int,
                  config: Optional[dict] = None, world_size: int = 1) -> dict:
    os.makedirs(out_dir, exist_ok=True)
    save_file({k: v.detach().cpu().contiguous() for k, v in params.items()}, os.path.join(out_dir, "model.safetensors"))
    save_file({k: v.detach().cpu().contiguous() for k, v in optimizer_state.items()}, os.path.join(out_dir, "optimizer.safetensors"))
    rng = torch.get_rng_state()
    with open(os.path.join(out_dir, "rng_state.bin"), "wb") as fh:
        fh.write(rng.numpy().tobytes())
    meta = {"format": "pmetal-cloud-bundle", "version": 1, "step": int(step), "world_size": int(world_size),
            "created": int(time.time()), "num_params": int(sum(v.numel() for v in params.values())), "config": config or {}}
    with open(os.path.join(out_dir, "metadata.json"), "w", encoding="utf-8") as fh:
        json.dump(meta, fh, indent=1)
    path = os.path.join(out_dir, "bootstrap_cluster.py")
    with open(path, "w", encoding="utf-8") as fh:
        fh.write(BOOTSTRAP)
    os.chmod(path, 0o755)
    return meta


def import_bundle(bundle_dir: str, restore_rng: bool = True):
    """Returns (params, optimizer_state, metadata)."""
    with open(os.path.join(bundle_dir, "metadata.json"), "r", encoding="utf-8") as fh:
        meta = json.load(fh)
    if meta.get("format") != "pmetal-cloud-bundle":
        raise ValueError(f"{bundle_dir} is not a run bundle")
    params = load_file(os.path.join(bundle_dir, "model.safetensors"))
    opt = load_file(os.path.join(bundle_dir, "optimizer.safetensors"))
    rng_path = os.path.join(bundle_dir, "rng_state.bin")
    if restore_rng and os.path.exists(rng_path):
        with open(rng_path, "rb") as fh:
            raw = fh.read()
        torch.set_rng_state(torch.frombuffer(bytearray(raw), dtype=torch.uint8))
    return params, opt, meta
