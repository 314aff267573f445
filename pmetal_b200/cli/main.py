"""``pmetal`` command line.

Sub-commands and flag names follow the reference CLI (crates/pmetal/src/main.rs:270-585,
crates/pmetal/src/cli/*.rs): train, infer, fuse, merge, quantize, distill, grpo, serve, cluster,
bench, bench-corpus, eval, info, memory, dataset, tokenize, init, search/download (offline: local
cache only). ``--log-events PATH`` writes the job-event JSONL stream for any command.
``tui`` opens the terminal application (``pmetal_b200/tui``); ``dashboard`` follows a JSONL event stream headlessly;
the reference's desktop GUI has no counterpart.
"""
from __future__ import annotations

import argparse
import json
import logging
import os
import sys
from typing import List, Optional


def _add_train(sp):
    p = sp.add_parser("train", help="LoRA / QLoRA / DoRA supervised fine-tuning")
    p.add_argument("-c", "--config")
    p.add_argument("-m", "--model")
    p.add_argument("-d", "--dataset")
    p.add_argument("--eval-dataset")
    p.add_argument("-o", "--output", default="./output")
    p.add_argument("--lora-r", type=int, default=16)
    p.add_argument("--lora-alpha", type=float, default=32.0)
    p.add_argument("--lora-targets", default=None, help="comma list, default q_proj,k_proj,v_proj,o_proj")
    p.add_argument("--use-rslora", action="store_true")
    p.add_argument("--use-dora", action="store_true")
    p.add_argument("--loraplus-ratio", type=float, default=None)
    p.add_argument("--learning-rate", type=float, default=2e-4)
    p.add_argument("--batch-size", type=int, default=1)
    p.add_argument("--epochs", type=int, default=1)
    p.add_argument("--max-steps", type=int, default=None)
    p.add_argument("--max-seq-len", type=int, default=0)
    p.add_argument("--gradient-accumulation-steps", type=int, default=4)
    p.add_argument("--max-grad-norm", type=float, default=1.0)
    p.add_argument("--resume", action="store_true")
    p.add_argument("--tensorboard", help="write TensorBoard scalars to this directory")
    p.add_argument("--resume-bundle", help="continue from a run bundle (parallel/cloud_bridge.py: model + optimiser + RNG)")
    p.add_argument("--quantization", default="none", choices=["none", "nf4", "fp4", "int8"])
    p.add_argument("--quant-block-size", type=int, default=64)
    p.add_argument("--double-quant", action="store_true")
    p.add_argument("--no-fused", action="store_true", help="run the PyTorch reference operators")
    p.add_argument("--no-sequence-packing", action="store_true")
    p.add_argument("--pack-max-seq-len", type=int, default=None)
    p.add_argument("--no-jit-compilation", action="store_true", help="do not capture the step in a CUDA graph")
    p.add_argument("--no-gradient-checkpointing", action="store_true")
    p.add_argument("--gradient-checkpointing-layers", type=int, default=0)
    p.add_argument("--activation-policy", choices=["save", "recompute", "offload-cpu", "offload-disk", "smart"], default=None,
                   help="what every decoder block does with the activations it needs for backward: keep them, recompute "
                        "them, park them in pinned host memory / on disk, or decide from the memory in use")
    p.add_argument("--offload-dir", default=None, help="directory for --activation-policy offload-disk")
    p.add_argument("--log-metrics")
    p.add_argument("--embedding-lr", type=float, default=None)
    p.add_argument("--warmup-steps", type=int, default=0)
    p.add_argument("--lr-schedule", default="cosine")
    p.add_argument("--weight-decay", type=float, default=0.01)
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--cut-cross-entropy", action="store_true")
    p.add_argument("--no-adaptive-lr", action="store_true")
    p.add_argument("--text-column")
    p.add_argument("--text-columns")
    p.add_argument("--column-separator", default="\n\n")
    p.add_argument("--prompt-column")
    p.add_argument("--response-column")
    p.add_argument("--max-samples", type=int, default=None)
    p.add_argument("--distributed-peers", default=None)
    p.add_argument("--distributed-auto", action="store_true")
    p.add_argument("--compression-strategy", default="none")
    p.add_argument("--dp-impl", default="fused", choices=["fused", "nccl"])
    p.add_argument("--expert-parallel", action="store_true",
                   help="mixture-of-experts models on several GPUs: every rank keeps its share of each layer's experts and "
                        "tokens travel to their expert's rank and back (differentiable all-to-all)")
    # accepted for command-line compatibility with the reference (crates/pmetal/src/cli/train.rs:10-186)
    p.add_argument("--no-flash-attention", action="store_true", help="same effect as --no-fused: PyTorch reference attention")
    p.add_argument("--no-metal-fused-optimizer", action="store_true",
                   help="same effect as --dp-impl nccl: separate all-reduce, clip and AdamW kernels instead of the fused step")
    p.add_argument("--loss-scale", type=float, default=None, help="ignored: bf16 training needs no loss scaling")
    p.add_argument("--ane", action="store_true", help="ignored: Apple Neural Engine path of the reference")
    p.add_argument("--device", default=None)
    p.add_argument("--dtype", default="bfloat16")
    p.set_defaults(func=cmd_train)


def cmd_train(a) -> int:
    from ..core.config import LoraConfig
    from ..core.events import JsonlSink
    from ..data.dataset import CustomColumns
    from ..trainer.orchestrator import TrainingJobConfig, run_training
    job = TrainingJobConfig.from_yaml(a.config) if a.config else TrainingJobConfig()
    explicit = {k for k in vars(a) if f"--{k.replace('_', '-')}" in " ".join(sys.argv)}
    if a.model:
        job.model = a.model
    if a.dataset:
        job.dataset = a.dataset
    if not job.model or not job.dataset:
        print("error: --model and --dataset (or --config) are required", file=sys.stderr)
        return 2
    job.eval_dataset, job.output = a.eval_dataset, a.output if ("output" in explicit or not a.config) else job.output
    if not a.config or "lora_r" in explicit:
        job.lora.r = a.lora_r
    if not a.config or "lora_alpha" in explicit:
        job.lora.alpha = a.lora_alpha
    if a.lora_targets:
        job.lora.target_modules = a.lora_targets.split(",")
    job.lora.use_rslora |= a.use_rslora
    job.lora.use_dora |= a.use_dora
    if a.loraplus_ratio:
        job.lora.loraplus_lr_ratio = a.loraplus_ratio
    t = job.training
    for flag, attr in (("learning_rate", "learning_rate"), ("batch_size", "batch_size"), ("epochs", "num_epochs"),
                       ("gradient_accumulation_steps", "gradient_accumulation_steps"),
                       ("max_grad_norm", "max_grad_norm"), ("warmup_steps", "warmup_steps"),
                       ("lr_schedule", "lr_scheduler"), ("weight_decay", "weight_decay"), ("seed", "seed")):
        if not a.config or flag in explicit:
            setattr(t, attr, getattr(a, flag))
    if a.max_steps:
        t.max_steps = a.max_steps
    if a.max_seq_len:
        t.max_seq_len = a.max_seq_len
    if a.embedding_lr:
        t.embedding_learning_rate = a.embedding_lr
    job.quantization, job.quant_block_size, job.double_quant = a.quantization, a.quant_block_size, a.double_quant
    job.use_packing = not a.no_sequence_packing
    job.pack_max_seq_len = a.pack_max_seq_len
    job.use_cuda_graph = not a.no_jit_compilation
    job.gradient_checkpointing_layers = 0 if a.no_gradient_checkpointing else a.gradient_checkpointing_layers
    job.activation_policy, job.offload_dir = a.activation_policy, a.offload_dir
    job.log_metrics, job.resume, job.adaptive_lr = a.log_metrics, a.resume, not a.no_adaptive_lr
    job.resume_bundle = a.resume_bundle
    job.tensorboard_dir = a.tensorboard
    job.max_samples, job.device, job.dtype, job.dp_impl = a.max_samples, a.device, a.dtype, a.dp_impl
    job.expert_parallel = a.expert_parallel
    job.distributed = bool(a.distributed_peers or a.distributed_auto)
    if a.text_column or a.text_columns or a.prompt_column:
        job.dataset_format = "custom"
        job.custom_columns = CustomColumns(a.text_column or "text", a.text_columns.split(",") if a.text_columns else None,
                                           a.column_separator, a.prompt_column, a.response_column)
    if a.no_fused or a.no_flash_attention:
        from ..ops.functional import set_force_reference
        set_force_reference(True)
    if a.no_metal_fused_optimizer:
        job.dp_impl = "nccl"
    for flag in ("ane", "loss_scale"):
        if getattr(a, flag):
            print(f"note: --{flag.replace('_', '-')} has no effect on this hardware", file=sys.stderr)
    sink = JsonlSink(a.log_events) if getattr(a, "log_events", None) else None
    summary = run_training(job, sink=sink)
    print(json.dumps(summary))
    return 0


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="pmetal", description="LLM fine-tuning, RL and serving on NVIDIA B200")
    ap.add_argument("--log-events", default=None, help="write job events as JSON lines to this file")
    ap.add_argument("-v", "--verbose", action="store_true")
    sp = ap.add_subparsers(dest="command")
    _add_train(sp)
    from . import commands
    commands.register(sp)
    return ap


def setup_logging(verbose: bool = False, log_file: Optional[str] = None) -> Optional[str]:
    """Log to stderr and to a file with one rotation: ``PMETAL_LOG_FILE`` or ``~/.cache/pmetal/logs/cli.log``; a file
    above 8 MiB is moved to ``.1`` first (crates/pmetal/src/main.rs:1318-1397). ``PMETAL_LOG_FILE=off`` disables the
    file; an unwritable location is skipped silently. Returns the file path in use."""
    level = logging.DEBUG if verbose else getattr(logging, os.environ.get("PMETAL_LOG", "INFO").upper(), logging.INFO)
    fmt = logging.Formatter("%(asctime)s %(levelname)s %(message)s")
    root = logging.getLogger()
    root.setLevel(level)
    for h in list(root.handlers):
        if getattr(h, "_pmetal", False):
            root.removeHandler(h)
            h.close()
    err = logging.StreamHandler(sys.stderr)
    err.setFormatter(fmt)
    err._pmetal = True
    root.addHandler(err)
    path = log_file or os.environ.get("PMETAL_LOG_FILE") or os.path.join(os.path.expanduser("~"), ".cache", "pmetal", "logs",
                                                                         "cli.log")
    if path.lower() in ("off", "none", "0"):
        return None
    try:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        if os.path.exists(path) and os.path.getsize(path) > 8 << 20:
            os.replace(path, path + ".1")
        fh = logging.FileHandler(path, encoding="utf-8")
    except OSError:
        return None
    fh.setFormatter(fmt)
    fh._pmetal = True
    root.addHandler(fh)
    return path


def main(argv: Optional[List[str]] = None) -> int:
    ap = build_parser()
    a = ap.parse_args(argv)
    setup_logging(a.verbose)
    logging.getLogger("pmetal").debug("command line: %s", " ".join(argv if argv is not None else sys.argv[1:]))
    if not getattr(a, "func", None):
        ap.print_help()
        return 1
    return int(a.func(a) or 0)


if __name__ == "__main__":
    sys.exit(main())
