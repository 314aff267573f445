"""End-to-end training job: config merge → model → tokenizer → dataset → loop → adapter files.

Phase order and artefacts follow the reference orchestrator
(crates/pmetal-trainer/src/orchestrator.rs:379-1332): explicit CLI values override YAML,
``max_seq_len`` auto = min(max_position_embeddings, 8192), checkpoints under
``<output>/checkpoints`` (keep 3), adaptive-LR control file ``.lr_control.json``, packed
loop preferred over the padded loop, ``lora_weights.safetensors`` + ``adapter_config.json``
written at the end by rank 0. Unlike the reference, sequence packing and the captured
(CUDA-graph) step stay enabled in data-parallel runs.
"""
from __future__ import annotations

import dataclasses
import json
import logging
import os
import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional

import torch

from ..core.callbacks import LoggingCallback, MetricsJsonCallback, TrainingCallback
from ..core.config import DatasetConfig, FullTrainingConfig, LoraConfig, ModelConfig, TrainingConfig
from ..core.events import JobEvent, NullSink

log = logging.getLogger("pmetal")


@dataclass
class TrainingJobConfig:
    model: str = ""
    dataset: str = ""
    eval_dataset: Optional[str] = None
    output: str = "./output"
    lora: LoraConfig = field(default_factory=LoraConfig)
    training: TrainingConfig = field(default_factory=TrainingConfig)
    quantization: str = "none"          # none | nf4 | fp4 | int8
    quant_block_size: int = 64
    double_quant: bool = False
    use_packing: bool = True
    pack_max_seq_len: Optional[int] = None
    packs_per_batch: Optional[int] = None
    use_cuda_graph: bool = True
    gradient_checkpointing_layers: int = 0
    activation_policy: Optional[str] = None      # save | recompute | offload-cpu | offload-disk | smart (utils/offload.py)
    offload_dir: Optional[str] = None
    log_metrics: Optional[str] = None
    tensorboard_dir: Optional[str] = None
    resume: bool = False
    resume_bundle: Optional[str] = None
    adaptive_lr: bool = True
    dataset_format: str = "auto"
    custom_columns: Optional[object] = None
    max_samples: Optional[int] = None
    device: Optional[str] = None
    dtype: str = "bfloat16"
    distributed: bool = False
    dp_impl: str = "fused"
    expert_parallel: bool = False        # mixture-of-experts models: every rank keeps 1 / world of each layer's experts
    cut_cross_entropy: bool = True
    job_id: str = "train"

    @classmethod
    def from_yaml(cls, path: str) -> "TrainingJobConfig":
        full = FullTrainingConfig.from_yaml(path)
        return cls(model=full.model.model_id, dataset=full.dataset.dataset_id, output=full.training.output_dir,
                   lora=full.lora, training=full.training, quantization=full.model.quantization,
                   use_packing=full.training.use_packing, max_samples=full.dataset.max_samples)


def _portable_model_dir(model: str) -> Optional[str]:
    """The model directory when its architecture is served by the portable implementations (anything but the
    llama / qwen2 / qwen3 / qwen3-moe / mistral family of the hand-written kernels), else None."""
    import json as _json

    from ..models.architectures import family_of
    from ..models.loader import resolve_model_path
    try:
        path = resolve_model_path(model)
    except FileNotFoundError:
        return None
    cfg_path = os.path.join(path, "config.json")
    if path.startswith("random:") or not os.path.exists(cfg_path):
        return None
    with open(cfg_path, "r", encoding="utf-8") as fh:
        fam = family_of(_json.load(fh))
    return path if fam not in (None, "fast") else None


def _run_portable_training(job: "TrainingJobConfig", model_dir: str, dev, dtype, out_dir: str, phase, callbacks, t_start) -> dict:
    """LoRA fine-tuning of a portable architecture: packed rows (documents side by side, attention kept inside each
    document) or padded batches through the modules with adapters wrapped around the target projections
    (``lora/portable.py``). Same dataset handling, schedule, callbacks and output files as the fast path; no CUDA graph or
    fused optimiser."""
    import torch

    from ..core.callbacks import CompositeCallback, LoggingCallback, MetricsJsonCallback
    from ..core.types import StepMetrics
    from ..data.chat_templates import ChatTemplate
    from ..data.dataloader import DataLoader
    from ..data.dataset import TrainingDataset
    from ..data.tokenizer import Tokenizer
    from ..lora.portable import PortableLoraTrainer, apply_lora_portable, load_adapter_portable, save_adapter_portable
    from ..models.architectures import load_pretrained as load_portable
    tcfg = job.training
    phase("loading_model")
    model = load_portable(model_dir, dtype, dev)
    if job.quantization != "none":                  # QLoRA: the block projections are stored packed, adapters stay in full precision
        from ..lora.portable import quantize_base_portable
        saved = quantize_base_portable(model, job.quantization, job.quant_block_size, job.double_quant)
        log.info("base projections stored as %s: %.1f MiB saved", job.quantization, saved / 2 ** 20)
    phase("loading_tokenizer")
    tok = Tokenizer.from_model_dir(model_dir)
    template = ChatTemplate.from_model_dir(model_dir, job.model)
    max_seq = tcfg.max_seq_len if tcfg.max_seq_len and tcfg.max_seq_len != 8192 else 2048
    phase("tokenizing_dataset")
    ds = TrainingDataset.from_file_tokenized(job.dataset, tok, max_seq, job.dataset_format, template, job.custom_columns,
                                             job.max_samples)
    log.info("dataset: %s", ds.stats())
    apply_lora_portable(model, job.lora, seed=tcfg.seed)
    if job.resume and os.path.exists(os.path.join(out_dir, "lora_weights.safetensors")):
        load_adapter_portable(model, out_dir)
    model.train()
    import inspect
    packing = (job.use_packing and tcfg.use_packing and hasattr(model, "forward_hidden")
               and "doc_ids" in inspect.signature(model.forward_hidden).parameters)
    if packing:
        # several documents per row: positions restart and attention stays inside each document (models/architectures/
        # generic.py: doc_ids); on a GPU the rows run on the varlen flash-attention kernels
        from ..data.dataloader import PackedDataLoader
        from ..data.packing import compute_pack_seq_len
        pack_len = job.pack_max_seq_len or compute_pack_seq_len([len(s) for s in ds.samples], max_seq)
        loader = PackedDataLoader(ds.samples, pack_len, tcfg.batch_size, True, tcfg.seed, 0, 1, tok.pad_token_id or 0)
        log.info("packing: %s", loader.stats.summary())
    else:
        loader = DataLoader(ds.samples, tcfg.batch_size, True, tcfg.seed, tok.pad_token_id or 0, max_seq)
    accum = max(tcfg.gradient_accumulation_steps, 1)
    per_epoch = max(len(loader) // accum, 1)        # optimiser steps per epoch: ``accum`` micro-batches each
    total = tcfg.max_steps or per_epoch * tcfg.num_epochs
    tr = PortableLoraTrainer(model, tcfg.learning_rate, tcfg.weight_decay, tcfg.max_grad_norm, tcfg.warmup_steps, total,
                             getattr(tcfg, "lr_scheduler", "cosine"), job.lora.loraplus_lr_ratio)
    state_path = os.path.join(out_dir, "portable_trainer_state.pt")
    step, running, tokens, epoch = 0, 0.0, 0, 0
    if job.resume and os.path.exists(state_path):
        sd = torch.load(state_path, map_location="cpu", weights_only=True)
        tr.load_state_dict(sd["trainer"])
        step, running, tokens, epoch = int(sd["step"]), float(sd["running"]), int(sd["tokens"]), int(sd["epoch"])
        log.info("resumed the portable trainer at step %d (epoch %d)", step, epoch)

    def save_state():
        torch.save({"trainer": tr.state_dict(), "step": step, "running": running, "tokens": tokens, "epoch": epoch},
                   state_path)
    cbs = callbacks + [LoggingCallback(tcfg.logging_steps)]
    if job.log_metrics:
        cbs.append(MetricsJsonCallback(job.log_metrics, config={"lora": dataclasses.asdict(job.lora),
                                                                "training": dataclasses.asdict(tcfg)}))
    cb = CompositeCallback(cbs)
    phase("training")
    cb.on_train_start()
    done = step >= total
    micro, acc_loss, acc_tok = 0, 0.0, 0
    t0 = time.perf_counter()
    while not done:
        loader.set_epoch(epoch)
        for batch in loader:
            if packing:
                rows = batch.input_ids.numel() // pack_len
                ids = batch.input_ids.view(rows, pack_len).to(dev)
                labels = batch.labels.view(rows, pack_len).to(dev)
                acc_loss += tr.micro_step(ids, labels, 1.0 / accum, batch.position_ids.view(rows, pack_len).to(dev).long(),
                                          batch.seq_start.view(rows, pack_len).to(dev).long())
                acc_tok += int(batch.total_tokens)
            else:
                ids, labels = batch["input_ids"].to(dev), batch["labels"].to(dev)
                acc_loss += tr.micro_step(ids, labels, 1.0 / accum)
                acc_tok += int(batch.get("tokens", ids.numel()))
            micro += 1
            if micro < accum:
                continue
            st = tr.optimizer_step()
            st["loss"] = acc_loss / accum
            step += 1
            tokens += acc_tok
            running = st["loss"] if step == 1 else 0.99 * running + 0.01 * st["loss"]
            dt = max(time.perf_counter() - t0, 1e-9)
            cb.on_step_end_with_metrics(StepMetrics(step=step, epoch=epoch, total_epochs=tcfg.num_epochs, total_steps=total,
                                                    loss=st["loss"], lr=st["lr"], tok_sec=acc_tok / dt,
                                                    total_ms=dt * 1e3, tokens=acc_tok, grad_norm=st["grad_norm"]))
            micro, acc_loss, acc_tok, t0 = 0, 0.0, 0, time.perf_counter()
            if tcfg.save_steps and step % tcfg.save_steps == 0:
                save_adapter_portable(model, out_dir, job.lora, base_model=job.model)
                save_state()
            if step >= total or cb.should_stop():
                done = True
                break
        epoch += 1
        if epoch >= tcfg.num_epochs and not tcfg.max_steps:
            done = True
    cb.on_train_end()
    phase("saving")
    adapter = save_adapter_portable(model, out_dir, job.lora, base_model=job.model)
    save_state()
    return {"steps": step, "final_loss": running, "tokens": tokens, "seconds": time.time() - t_start, "adapter": adapter,
            "output": out_dir, "path": "portable"}


def run_training(job: TrainingJobConfig, phase_cb: Optional[Callable[[str], None]] = None,
                 callbacks: Optional[List[TrainingCallback]] = None, sink=None) -> dict:
    from ..data.chat_templates import ChatTemplate
    from ..data.dataloader import DataLoader, PackedDataLoader
    from ..data.dataset import TrainingDataset
    from ..data.packing import compute_pack_seq_len
    from ..data.tokenizer import ByteTokenizer, Tokenizer
    from ..lora import apply_lora, load_adapter, save_adapter
    from ..models.loader import load_pretrained
    from .adaptive_lr import AdaptiveLrController
    from .checkpoint import CheckpointManager
    from .loop import TrainingLoop

    sink = sink or NullSink()
    sink.emit(JobEvent.started(job.job_id, "train"))

    def phase(name: str):
        sink.emit(JobEvent.phase(job.job_id, name))
        if phase_cb:
            phase_cb(name)
        log.info("phase: %s", name)

    t_start = time.time()
    try:
        out_dir = os.path.abspath(job.output)
        os.makedirs(out_dir, exist_ok=True)
        tcfg = job.training
        tcfg.output_dir = out_dir
        torch.manual_seed(tcfg.seed)
        # ---- distributed context
        dctx = None
        if job.distributed or int(os.environ.get("WORLD_SIZE", "1")) > 1:
            if job.dp_impl == "fused" and torch.cuda.is_available():
                from ..parallel.dp import DistContext
                DistContext.from_env()
                from ..parallel.fused_dp import FusedDataParallel
                dctx = FusedDataParallel()
            else:
                from ..parallel.dp import DistContext
                dctx = DistContext.from_env()
        rank = dctx.rank if dctx else 0
        world = dctx.world_size if dctx else 1
        dev = torch.device(job.device) if job.device else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        dtype = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[job.dtype]
        if dev.type == "cpu":
            dtype = torch.float32
        # ---- model
        phase("resolving_model")
        portable_dir = _portable_model_dir(job.model)
        if portable_dir is not None:
            summary = _run_portable_training(job, portable_dir, dev, dtype, out_dir, phase, list(callbacks or []), t_start)
            sink.emit(JobEvent.completed(job.job_id, **summary))
            return summary
        phase("loading_model")
        model, margs, model_dir = load_pretrained(job.model, dtype, dev, seed=tcfg.seed)
        max_seq = tcfg.max_seq_len if tcfg.max_seq_len and tcfg.max_seq_len != 8192 else min(
            margs.max_position_embeddings, 8192)
        # ---- tokenizer + dataset
        phase("loading_tokenizer")
        tok = Tokenizer.from_model_dir(model_dir) if model_dir else ByteTokenizer()
        template = ChatTemplate.from_model_dir(model_dir, job.model) if model_dir else None
        phase("tokenizing_dataset")
        ds = TrainingDataset.from_file_tokenized(job.dataset, tok, max_seq, job.dataset_format, template,
                                                 job.custom_columns, job.max_samples)
        stats = ds.stats()
        log.info("dataset: %s", stats)
        eval_ds = None
        if job.eval_dataset:
            eval_ds = TrainingDataset.from_file_tokenized(job.eval_dataset, tok, max_seq, job.dataset_format, template,
                                                          job.custom_columns)
        # ---- expert parallelism: the (frozen) expert stacks are cut over the ranks before anything else looks at them;
        # adapters on the replicated projections keep going through the data-parallel exchange
        if job.expert_parallel and world > 1 and getattr(model.cfg, "num_experts", 0):
            from ..parallel.ep_train import shard_experts_for_training
            n_ep = shard_experts_for_training(model)
            log.info("expert parallelism: %d layers, %d of %d experts on this rank", n_ep,
                     model.cfg.num_experts // world, model.cfg.num_experts)
            job.use_cuda_graph = False           # the token exchange sizes its messages on the host every step
        # ---- adapters
        if job.quantization != "none":
            from ..lora.qlora import quantize_base
            quantize_base(model, job.quantization, job.quant_block_size, job.double_quant)
        apply_lora(model, job.lora, seed=tcfg.seed)
        if job.gradient_checkpointing_layers:
            model.gradient_checkpointing = job.gradient_checkpointing_layers
        if job.activation_policy:
            from ..utils import offload as off
            n_layers = len(model.layers)
            if job.activation_policy == "smart":
                used = 0.0
                if torch.cuda.is_available() and model.embed_tokens.is_cuda:
                    free, total = torch.cuda.mem_get_info(model.embed_tokens.device)
                    used = (total - free) / total
                sc = off.SmartCheckpointConfig().with_cpu_offload()
                plan = off.plan_decoder_layers(sc, n_layers, bool(getattr(model.cfg, "num_experts", 0)), used)
            else:
                plan = [job.activation_policy.replace("-", "_")] * n_layers
            off.apply_to_model(model, plan, off.OffloadConfig(offload_dir=job.offload_dir))
            job.use_cuda_graph = False           # host copies and recomputation do not replay from a captured step
        model.prepare_for_training()
        cbs = list(callbacks or []) + [LoggingCallback(tcfg.logging_steps)]
        if not isinstance(sink, NullSink) and rank == 0:
            from ..core.callbacks import EventSinkCallback
            cbs.append(EventSinkCallback(sink, job.job_id))      # per-step metric events for the front ends
        if getattr(job, "tensorboard_dir", None) and rank == 0:
            from ..core.callbacks import TensorBoardCallback
            cbs.append(TensorBoardCallback(job.tensorboard_dir))
        if job.log_metrics and rank == 0:
            cbs.append(MetricsJsonCallback(job.log_metrics, config={"lora": dataclasses.asdict(job.lora),
                                                                    "training": dataclasses.asdict(tcfg)}))
        ckpt = CheckpointManager(os.path.join(out_dir, "checkpoints"), keep=3) if rank == 0 else None
        adaptive = AdaptiveLrController.lora_preset(os.path.join(out_dir, ".lr_control.json")) if job.adaptive_lr else None
        # ---- loaders
        use_pack = job.use_packing and tcfg.use_packing
        if use_pack:
            pack_len = job.pack_max_seq_len or compute_pack_seq_len([len(s) for s in ds.samples], max_seq)
            if os.environ.get("PMETAL_PY_LOADER") == "1":     # pure-Python packer and collation (same batches)
                loader = PackedDataLoader(ds.samples, pack_len, job.packs_per_batch or tcfg.batch_size, True, tcfg.seed,
                                          rank, world, tok.pad_token_id or 0)
            else:                                              # native packer, collation into pinned buffers
                from ..data.fastpack import FastPackedLoader, TokenStore
                loader = FastPackedLoader(TokenStore.from_samples(ds.samples), pack_len,
                                          job.packs_per_batch or tcfg.batch_size, True, tcfg.seed, rank, world,
                                          tok.pad_token_id or 0)
            log.info("packing: %s", loader.stats.summary())
            if loader.stats.max_sequences_per_batch <= 1:     # nothing gained: fall back (run_packed.rs:99-105)
                use_pack = False
        if not use_pack:
            loader = DataLoader(ds.samples, tcfg.batch_size, True, tcfg.seed, tok.pad_token_id or 0, max_seq, rank, world)
        eval_loader = None
        if eval_ds is not None:
            eval_loader = DataLoader(eval_ds.samples, tcfg.batch_size, False, tcfg.seed, tok.pad_token_id or 0, max_seq)
        per_epoch = max(len(loader) // max(tcfg.gradient_accumulation_steps, 1), 1)
        total_steps = tcfg.max_steps or per_epoch * tcfg.num_epochs
        loop = TrainingLoop(model, tcfg, cbs, dctx, job.lora.loraplus_lr_ratio, checkpoint_manager=ckpt,
                            adaptive_lr=adaptive, total_steps=total_steps)
        if job.resume:
            # every rank restores the same checkpoint (parameters, step, epoch, optimizer moments): rank 0 names it,
            # the others read the same directory; only the writes stay on rank 0
            latest = ckpt.latest_path() if ckpt is not None else None
            if dctx is not None:
                latest = dctx.broadcast_object(latest, src=0)
            if latest:
                loop.resume(latest)
                log.info("rank %d resumed from %s at step %d", rank, latest, loop.state.step)
        if getattr(job, "resume_bundle", None):
            from ..parallel.cloud_bridge import import_bundle
            params, _opt, meta = import_bundle(job.resume_bundle)
            loop.load_lora_tensors(params)
            loop.state.step = int(meta.get("step", 0))
            log.info("continued from bundle %s at step %d", job.resume_bundle, loop.state.step)
        phase("training")
        state = loop.run(loader, eval_loader)
        # ---- save
        phase("saving")
        adapter_path = None
        if rank == 0:
            adapter_path = save_adapter(model, out_dir, job.lora, base_model=job.model)
        if dctx:
            dctx.barrier()
        summary = {"steps": state.step, "final_loss": state.running_loss, "tokens": state.tokens_seen,
                   "seconds": time.time() - t_start, "adapter": adapter_path, "output": out_dir}
        sink.emit(JobEvent.completed(job.job_id, **summary))
        return summary
    except BaseException as e:
        sink.emit(JobEvent.failed(job.job_id, f"{type(e).__name__}: {e}"))
        raise
