"""Python convenience API (the counterpart of the reference's ``pmetal`` Python module: crates/pmetal-py/src/easy.rs,
trainer.rs, model.rs — ``finetune``, ``infer``, ``Trainer``, ``Model``, ``Tokenizer``).

    import pmetal_b200 as pm
    pm.finetune("path/to/model", "data.jsonl", output="./out", lora_r=16, epochs=1)
    model = pm.Model.load("path/to/model", lora="./out")
    print(model.generate("Hello", max_tokens=64))"""
from __future__ import annotations

from typing import Iterator, List, Optional


def finetune(model: str, dataset: str, output: str = "./output", lora_r: int = 16, lora_alpha: float = 32.0,
             learning_rate: float = 2e-4, epochs: int = 1, max_steps: Optional[int] = None, batch_size: int = 1,
             quantization: str = "none", max_seq_len: int = 0, **kw) -> dict:
    from .trainer.orchestrator import TrainingJobConfig, run_training
    job = TrainingJobConfig()
    job.model, job.dataset, job.output = model, dataset, output
    job.lora.r, job.lora.alpha = lora_r, lora_alpha
    t = job.training
    t.learning_rate, t.num_epochs, t.batch_size = learning_rate, epochs, batch_size
    if max_steps:
        t.max_steps = max_steps
    if max_seq_len:
        t.max_seq_len = max_seq_len
    job.quantization = quantization
    for k, v in kw.items():
        if hasattr(job, k):
            setattr(job, k, v)
        elif hasattr(t, k):
            setattr(t, k, v)
        else:
            raise TypeError(f"unknown option {k!r}")
    return run_training(job)


class Model:
    def __init__(self, model, tokenizer, template, eos_ids, model_dir=None):
        self.model, self.tokenizer, self.template, self.eos_ids, self.model_dir = model, tokenizer, template, eos_ids, model_dir
        self._gen = None

    @classmethod
    def load(cls, path: str, lora: Optional[str] = None, device: Optional[str] = None, fp8: bool = False) -> "Model":
        from types import SimpleNamespace

        from .cli.commands import _load_for_inference
        from .trainer.orchestrator import _portable_model_dir
        pdir = _portable_model_dir(path)
        if pdir is not None:                       # a config-driven architecture (Gemma, Phi, Cohere, ...)
            return cls._load_portable(pdir, lora, device)
        m, tok, tpl, eos, mdir = _load_for_inference(SimpleNamespace(model=path, lora=lora, device=device, fp8=fp8, seed=0))
        return cls(m, tok, tpl, eos, mdir)

    @classmethod
    def _load_portable(cls, model_dir: str, lora: Optional[str], device: Optional[str]) -> "Model":
        import torch

        from .data.chat_templates import ChatTemplate
        from .data.inference_config import collect_all_stop_tokens
        from .data.tokenizer import Tokenizer
        from .models.architectures import load_pretrained as load_portable
        dev = device or ("cuda" if torch.cuda.is_available() else "cpu")
        m = load_portable(model_dir, torch.bfloat16 if dev.startswith("cuda") else torch.float32, dev).eval()
        if lora:
            from .lora.adapter import load_adapter_config
            from .lora.portable import apply_lora_portable, load_adapter_portable, merge_lora_portable
            apply_lora_portable(m, load_adapter_config(lora))
            load_adapter_portable(m, lora)
            merge_lora_portable(m)
        for p in m.parameters():
            p.requires_grad_(False)
        tok, tpl = Tokenizer.from_model_dir(model_dir), ChatTemplate.from_model_dir(model_dir)
        return cls(m, tok, tpl, collect_all_stop_tokens(model_dir, tok, tpl.eos()), model_dir)

    @property
    def architecture(self) -> str:
        """The ``model_type`` of the checkpoint (llama, qwen3, qwen3_moe, gemma3, ...)."""
        for holder in (getattr(self.model, "cfg", None), getattr(self.model, "c", None)):
            mt = getattr(holder, "model_type", None)
            if mt:
                return str(mt)
        cfg = getattr(self.model, "config", None)
        if isinstance(cfg, dict) and cfg.get("model_type"):
            return str(cfg["model_type"])
        return type(self.model).__name__

    @property
    def portable(self) -> bool:
        return not hasattr(self.model, "fused_linears")

    def _generator(self):
        if self._gen is None:
            if self.portable:
                from .serve.portable_engine import PortableEngine
                self._gen = PortableEngine(self.model, self.eos_ids)
            else:
                from .models.generation import Generator
                self._gen = Generator(self.model)
        return self._gen

    def _encode(self, prompt, system=None, chat=False) -> List[int]:
        if chat or system:
            from .data.chat_templates import Message
            msgs = ([Message("system", system)] if system else []) + [Message("user", prompt)]
            return self.tokenizer.encode_with_special_tokens(self.template.apply_inference(msgs))
        return self.tokenizer.encode(prompt)

    def generate(self, prompt: str, max_tokens: int = 256, temperature: float = 0.7, system: Optional[str] = None,
                 chat: bool = False, **sampling) -> str:
        from .models.sampling import SamplingParams
        sp = SamplingParams.greedy(max_tokens) if temperature <= 0 else SamplingParams(temperature=temperature,
                                                                                        max_tokens=max_tokens, **sampling)
        if self.portable:
            req = self._generator().generate(self._encode(prompt, system, chat), sp)
            return self.tokenizer.decode([t for t in req.output if t not in self.eos_ids])
        res = self._generator().generate([self._encode(prompt, system, chat)], sp, self.eos_ids)
        return self.tokenizer.decode([t for t in res.tokens[0] if t not in self.eos_ids])

    def stream(self, prompt: str, max_tokens: int = 256, temperature: float = 0.7, **kw) -> Iterator[str]:
        from .data.tokenizer import StreamDecoder
        from .models.sampling import SamplingParams
        sp = SamplingParams.greedy(max_tokens) if temperature <= 0 else SamplingParams(temperature=temperature, max_tokens=max_tokens)
        dec = StreamDecoder(self.tokenizer)
        if self.portable:
            from .serve.engine import Request
            eng = self._generator()
            req = eng.submit(Request(self._encode(prompt, kw.get("system"), kw.get("chat", False)), sp))
            sent = 0
            while not req.done.is_set() or sent < len(req.output):
                if not req.done.is_set():
                    eng.tick()
                while sent < len(req.output):
                    t = req.output[sent]
                    sent += 1
                    if t not in self.eos_ids:
                        piece = dec.push(t)
                        if piece:
                            yield piece
            return
        for t in self._generator().stream(self._encode(prompt, kw.get("system"), kw.get("chat", False)), sp, self.eos_ids):
            if t not in self.eos_ids:
                piece = dec.push(t)
                if piece:
                    yield piece

    def save(self, out_dir: str, merged: bool = True) -> None:
        if self.portable:
            from .models.architectures import save_pretrained as save_portable
            return save_portable(self.model, out_dir, copy_from=self.model_dir)
        from .models.loader import save_pretrained
        save_pretrained(self.model, out_dir, merged=merged, copy_from=self.model_dir)


def infer(model: str, prompt: str, lora: Optional[str] = None, **kw) -> str:
    return Model.load(model, lora).generate(prompt, **kw)


class Trainer:
    """Object form of :func:`finetune` (crates/pmetal-py/src/trainer.rs:69-360): configure, attach callbacks, ``train()``.

    Callbacks are ``core.callbacks.TrainingCallback`` objects, or any object with some of the methods ``on_train_start``,
    ``on_step_end(metrics)``, ``on_eval(metrics)``, ``on_train_end`` (duck-typed, as the reference accepts plain Python
    objects)."""

    def __init__(self, model_id: str, lora_config=None, training_config=None, dataset_path: str = "",
                 eval_dataset_path: Optional[str] = None, output: Optional[str] = None):
        from .core.config import LoraConfig, TrainingConfig
        from .trainer.orchestrator import TrainingJobConfig
        self.job = TrainingJobConfig()
        self.job.model, self.job.dataset, self.job.eval_dataset = model_id, dataset_path, eval_dataset_path
        self.job.lora = lora_config or LoraConfig()
        self.job.training = training_config or TrainingConfig()
        out = output or getattr(self.job.training, "output_dir", None)
        if out:
            self.job.output = out
        self.callbacks: list = []

    def add_callback(self, callback) -> None:
        self.callbacks.append(callback)

    def set_sequence_packing(self, enabled: bool) -> None:
        self.job.use_packing = bool(enabled)

    def set_gradient_checkpointing(self, enabled: bool, layers: int = 4) -> None:
        self.job.gradient_checkpointing_layers = layers if enabled else 0

    def set_fused_optimizer(self, enabled: bool) -> None:
        """Fused reduce + clip + AdamW step across GPUs (on) or NCCL all-reduce followed by separate kernels (off)."""
        self.job.dp_impl = "fused" if enabled else "nccl"

    set_metal_fused_optimizer = set_fused_optimizer          # the reference's name for the same switch

    def set_embedding_lr(self, lr: float) -> None:
        self.job.training.embedding_learning_rate = float(lr)

    def set_quantization(self, kind: str, block_size: int = 64, double_quant: bool = False) -> None:
        self.job.quantization, self.job.quant_block_size, self.job.double_quant = kind, block_size, double_quant

    def train(self) -> dict:
        from .core.callbacks import TrainingCallback
        from .trainer.orchestrator import run_training

        class _Duck(TrainingCallback):
            def __init__(self, obj):
                self.obj = obj

            def __getattribute__(self, name):
                if name.startswith("on_") or name == "should_stop":
                    obj = object.__getattribute__(self, "obj")
                    if hasattr(obj, name):
                        return getattr(obj, name)
                return object.__getattribute__(self, name)
        cbs = [c if isinstance(c, TrainingCallback) else _Duck(c) for c in self.callbacks]
        return run_training(self.job, callbacks=cbs)

    def __repr__(self) -> str:
        return f"Trainer(model={self.job.model!r}, dataset={self.job.dataset!r}, lora_r={self.job.lora.r})"


class GenerationConfig:
    """Sampling options of ``Model.generate`` (a thin, keyword-checked view of ``models.sampling.SamplingParams``)."""

    def __init__(self, **kw):
        from .models.sampling import SamplingParams
        self.params = SamplingParams(**kw)

    def __getattr__(self, name):
        return getattr(object.__getattribute__(self, "params"), name)


class DataLoaderConfig:
    def __init__(self, batch_size: int = 1, max_seq_len: int = 2048, shuffle: bool = True, seed: int = 42,
                 pad_token_id: int = 0, drop_last: bool = False):
        self.batch_size, self.max_seq_len, self.shuffle, self.seed = batch_size, max_seq_len, shuffle, seed
        self.pad_token_id, self.drop_last = pad_token_id, drop_last


def download_model(model_id: str, revision: str = "main", token: Optional[str] = None, cache_dir: Optional[str] = None) -> str:
    """Local path of a hub model: an existing directory or cached snapshot if there is one, else a (resumable,
    checksum-verified) download."""
    import os

    from . import hub
    from .models.loader import resolve_model_path
    try:
        path = resolve_model_path(model_id)
        if os.path.isdir(path):
            return path
    except Exception:
        pass
    return hub.download_model(model_id, revision=revision, token=token, dest_dir=cache_dir)


def download_file(model_id: str, filename: str, revision: str = "main", token: Optional[str] = None,
                  cache_dir: Optional[str] = None) -> str:
    from . import hub
    return hub.download_file(model_id, filename, dest_dir=cache_dir, revision=revision, token=token)


class DFlashGenerator:
    """Speculative generation with a DFlash block-diffusion draft (crates/pmetal-py/src/dflash.rs). ``generate`` takes
    and returns token ids: (prompt + generated tokens, acceptance metrics). Verification is greedy, so the output equals
    plain greedy decoding of the target."""

    def __init__(self, target_model: str, draft_model: str, device: Optional[str] = None):
        import torch

        from .models.dflash import DFlashDecoder, load_dflash_pair
        from .models.loader import is_hf_id, resolve_model_path
        self.device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        resolve = lambda m: m if m == "random" or m.startswith("random:") or not is_hf_id(m) else resolve_model_path(m)
        self.target_model, self.draft_model = target_model, draft_model
        self.target, self.draft, self.tokenizer = load_dflash_pair(resolve(target_model), resolve(draft_model), self.device)
        self.decoder = DFlashDecoder(self.target, self.draft)

    def generate(self, prompt_ids, max_new_tokens: int = 256, temperature: float = 0.0, stop_tokens=None,
                 speculative_tokens: Optional[int] = None, tree_budget: int = 0):
        if temperature > 0:
            raise ValueError("block-diffusion drafting verifies greedily: temperature must be 0")
        import time
        from .models.dflash import DFlashStats
        self.decoder.stats = DFlashStats()
        stops = tuple(stop_tokens or ())
        t0 = time.perf_counter()
        if tree_budget > 0:
            new = self.decoder.generate_tree(list(prompt_ids), max_new_tokens, tree_budget, speculative_tokens, stops)
        else:
            new = self.decoder.generate(list(prompt_ids), max_new_tokens, speculative_tokens, stops)
        dt = time.perf_counter() - t0
        st = self.decoder.stats
        return list(prompt_ids) + new, {"generated_tokens": len(new), "steps": len(st.acceptance_lengths),
                                         "avg_acceptance_length": st.avg_acceptance_length,
                                         "acceptance_rate": st.acceptance_rate, "tokens_per_s": len(new) / max(dt, 1e-9)}

    def close(self) -> None:
        self.decoder.close()

    def __repr__(self) -> str:
        return f"DFlashGenerator(target={self.target_model!r}, draft={self.draft_model!r}, device={self.device!r})"
