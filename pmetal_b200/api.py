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
        m, tok, tpl, eos, mdir = _load_for_inference(SimpleNamespace(model=path, lora=lora, device=device, fp8=fp8, seed=0))
        return cls(m, tok, tpl, eos, mdir)

    def _generator(self):
        if self._gen is None:
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
        res = self._generator().generate([self._encode(prompt, system, chat)], sp, self.eos_ids)
        return self.tokenizer.decode([t for t in res.tokens[0] if t not in self.eos_ids])

    def stream(self, prompt: str, max_tokens: int = 256, temperature: float = 0.7, **kw) -> Iterator[str]:
        from .data.tokenizer import StreamDecoder
        from .models.sampling import SamplingParams
        sp = SamplingParams.greedy(max_tokens) if temperature <= 0 else SamplingParams(temperature=temperature, max_tokens=max_tokens)
        dec = StreamDecoder(self.tokenizer)
        for t in self._generator().stream(self._encode(prompt, kw.get("system"), kw.get("chat", False)), sp, self.eos_ids):
            if t not in self.eos_ids:
                piece = dec.push(t)
                if piece:
                    yield piece

    def save(self, out_dir: str, merged: bool = True) -> None:
        from .models.loader import save_pretrained
        save_pretrained(self.model, out_dir, merged=merged, copy_from=self.model_dir)


def infer(model: str, prompt: str, lora: Optional[str] = None, **kw) -> str:
    return Model.load(model, lora).generate(prompt, **kw)
