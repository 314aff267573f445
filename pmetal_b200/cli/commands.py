"""Sub-commands other than ``train``. Each ``cmd_*`` imports its subsystem lazily."""
from __future__ import annotations

import json
import os
import sys


def register(sp) -> None:
    for fn in list(globals().values()):
        if callable(fn) and getattr(fn, "_register", None):
            fn._register(sp)


def _command(setup):
    def deco(fn):
        def reg(sp):
            p = setup(sp)
            p.set_defaults(func=fn)
        fn._register = reg
        return fn
    return deco


# ------------------------------------------------------------------------------------------- info / memory
def _info_args(sp):
    return sp.add_parser("info", help="device, interconnect and library information")


@_command(_info_args)
def cmd_info(a) -> int:
    from ..utils.sysinfo import system_info
    print(json.dumps(system_info(), indent=2))
    return 0


def _memory_args(sp):
    p = sp.add_parser("memory", help="estimate memory use and throughput for a model on this device")
    p.add_argument("-m", "--model", required=True)
    p.add_argument("--seq-len", type=int, default=4096)
    p.add_argument("--batch-size", type=int, default=1)
    p.add_argument("--lora-r", type=int, default=16)
    p.add_argument("--quantization", default="none")
    return p


@_command(_memory_args)
def cmd_memory(a) -> int:
    from ..utils.sysinfo import estimate_fit
    print(json.dumps(estimate_fit(a.model, a.seq_len, a.batch_size, a.lora_r, a.quantization), indent=2))
    return 0


# ------------------------------------------------------------------------------------------- init
def _init_args(sp):
    p = sp.add_parser("init", help="write a starter YAML training config")
    p.add_argument("-o", "--output", default="pmetal.yaml")
    return p


@_command(_init_args)
def cmd_init(a) -> int:
    import yaml
    from ..core.config import FullTrainingConfig
    d = FullTrainingConfig().to_dict()
    d["model"]["model_id"] = "Qwen/Qwen3-0.6B"
    d["dataset"]["dataset_id"] = "train.jsonl"
    d.pop("distributed", None)
    with open(a.output, "w", encoding="utf-8") as fh:
        yaml.safe_dump(d, fh, sort_keys=False)
    print(a.output)
    return 0


# ------------------------------------------------------------------------------------------- tokenize
def _tokenize_args(sp):
    p = sp.add_parser("tokenize", help="tokenise text with a model's tokenizer")
    p.add_argument("-m", "--model", required=True)
    p.add_argument("text", nargs="?")
    p.add_argument("--decode", default=None, help="comma separated ids to decode")
    return p


@_command(_tokenize_args)
def cmd_tokenize(a) -> int:
    from ..data.tokenizer import Tokenizer
    from ..models.loader import resolve_model_path
    tok = Tokenizer.from_model_dir(resolve_model_path(a.model))
    if a.decode:
        print(tok.decode([int(x) for x in a.decode.split(",")]))
    else:
        text = a.text if a.text is not None else sys.stdin.read()
        ids = tok.encode_with_special_tokens(text)
        print(json.dumps({"ids": ids, "count": len(ids)}))
    return 0


# ------------------------------------------------------------------------------------------- dataset
def _dataset_args(sp):
    p = sp.add_parser("dataset", help="dataset tools")
    s = p.add_subparsers(dest="dataset_cmd")
    an = s.add_parser("analyze")
    an.add_argument("path")
    an.add_argument("-m", "--model", default=None)
    an.add_argument("--max-seq-len", type=int, default=8192)
    cv = s.add_parser("convert")
    cv.add_argument("path")
    cv.add_argument("-o", "--output", required=True)
    cv.add_argument("--to", default="openai", choices=["openai", "simple"])
    dl = s.add_parser("download")
    dl.add_argument("dataset_id")
    return p


@_command(_dataset_args)
def cmd_dataset(a) -> int:
    from ..data import dataset as ds
    from ..data.tokenizer import ByteTokenizer, Tokenizer
    if a.dataset_cmd == "analyze":
        tok = ByteTokenizer()
        if a.model:
            from ..models.loader import resolve_model_path
            tok = Tokenizer.from_model_dir(resolve_model_path(a.model))
        d = ds.TrainingDataset.from_file_tokenized(a.path, tok, a.max_seq_len)
        st = d.stats()
        st["format"] = d.format
        from ..data.packing import compute_pack_seq_len
        st["suggested_pack_len"] = compute_pack_seq_len([len(s) for s in d.samples], a.max_seq_len)
        print(json.dumps(st, indent=2))
        return 0
    if a.dataset_cmd == "convert":
        recs = ds.read_records(a.path)
        fmt = ds.detect_format(recs[0])
        with open(a.output, "w", encoding="utf-8") as fh:
            for r in recs:
                ts = ds.parse_record(r, fmt)
                if a.to == "simple":
                    fh.write(json.dumps({"text": ts.text}) + "\n")
                else:
                    p = ts.prompt or ""
                    fh.write(json.dumps({"messages": [{"role": "user", "content": p},
                                                      {"role": "assistant", "content": ts.text[len(p):]}]}) + "\n")
        print(json.dumps({"converted": len(recs), "from": fmt, "to": a.to}))
        return 0
    print("dataset download needs network access, which this machine does not have", file=sys.stderr)
    return 2
