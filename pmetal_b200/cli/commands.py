"""Sub-commands other than ``train``. Each ``cmd_*`` imports its subsystem lazily."""
from __future__ import annotations

import json
import logging
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
    p = sp.add_parser("tokenize", help="tokenise text, or turn a JSONL / text corpus into pre-training token shards")
    p.add_argument("-m", "--model", "--tokenizer", dest="model", required=True)
    p.add_argument("text", nargs="?")
    p.add_argument("--text", dest="text_flag")
    p.add_argument("--decode", default=None, help="comma separated ids to decode")
    p.add_argument("-i", "--input", help="corpus file: JSONL (one document per line) or plain text (one document per line)")
    p.add_argument("-o", "--output", help="directory for shard_NNNNN.bin / .idx files")
    p.add_argument("--text-column", default="text")
    p.add_argument("--docs-per-shard", type=int, default=10000)
    return p


@_command(_tokenize_args)
def cmd_tokenize(a) -> int:
    from ..data.tokenizer import ByteTokenizer, Tokenizer
    from ..models.loader import resolve_model_path
    path = resolve_model_path(a.model)
    tok = ByteTokenizer() if path.startswith("random:") else Tokenizer.from_model_dir(path)
    if a.input:
        if not a.output:
            print("error: --output is required with --input", file=sys.stderr)
            return 2
        from ..data.streaming import ShardWriter
        os.makedirs(a.output, exist_ok=True)
        shard = docs = tokens = in_shard = 0
        writer = None
        with open(a.input, "r", encoding="utf-8", errors="replace") as fh:
            for line in fh:
                line = line.rstrip("\n")
                if not line.strip():
                    continue
                text = line
                if line.lstrip().startswith("{"):
                    try:
                        rec = json.loads(line)
                        text = rec.get(a.text_column) if isinstance(rec, dict) else None
                    except ValueError:
                        text = line
                if not isinstance(text, str) or not text:
                    continue
                ids = tok.encode(text)
                if tok.eos_token_id is not None:
                    ids = list(ids) + [tok.eos_token_id]          # documents are separated by the end-of-sequence token
                if writer is None:
                    writer = ShardWriter(os.path.join(a.output, f"shard_{shard:05d}.bin"))
                writer.add_document(ids)
                docs, tokens, in_shard = docs + 1, tokens + len(ids), in_shard + 1
                if in_shard >= a.docs_per_shard:
                    writer.close()
                    writer, shard, in_shard = None, shard + 1, 0
        if writer is not None:
            writer.close()
            shard += 1
        print(json.dumps({"shards": shard, "documents": docs, "tokens": tokens, "output": a.output}))
        return 0
    if a.decode:
        print(tok.decode([int(x) for x in a.decode.split(",")]))
    else:
        text = a.text if a.text is not None else (a.text_flag if a.text_flag is not None else sys.stdin.read())
        ids = tok.encode_with_special_tokens(text)
        print(json.dumps({"ids": ids, "count": len(ids)}))
    return 0


# ------------------------------------------------------------------------------------------- dataset
def _dataset_args(sp):
    p = sp.add_parser("dataset", help="dataset tools: analyze, validate, preview, convert, filter, split, merge, sample, "
                                      "template, prepare, formats, download")
    s = p.add_subparsers(dest="dataset_cmd")

    def io(q, out=True):
        q.add_argument("-i", "--input", required=True)
        if out:
            q.add_argument("-o", "--output", required=True)
    an = s.add_parser("analyze")
    an.add_argument("path", nargs="?")
    an.add_argument("-p", "--path", dest="path_flag")
    an.add_argument("-m", "--model", default=None)
    an.add_argument("--max-seq-len", type=int, default=8192)
    va = s.add_parser("validate")
    va.add_argument("path", nargs="?")
    va.add_argument("-p", "--path", dest="path_flag")
    va.add_argument("-m", "--model", default=None)
    va.add_argument("--max-seq-len", type=int, default=2048)
    pv = s.add_parser("preview")
    pv.add_argument("dataset_id")
    pv.add_argument("--split", default="train")
    pv.add_argument("-n", "--num", type=int, default=5)
    cv = s.add_parser("convert")
    cv.add_argument("path", nargs="?")
    cv.add_argument("-i", "--input", dest="path_flag")
    cv.add_argument("-o", "--output", required=True)
    cv.add_argument("--to", default="openai", choices=["openai", "simple"])
    cv.add_argument("--columns", help='column mapping, e.g. "instruction=problem,output=solution"')
    cv.add_argument("--shuffle", action="store_true")
    cv.add_argument("--seed", type=int, default=42)
    fl = s.add_parser("filter")
    io(fl)
    fl.add_argument("-m", "--model")
    fl.add_argument("--min-tokens", type=int)
    fl.add_argument("--max-tokens", type=int)
    fl.add_argument("--dedup", action="store_true")
    fl.add_argument("--pattern")
    fl.add_argument("--invert", action="store_true")
    fl.add_argument("--complete-only", action="store_true")
    sl = s.add_parser("split")
    io(sl, out=False)
    sl.add_argument("-o", "--output-dir", required=True)
    sl.add_argument("--val-ratio", type=float, default=0.1)
    sl.add_argument("--test-ratio", type=float, default=0.0)
    sl.add_argument("--seed", type=int, default=42)
    sl.add_argument("--stratify")
    mg = s.add_parser("merge")
    mg.add_argument("-i", "--inputs", nargs="+", required=True)
    mg.add_argument("-o", "--output", required=True)
    mg.add_argument("--shuffle", action="store_true")
    mg.add_argument("--seed", type=int, default=42)
    mg.add_argument("--interleave", action="store_true")
    mg.add_argument("--weights", help="comma-separated, one per input")
    sm = s.add_parser("sample")
    io(sm)
    sm.add_argument("-n", "--num", type=int, required=True)
    sm.add_argument("--seed", type=int, default=42)
    tp = s.add_parser("template")
    io(tp)
    tp.add_argument("--template", default="chatml")
    tp.add_argument("--system")
    tp.add_argument("-m", "--model")
    tp.add_argument("--add-generation-prompt", action="store_true")
    tp.add_argument("--mask-prompt", action="store_true")
    pr = s.add_parser("prepare")
    pr.add_argument("dataset")
    pr.add_argument("-o", "--output-dir", required=True)
    pr.add_argument("-m", "--model", required=True)
    pr.add_argument("--template", default="chatml")
    pr.add_argument("--max-seq-len", type=int, default=2048)
    pr.add_argument("--val-ratio", type=float, default=0.05)
    pr.add_argument("--seed", type=int, default=42)
    pr.add_argument("--no-dedup", action="store_true")
    pr.add_argument("--columns")
    s.add_parser("formats")
    dl = s.add_parser("download")
    dl.add_argument("dataset_id")
    dl.add_argument("--split", default="train")
    dl.add_argument("-o", "--output")
    dl.add_argument("--revision")
    return p


def _dataset_tokenizer(model):
    """(tokenizer, model directory) for ``--model``; the byte tokenizer for ``random:`` presets."""
    from ..data.tokenizer import ByteTokenizer, Tokenizer
    from ..models.loader import resolve_model_path
    if not model:
        return None, None
    path = resolve_model_path(model)
    if path.startswith("random:") or not os.path.exists(os.path.join(path, "tokenizer.json")):
        return ByteTokenizer(), None
    return Tokenizer.from_model_dir(path), path


@_command(_dataset_args)
def cmd_dataset(a) -> int:
    from ..data import dataset as ds
    from ..data import tools as dt
    from ..data.tokenizer import ByteTokenizer
    cmd = a.dataset_cmd
    path = getattr(a, "path", None) or getattr(a, "path_flag", None)
    if cmd in ("analyze", "validate", "convert") and not path:
        print("error: a dataset path is required", file=sys.stderr)
        return 2
    if cmd == "analyze":
        tok = _dataset_tokenizer(a.model)[0] or ByteTokenizer()
        d = ds.TrainingDataset.from_file_tokenized(path, tok, a.max_seq_len)
        st = d.stats()
        st["format"] = d.format
        from ..data.packing import compute_pack_seq_len
        st["suggested_pack_len"] = compute_pack_seq_len([len(s) for s in d.samples], a.max_seq_len)
        print(json.dumps(st, indent=2))
        return 0
    if cmd == "validate":
        rep = dt.validate(path, _dataset_tokenizer(a.model)[0], a.max_seq_len)
        print(json.dumps(rep, indent=2))
        return 0 if rep["ok"] else 1
    if cmd == "preview":
        if not os.path.exists(a.dataset_id):
            print("dataset preview of a hub id needs network access; pass a local file", file=sys.stderr)
            return 2
        print(json.dumps(dt.preview(a.dataset_id, a.num), indent=2, ensure_ascii=False))
        return 0
    if cmd == "convert":
        recs = dt.remap_columns(ds.read_records(path), a.columns)
        if a.shuffle:
            import random
            random.Random(a.seed).shuffle(recs)
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
    if cmd == "filter":
        try:
            kept, rep = dt.filter_records(ds.read_records(a.input), _dataset_tokenizer(a.model)[0], a.min_tokens, a.max_tokens,
                                          a.dedup, a.pattern, a.invert, a.complete_only)
        except ValueError as e:
            print(f"error: {e}", file=sys.stderr)
            return 2
        dt.write_jsonl(kept, a.output)
        print(json.dumps(rep))
        return 0
    if cmd == "split":
        parts = dt.split_records(ds.read_records(a.input), a.val_ratio, a.test_ratio, a.seed, a.stratify)
        rep = {}
        for name, rows in parts.items():
            if rows or name == "train":
                rep[name] = dt.write_jsonl(rows, os.path.join(a.output_dir, f"{name}.jsonl"))
        print(json.dumps(rep))
        return 0
    if cmd == "merge":
        w = [float(x) for x in a.weights.split(",")] if a.weights else None
        out = dt.merge_records([ds.read_records(p) for p in a.inputs], a.shuffle, a.seed, a.interleave, w)
        print(json.dumps({"merged": dt.write_jsonl(out, a.output), "inputs": len(a.inputs)}))
        return 0
    if cmd == "sample":
        print(json.dumps({"sampled": dt.write_jsonl(dt.sample_records(ds.read_records(a.input), a.num, a.seed), a.output)}))
        return 0
    if cmd == "template":
        out, rep = dt.apply_template(ds.read_records(a.input), a.template, a.system, _dataset_tokenizer(a.model)[1],
                                     a.add_generation_prompt, a.mask_prompt)
        dt.write_jsonl(out, a.output)
        print(json.dumps(rep))
        return 0
    if cmd == "prepare":
        if not os.path.exists(a.dataset):
            print("dataset prepare of a hub id needs network access; pass a local file", file=sys.stderr)
            return 2
        tok, mdir = _dataset_tokenizer(a.model)
        print(json.dumps(dt.prepare(a.dataset, a.output_dir, tok, mdir, a.template, a.max_seq_len, a.val_ratio, a.seed,
                                    not a.no_dedup, a.columns), indent=2))
        return 0
    if cmd == "formats":
        print(json.dumps(dt.formats(), indent=2))
        return 0
    print("dataset download needs network access, which this machine does not have", file=sys.stderr)
    return 2


# ------------------------------------------------------------------------------------------- shared helpers
def _load_for_inference(a):
    """(model, tokenizer, template, eos ids, model_dir) for commands that generate text."""
    import torch

    from ..data.chat_templates import ChatTemplate
    from ..data.tokenizer import ByteTokenizer, Tokenizer
    from ..models.loader import load_pretrained
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    dtype = torch.bfloat16 if dev.startswith("cuda") else torch.float32
    model, args, mdir = load_pretrained(a.model, dtype=dtype, device=dev, seed=getattr(a, "seed", 0) or 0,
                                        experts_dir=getattr(a, "experts_dir", None))
    if getattr(a, "ane", False):
        print("note: --ane has no effect on this hardware", file=sys.stderr)
    if getattr(a, "minimal", False):
        a.backend = "minimal"
    lora = getattr(a, "lora", None)
    if lora:
        from ..lora import apply_lora
        from ..lora.adapter import load_adapter, load_adapter_config
        apply_lora(model, load_adapter_config(lora))
        model.to(dev)
        load_adapter(model, lora)
    if getattr(a, "fp8", False) and dev.startswith("cuda"):
        from ..models.fp8 import quantize_model_fp8
        quantize_model_fp8(model)
    model.eval()
    for p in model.parameters():
        p.requires_grad_(False)
    if mdir and os.path.exists(os.path.join(mdir, "tokenizer.json")):
        tok = Tokenizer.from_model_dir(mdir)
        tpl = ChatTemplate.from_model_dir(mdir)
    else:
        tok, tpl = ByteTokenizer(), ChatTemplate("chatml")
    if mdir:
        from ..data.inference_config import collect_all_stop_tokens
        eos = collect_all_stop_tokens(mdir, tok, tpl.eos())
    else:
        eos = [i for i in (tok.eos_token_id,) if i is not None]
    return model, tok, tpl, eos, mdir


def _sampling_from_args(a, model_dir=None, template_type=None, thinking=False):
    """Explicit flags win over the ``--mode`` preset of the model family, which wins over the model's
    ``generation_config.json``, which wins over the global fallback (temperature 0.7, top-k 20, top-p 0.8)."""
    from ..data.inference_config import load_sampling_defaults
    from ..models.sampling import SamplingParams
    d = load_sampling_defaults(model_dir, template_type, getattr(a, "mode", "auto") or "auto", thinking,
                               use_preset=model_dir is not None)

    def pick(name):
        v = getattr(a, name, None)
        return getattr(d, name) if v is None else v
    temperature = pick("temperature")
    if getattr(a, "greedy", False) or temperature <= 0:
        return SamplingParams.greedy(a.max_tokens)
    return SamplingParams(temperature=temperature, top_k=pick("top_k"), top_p=pick("top_p"), min_p=pick("min_p"),
                          repetition_penalty=pick("repetition_penalty"), frequency_penalty=pick("frequency_penalty"),
                          presence_penalty=pick("presence_penalty"), max_tokens=a.max_tokens, seed=a.seed)


def _add_sampling_flags(p, defaults=None):
    d = defaults or {}
    p.add_argument("--temperature", type=float, default=d.get("temperature"))
    p.add_argument("--top-k", type=int, default=d.get("top_k"))
    p.add_argument("--top-p", type=float, default=d.get("top_p"))
    p.add_argument("--min-p", type=float, default=d.get("min_p"))
    p.add_argument("--repetition-penalty", type=float, default=d.get("repetition_penalty"))
    p.add_argument("--frequency-penalty", type=float, default=d.get("frequency_penalty"))
    p.add_argument("--presence-penalty", type=float, default=d.get("presence_penalty"))
    p.add_argument("--max-tokens", type=int, default=256)
    p.add_argument("--seed", type=int, default=None)
    p.add_argument("--greedy", action="store_true")


def _add_platform_flags(p, infer: bool = False) -> None:
    """Expert streaming, and the reference's Apple-only switches (accepted so that its command lines run unchanged)."""
    p.add_argument("--experts-dir", help="serve the routed experts of a mixture-of-experts model from this "
                                         "`pack-experts` directory instead of holding them in memory")
    p.add_argument("--ane", action="store_true", help="ignored: Apple Neural Engine path of the reference")
    p.add_argument("--ane-max-seq-len", type=int, default=None, help="ignored with --ane")
    p.add_argument("--ane-real-time", action="store_true", help="ignored with --ane")
    if infer:
        p.add_argument("--metal-sampler", action="store_true", help="ignored: sampling already runs on the device")
        p.add_argument("--minimal", action="store_true", help="same as --backend minimal (eager launches)")


# ------------------------------------------------------------------------------------------- infer
def _infer_args(sp):
    p = sp.add_parser("infer", help="generate text (paged KV cache, optional LoRA, speculative draft)")
    p.add_argument("-m", "--model", required=True)
    p.add_argument("-l", "--lora")
    p.add_argument("-p", "--prompt", required=True)
    p.add_argument("--system")
    p.add_argument("--chat", action="store_true", help="apply the chat template")
    p.add_argument("--no-thinking", action="store_true")
    p.add_argument("--hide-thinking", action="store_true", help="with --stream: do not print the reasoning channel")
    p.add_argument("--mode", default="auto", help="sampling preset of the model family: auto, thinking-general, "
                   "thinking-coding, instruct-general, instruct-reasoning")
    p.add_argument("--stream", action="store_true")
    p.add_argument("--draft-model", help="two-model speculative decoding with this draft")
    p.add_argument("--speculative-k", type=int, default=5)
    p.add_argument("--fp8", action="store_true", help="block-scaled FP8 weights")
    p.add_argument("--kv-blocks", type=int, default=4096)
    p.add_argument("--device")
    p.add_argument("--json", action="store_true")
    p.add_argument("--tools", help="JSON file with tool (function) definitions passed to the chat template")
    p.add_argument("--benchmark", action="store_true", help="time prefill and decode on a synthetic prompt")
    p.add_argument("--benchmark-iters", type=int, default=3)
    p.add_argument("--benchmark-prompt-tokens", type=int, default=512)
    p.add_argument("--backend", default="auto", choices=["auto", "standard", "compiled", "minimal", "dflash", "metal-sampler", "ane"],
                   help="auto / compiled: CUDA-graph decode; standard / minimal: eager launches")
    p.add_argument("--compiled", action="store_true", help="same as --backend compiled")
    p.add_argument("--detect-repetition", action="store_true", help="cut the output where it starts to loop")
    p.add_argument("--profile-layers", action="store_true", help="per-layer device timing of one forward pass")
    p.add_argument("--profile-output", help="write the --profile-layers table to this JSON file")
    _add_kv_quant_flags(p)
    _add_sampling_flags(p)
    _add_platform_flags(p, infer=True)
    return p


def _add_kv_quant_flags(p):
    """KV-cache flags (crates/pmetal/src/cli/infer.rs:150-180). On the fast path the paged cache holds bf16 or int8
    blocks (the attention kernel expands int8 blocks as it loads them); without flags int8 is chosen by itself when
    weights plus a 16-bit cache would not fit comfortably (``models.kv_cache.select_cache_mode``). Narrower widths and
    TurboQuant run on the portable models' cache (``GenericDecoderLM.new_cache(kv_bits=...)``). ``--kv-window`` /
    ``--kv-keep`` turn the cache into a rotating one: only the last N tokens (plus the first ``keep``) stay resident."""
    p.add_argument("--kv-quant", nargs="?", const=8, type=int, default=None, metavar="BITS",
                   help="quantise the KV cache (8 when no width is given; 0 = off)")
    p.add_argument("--no-kv-quant", action="store_true")
    p.add_argument("--kv-group-size", type=int, default=64)
    p.add_argument("--kv-k-bits", type=int)
    p.add_argument("--kv-v-bits", type=int)
    p.add_argument("--kv-qjl", action="store_true")
    p.add_argument("--kv-turboquant", action="store_true")
    p.add_argument("--kv-turboquant-preset")
    p.add_argument("--kv-quant-preset")
    p.add_argument("--kv-window", type=int, default=0, help="rotating cache: keep only the last N tokens")
    p.add_argument("--kv-keep", type=int, default=0, help="rotating cache: leading tokens that are never dropped")


def _paged_cache_options(a, model, num_blocks: int) -> dict:
    """Keyword arguments for ``DecoderLM.new_cache`` from the ``--kv-*`` flags and the memory estimate."""
    import torch
    from ..models.kv_cache import BLOCK, select_cache_mode
    cfg = model.cfg
    weight_bytes = sum(p.numel() * p.element_size() for p in model.parameters())
    kv16 = 2 * cfg.num_hidden_layers * num_blocks * BLOCK * cfg.num_key_value_heads * cfg.head_dim * 2
    dev = model.embed_tokens.device
    total = torch.cuda.get_device_properties(dev).total_memory if dev.type == "cuda" else None
    turbo = bool(a.kv_turboquant or a.kv_turboquant_preset or a.kv_quant_preset)
    mode = select_cache_mode(weight_bytes, kv16, total, a.kv_quant, a.no_kv_quant, a.kv_k_bits, a.kv_v_bits, turbo,
                             a.kv_group_size)
    quant = None
    if mode.kind != "standard":
        quant = "int8"
        if (mode.kind == "turboquant" or (mode.kind == "quantized" and mode.bits == 4)) and cfg.head_dim == 128 \
                and not a.kv_qjl:
            quant = "tq4"         # rotated 4-bit code-book cache (TurboQuant without the residual sketch)
        elif mode.kind != "quantized" or mode.bits != 8 or a.kv_group_size != 64 or a.kv_qjl:
            print(f"note: the paged cache stores bf16, int8 (group 64) or rotated 4-bit codes; using int8 instead of "
                  f"{mode.kind} k{mode.k_bits}/v{mode.v_bits} (other layouts run on the portable models)", file=sys.stderr)
        if cfg.head_dim % 64:
            quant = None
    if quant or a.kv_window:
        logging.getLogger("pmetal").info("kv cache: %s (%s)%s", quant or "bf16", mode.source,
                                         f", window {a.kv_window} keep {a.kv_keep}" if a.kv_window else "")
    return dict(quant=quant, window=int(a.kv_window or 0), sink=int(a.kv_keep or 0))


def cut_repetition(tokens, min_period: int = 1, max_period: int = 64, min_repeats: int = 4, min_span: int = 24):
    """Index at which ``tokens`` starts to loop, or None: the tail consists of one block of ``period`` tokens repeated
    at least ``min_repeats`` times over at least ``min_span`` tokens. The first copy of the block is kept."""
    n = len(tokens)
    for period in range(min_period, min(max_period, n // min_repeats) + 1):
        reps = 1
        while (reps + 1) * period <= n and tokens[n - (reps + 1) * period:n - reps * period] == tokens[n - period:]:
            reps += 1
        if reps >= min_repeats and reps * period >= min_span:
            return n - (reps - 1) * period
    return None


def _infer_benchmark(a, model, gen, sp_, eos) -> int:
    import torch
    g = torch.Generator().manual_seed(0)
    vocab = model.cfg.vocab_size
    rows = []
    for it in range(a.benchmark_iters + 1):                      # the first pass warms up (graph capture, caches)
        prompt = torch.randint(0, vocab, (a.benchmark_prompt_tokens,), generator=g).tolist()
        res = gen.generate([prompt], sp_, ())                     # no stop tokens: always max_tokens new tokens
        if it:
            rows.append((res.prefill_tok_per_s, res.decode_tok_per_s))
    pre = sorted(r[0] for r in rows)[len(rows) // 2]
    dec = sorted(r[1] for r in rows)[len(rows) // 2]
    print(json.dumps({"benchmark": "infer", "prompt_tokens": a.benchmark_prompt_tokens, "new_tokens": a.max_tokens,
                      "iters": a.benchmark_iters, "prefill_tok_per_s": round(pre, 1), "decode_tok_per_s": round(dec, 1),
                      "decode_ms_per_token": round(1e3 / dec, 3) if dec else None, "backend": a.backend}))
    return 0


def _infer_profile_layers(a, model, ids) -> int:
    """Device time of every decoder layer for one forward pass over the prompt (CUDA events; wall clock on CPU)."""
    import time

    import torch
    dev = next(model.parameters()).device
    cuda = dev.type == "cuda"
    marks = []

    def stamp():
        if cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            return e
        return time.perf_counter()
    hooks = []
    for i, layer in enumerate(model.layers):
        hooks.append(layer.register_forward_pre_hook(lambda m, x, i=i: marks.append((i, "start", stamp()))))
        hooks.append(layer.register_forward_hook(lambda m, x, y, i=i: marks.append((i, "end", stamp()))))
    t = torch.tensor(ids, dtype=torch.int64, device=dev)
    with torch.no_grad():
        for rep in range(2):                                       # the second pass is the measured one
            marks.clear()
            model(t)
    if cuda:
        torch.cuda.synchronize()
    for h in hooks:
        h.remove()
    start = {i: m for i, k, m in marks if k == "start"}
    table = []
    for i, k, m in marks:
        if k == "end":
            ms = start[i].elapsed_time(m) if cuda else (m - start[i]) * 1e3
            table.append({"layer": i, "ms": round(ms, 4)})
    rep = {"tokens": len(ids), "total_ms": round(sum(r["ms"] for r in table), 4), "layers": table}
    if a.profile_output:
        with open(a.profile_output, "w", encoding="utf-8") as fh:
            json.dump(rep, fh, indent=2)
    print(json.dumps(rep if a.json else {k: rep[k] for k in ("tokens", "total_ms")}))
    return 0


def _infer_portable(a, model_dir: str) -> int:
    """Generation with a portable architecture (Gemma, Phi, Cohere, Granite, DeepSeek, GPT-OSS, Llama 4, Mixtral, ...):
    contiguous KV cache (optionally quantised with --kv-quant / --kv-turboquant), the same sampler and stop tokens."""
    import time

    import torch

    from ..data.chat_templates import ChatTemplate, Message
    from ..data.inference_config import collect_all_stop_tokens
    from ..data.stream_format import StreamFormatter
    from ..data.tokenizer import Tokenizer
    from ..models.architectures import load_pretrained as load_portable
    from ..models.sampling import Sampler
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    dtype = torch.bfloat16 if dev.startswith("cuda") else torch.float32
    model = load_portable(model_dir, dtype, dev).eval()
    if a.lora:
        from ..lora.adapter import load_adapter_config
        from ..lora.portable import apply_lora_portable, load_adapter_portable, merge_lora_portable
        apply_lora_portable(model, load_adapter_config(a.lora))
        load_adapter_portable(model, a.lora)
        merge_lora_portable(model)
    tok = Tokenizer.from_model_dir(model_dir)
    tpl = ChatTemplate.from_model_dir(model_dir)
    eos = set(collect_all_stop_tokens(model_dir, tok, tpl.eos()))
    if a.chat or a.system:
        msgs = ([Message("system", a.system)] if a.system else []) + [Message("user", a.prompt)]
        ids = tok.encode_with_special_tokens(tpl.apply_inference(msgs, a.no_thinking))
    else:
        ids = tok.encode(a.prompt)
    sp_ = _sampling_from_args(a, model_dir, tpl.template_type, thinking=bool(a.chat or a.system) and not a.no_thinking)
    sampler = Sampler(sp_, torch.device(dev))
    kv_bits = None
    if a.kv_turboquant or a.kv_quant or a.kv_k_bits:
        kv_bits = a.kv_k_bits or (4 if a.kv_turboquant else (a.kv_quant if isinstance(a.kv_quant, int) and a.kv_quant > 0 else 8))
    cache = model.new_cache(kv_bits, a.kv_group_size, bool(a.kv_turboquant), bool(a.kv_qjl)) if hasattr(model, "new_cache") \
        else None
    if cache is None:
        print("error: this architecture has no text-generation head", file=sys.stderr)
        return 2
    if getattr(a, "draft_model", None):
        # two-model speculative decoding on the contiguous caches (models/architectures/speculative.py)
        from ..models.architectures.speculative import speculative_generate
        from ..trainer.orchestrator import _portable_model_dir
        ddir = _portable_model_dir(a.draft_model)
        if ddir is None:
            print("error: --draft-model must be a directory of a config-driven architecture for this target", file=sys.stderr)
            return 2
        if kv_bits is not None:
            print("error: speculative decoding keeps plain caches (no --kv-quant / --kv-turboquant)", file=sys.stderr)
            return 2
        draft = load_portable(ddir, dtype, dev).eval()
        t0 = time.perf_counter()
        st = speculative_generate(model, draft, ids, a.max_tokens, k=a.speculative_k, eos_ids=eos,
                                  temperature=0.0 if sp_.is_greedy else sp_.temperature)
        out = [t for t in st.tokens if t not in eos]
        dt = max(time.perf_counter() - t0, 1e-9)
        if a.json:
            print(json.dumps({"text": tok.decode(out), "prompt_tokens": len(ids), "generated_tokens": len(out),
                              "tok_per_s": round(len(out) / dt, 1), "path": "portable", "speculative": True,
                              "rounds": st.rounds, "acceptance_rate": round(st.acceptance_rate, 3)}))
        else:
            print(tok.decode(out))
        return 0
    fmt = StreamFormatter(tok, show_thinking=not a.hide_thinking) if a.stream and not a.json else None
    out, t0 = [], time.perf_counter()
    cur = torch.tensor([ids], device=dev)
    t_first = None
    with torch.no_grad():
        for _ in range(a.max_tokens):
            logits = model(cur, cache)[:, -1].float()
            nxt = int(sampler.sample(logits, None)[0])
            if t_first is None:
                t_first = time.perf_counter()
            if nxt in eos:
                break
            out.append(nxt)
            if fmt is not None:
                sys.stdout.write(fmt.push(nxt))
                sys.stdout.flush()
            cur = torch.tensor([[nxt]], device=dev)
    t1 = time.perf_counter()
    if fmt is not None:
        sys.stdout.write("\n")
        return 0
    text = tok.decode(out)
    if a.json:
        dec = max(t1 - (t_first or t1), 1e-9)
        print(json.dumps({"text": text, "prompt_tokens": len(ids), "generated_tokens": len(out),
                          "prefill_tok_per_s": round(len(ids) / max((t_first or t1) - t0, 1e-9), 1),
                          "decode_tok_per_s": round(max(len(out) - 1, 0) / dec, 1), "path": "portable",
                          "finish_reason": "length" if len(out) >= a.max_tokens else "stop"}))
    else:
        print(text)
    return 0


@_command(_infer_args)
def cmd_infer(a) -> int:
    from ..trainer.orchestrator import _portable_model_dir
    pdir = _portable_model_dir(a.model)
    if pdir is not None:
        return _infer_portable(a, pdir)
    from ..data.chat_templates import Message
    from ..data.stream_format import StreamFormatter
    from ..models.generation import Generator
    model, tok, tpl, eos, mdir = _load_for_inference(a)
    tools = None
    if a.tools:
        with open(a.tools, "r", encoding="utf-8") as fh:
            tools = json.load(fh)
    if a.chat or a.system or tools:
        msgs = ([Message("system", a.system)] if a.system else []) + [Message("user", a.prompt)]
        ids = tok.encode_with_special_tokens(tpl.apply_inference(msgs, a.no_thinking, tools))
    else:
        ids = tok.encode(a.prompt)
    sp_ = _sampling_from_args(a, mdir, tpl.template_type, thinking=bool(a.chat or a.system) and not a.no_thinking)
    if a.profile_layers:
        return _infer_profile_layers(a, model, ids)
    if a.draft_model:
        from ..models.loader import load_pretrained
        from ..models.speculative import SpeculativeConfig, SpeculativeDecoder
        draft, _, _ = load_pretrained(a.draft_model, dtype=next(model.parameters()).dtype,
                                      device=str(model.embed_tokens.device))
        draft.eval()
        sg = SpeculativeDecoder(model, draft, SpeculativeConfig(num_draft_tokens=a.speculative_k,
                                                                  temperature=0.0 if sp_.is_greedy else sp_.temperature))
        out = sg.generate([ids], a.max_tokens, eos)
        text = tok.decode([t for t in out[0] if t not in eos])
        info = {"text": text, "tokens": len(out[0]), "acceptance_rate": sg.stats.acceptance_rate,
                "tokens_per_round": sg.stats.tokens_per_round}
        print(json.dumps(info) if a.json else text)
        return 0
    graphs = None if a.backend == "auto" and not a.compiled else (a.compiled or a.backend == "compiled")
    gen = Generator(model, cache=model.new_cache(a.kv_blocks, **_paged_cache_options(a, model, a.kv_blocks)),
                    cuda_graphs=graphs)
    if a.benchmark:
        return _infer_benchmark(a, model, gen, sp_, eos)
    if a.stream and not a.json:
        dec = StreamFormatter(tok, show_thinking=not a.hide_thinking)
        for t in gen.stream(ids, sp_, eos):
            if t not in eos:
                sys.stdout.write(dec.push(t))
                sys.stdout.flush()
        sys.stdout.write("\n")
        return 0
    res = gen.generate([ids], sp_, eos)
    if a.detect_repetition:
        cut = cut_repetition(res.tokens[0])
        if cut is not None:
            res.tokens[0] = res.tokens[0][:cut]
            res.finish_reasons[0] = "repetition"
    text = tok.decode([t for t in res.tokens[0] if t not in eos])
    if a.json:
        print(json.dumps({"text": text, "prompt_tokens": res.prompt_tokens, "generated_tokens": res.generated_tokens,
                          "prefill_tok_per_s": round(res.prefill_tok_per_s, 1), "decode_tok_per_s": round(res.decode_tok_per_s, 1),
                          "finish_reason": res.finish_reasons[0]}))
    else:
        print(text)
    return 0


# ------------------------------------------------------------------------------------------- serve
def _serve_args(sp):
    p = sp.add_parser("serve", help="OpenAI / Anthropic compatible server with continuous batching")
    p.add_argument("-m", "--model", required=True)
    p.add_argument("-l", "--lora")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=8080)
    p.add_argument("--max-slots", "--cb-max-slots", dest="max_slots", type=int, default=64)
    p.add_argument("--kv-blocks", "--cb-max-blocks", dest="kv_blocks", type=int, default=8192)
    p.add_argument("--cb-block-size", type=int, default=64, help="KV block size; the attention kernels use 64")
    p.add_argument("--cb-max-queue-depth", type=int, default=1024, help="requests waiting for a slot before new ones are refused")
    p.add_argument("--continuous-batch", action="store_true", help="always on (accepted for compatibility)")
    p.add_argument("--max-seq-len", type=int, default=None, help="sizes the KV pool: slots x ceil(len / 64) blocks")
    p.add_argument("--fp8", action="store_true")
    p.add_argument("--device")
    p.add_argument("--adapter", action="append", default=[], metavar="NAME=DIR",
                   help="serve this LoRA adapter beside the base model (repeatable); a request selects it with "
                        "\"adapter\": NAME or \"model\": NAME, and requests with different adapters share a batch")
    _add_platform_flags(p)
    p.add_argument("--tp", type=int, default=1, help="cut attention heads (and dense feed-forward channels) over N GPUs")
    p.add_argument("--ep", type=int, default=0, help="cut experts over N GPUs (the same ranks as --tp; default: = --tp)")
    p.add_argument("--reduce", choices=["peer", "nccl"], default="nccl",
                   help="sum of the partial layer outputs: NCCL (in-switch reduction; measured faster at 8 ranks), or one "
                        "kernel over symmetric memory")
    _add_kv_quant_flags(p)
    return p


@_command(_serve_args)
def cmd_serve(a) -> int:
    from ..serve.server import serve
    if a.cb_block_size != 64:
        print("error: the paged attention kernels use 64-token blocks (--cb-block-size 64)", file=sys.stderr)
        return 2
    ways = max(a.tp, a.ep or a.tp)
    if a.ep and a.tp > 1 and a.ep != a.tp:
        print("error: heads and experts are cut over the same ranks (--ep must equal --tp)", file=sys.stderr)
        return 2
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if ways > 1 and world == 1:
        # one process per GPU: start this same command under the launcher
        from ..parallel.cluster_cli import _torchrun
        return _torchrun(ways, ["-m", "pmetal_b200.cli.main"] + sys.argv[1:])
    from ..trainer.orchestrator import _portable_model_dir
    pdir = _portable_model_dir(a.model) if world == 1 else None
    if pdir is not None:
        return _serve_portable(a, pdir)
    channel = None
    if world > 1:
        import torch
        import torch.distributed as dist
        local = int(os.environ.get("LOCAL_RANK", "0"))
        if torch.cuda.is_available():
            torch.cuda.set_device(local)
            a.device = f"cuda:{local}"
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        else:
            dist.init_process_group("gloo")
    model, tok, tpl, eos, mdir = _load_for_inference(a)
    blocks = a.kv_blocks
    if a.max_seq_len:
        blocks = max(blocks, a.max_slots * (-(-a.max_seq_len // 64) + 1))
    opts = _paged_cache_options(a, model, blocks)
    if world > 1:
        from ..parallel.dp import shutdown_process_group
        from ..parallel.tp_model import AllReduce, PeerAllReduce, shard_for_serving
        from ..serve.replica import StepChannel, follow
        red = PeerAllReduce(None) if (a.reduce == "peer" and a.device.startswith("cuda")) else AllReduce(None)
        shard_for_serving(model, None, red)
        channel = model.step_channel = StepChannel(StepChannel.control_group())
        if not channel.leader:
            cache = model.new_cache(blocks, **(opts or {}))
            try:
                steps = follow(model, cache, channel)
                logging.getLogger("pmetal").info("rank %d replayed %d steps", dist.get_rank(), steps)
            except KeyboardInterrupt:          # an interrupt of the whole process group ends the followers too
                return 0
            shutdown_process_group()
            return 0
    adapters = None
    if a.adapter:
        if world > 1:
            print("error: --adapter is not available together with --tp", file=sys.stderr)
            return 2
        from ..lora.adapter import load_adapter_config
        from ..lora.batched import AdapterSet
        pairs = [x.split("=", 1) if "=" in x else (os.path.basename(os.path.normpath(x)), x) for x in a.adapter]
        adapters = AdapterSet(model, len(pairs), load_adapter_config(pairs[0][1]).r)
        for name, path in pairs:
            adapters.load(name, path)
    try:
        serve(model, tok, tpl, a.host, a.port, eos, os.path.basename(os.path.normpath(mdir or a.model)), a.max_slots,
              blocks, a.cb_max_queue_depth, cache_options=opts, channel=channel, adapters=adapters)
    finally:
        if world > 1:
            from ..parallel.dp import shutdown_process_group
            shutdown_process_group()
    return 0


def _serve_portable(a, model_dir: str) -> int:
    """``serve`` for the config-driven architectures: same HTTP routes, requests interleaved token by token on the models'
    own contiguous caches (serve/portable_engine.py)."""
    import torch

    from ..data.chat_templates import ChatTemplate
    from ..data.inference_config import collect_all_stop_tokens
    from ..data.tokenizer import Tokenizer
    from ..models.architectures import load_pretrained as load_portable
    from ..serve.portable_engine import PortableEngine
    from ..serve.server import serve
    if a.tp > 1 or a.ep or a.adapter:
        print("error: --tp / --ep / --adapter serve the llama / qwen family only", file=sys.stderr)
        return 2
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    model = load_portable(model_dir, torch.bfloat16 if dev.startswith("cuda") else torch.float32, dev).eval()
    for p in model.parameters():
        p.requires_grad_(False)
    lora = getattr(a, "lora", None)
    if lora:
        from ..lora.adapter import load_adapter_config
        from ..lora.portable import apply_lora_portable, load_adapter_portable, merge_lora_portable
        apply_lora_portable(model, load_adapter_config(lora))
        load_adapter_portable(model, lora)
        merge_lora_portable(model)
    tok = Tokenizer.from_model_dir(model_dir)
    tpl = ChatTemplate.from_model_dir(model_dir)
    eos = collect_all_stop_tokens(model_dir, tok, tpl.eos())
    opts = {}
    if getattr(a, "kv_turboquant", False) or getattr(a, "kv_quant", None):
        bits = 4 if getattr(a, "kv_turboquant", False) else (a.kv_quant if isinstance(a.kv_quant, int) and a.kv_quant > 0 else 8)
        opts = dict(kv_bits=bits, turbo=bool(getattr(a, "kv_turboquant", False)))
    engine = PortableEngine(model, eos, max_slots=min(a.max_slots, 16), max_queue=a.cb_max_queue_depth, cache_options=opts)
    serve(model, tok, tpl, a.host, a.port, eos, os.path.basename(os.path.normpath(model_dir)), engine=engine)
    return 0


# ------------------------------------------------------------------------------------------- fuse / merge / quantize
def _fuse_args(sp):
    p = sp.add_parser("fuse", help="merge a LoRA adapter into its base model")
    p.add_argument("-m", "--model", required=True)
    p.add_argument("-l", "--lora", required=True)
    p.add_argument("-o", "--output", required=True)
    p.add_argument("--dtype", default="bfloat16")
    p.add_argument("--alpha", type=float, help="LoRA alpha (default: from adapter_config.json)")
    p.add_argument("--rank", type=int, help="LoRA rank (default: from adapter_config.json)")
    p.add_argument("--accurate", action="store_true", help="float64 accumulation (the default)")
    p.add_argument("--fast", action="store_true", help="float32 accumulation")
    p.add_argument("--low-memory", action="store_true", help="merge 1024 output rows at a time")
    return p


@_command(_fuse_args)
def cmd_fuse(a) -> int:
    from ..merge.merge import merge_lora_into_base
    from ..models.loader import resolve_model_path
    print(json.dumps(merge_lora_into_base(resolve_model_path(a.model), a.lora, a.output, a.dtype, a.alpha, a.rank,
                                          not a.fast, a.low_memory)))
    return 0


def _merge_args(sp):
    p = sp.add_parser("merge", help="merge models (linear, slerp, ties, dare, della, ...) from a YAML recipe or flags")
    p.add_argument("-c", "--config")
    p.add_argument("--models", nargs="*")
    p.add_argument("--model-a")
    p.add_argument("--model-b")
    p.add_argument("--t", type=float, default=None, help="slerp interpolation: 0 = model a, 1 = model b")
    p.add_argument("--sanity", choices=["off", "quick", "full"], default=None,
                   help="checks on every merged tensor: NaN / infinity counts (quick, the default) plus statistics (full)")
    p.add_argument("--align-experts", action="store_true",
                   help="mixture-of-experts models: match every model's experts to the first model's before merging")
    p.add_argument("--weight-a", type=float, default=None)
    p.add_argument("--weight-b", type=float, default=None)
    p.add_argument("--base")
    p.add_argument("--method", default="linear")
    p.add_argument("--weights", nargs="*", type=float)
    p.add_argument("--density", type=float, default=1.0)
    p.add_argument("-o", "--output", required=True)
    p.add_argument("--dtype", default="bfloat16")
    p.add_argument("--device")
    return p


@_command(_merge_args)
def cmd_merge(a) -> int:
    from ..merge.merge import MergeConfig, run_merge
    if a.config:
        cfg = MergeConfig.from_yaml(a.config)
    else:
        if a.model_a and a.model_b and not a.models:          # two-model form: --model-a / --model-b [--t | --weight-a/-b]
            a.models = [a.model_a, a.model_b]
            if a.weights is None and (a.weight_a is not None or a.weight_b is not None):
                a.weights = [a.weight_a if a.weight_a is not None else 0.5, a.weight_b if a.weight_b is not None else 0.5]
        if not a.models:
            print("error: --config, --models or --model-a/--model-b is required", file=sys.stderr)
            return 2
        ws = a.weights or [1.0 / len(a.models)] * len(a.models)
        d = {"merge_method": a.method, "base_model": a.base, "dtype": a.dtype,
             "models": [{"model": m, "parameters": {"weight": w, "density": a.density}} for m, w in zip(a.models, ws)]}
        if a.t is not None:
            d["parameters"] = {"t": a.t}
        cfg = MergeConfig.from_dict(d)
    if a.align_experts:
        cfg.align_moe_experts = True
    if a.sanity:
        cfg.sanity = a.sanity
    cfg.output_path = a.output
    print(json.dumps(run_merge(cfg, a.device)))
    return 0


def _quantize_args(sp):
    from ..gguf.types import QUANT_METHODS
    p = sp.add_parser("quantize", help="export a model as GGUF (K-quants, legacy quants, dynamic with imatrix)")
    p.add_argument("-m", "--model", required=True)
    p.add_argument("-o", "--output", required=True)
    p.add_argument("--method", default="q4_k_m", choices=sorted(QUANT_METHODS))
    p.add_argument("--imatrix")
    p.add_argument("--kl-calibrate", action="store_true")
    p.add_argument("--target-bpw", type=float)
    p.add_argument("--threads", type=int, default=0)
    p.add_argument("--format", default="gguf", choices=["gguf", "fp8", "mlx"],
                   help="mlx: affine group quantisation with quality-driven bit allocation (--target-bpw, default 4.5)")
    p.add_argument("--group-size", type=int, default=64)
    p.add_argument("--bits", type=int, choices=[3, 4, 5, 6, 8], help="--format mlx: default bit width (sets the "
                   "bits-per-weight target when --target-bpw is not given)")
    p.add_argument("--kl-threshold", type=float, default=0.01, help="dynamic: quality-loss budget of the calibration")
    p.add_argument("--lora", help="fuse this LoRA adapter into the model before quantising")
    return p


@_command(_quantize_args)
def cmd_quantize(a) -> int:
    from ..models.loader import resolve_model_path
    mdir = resolve_model_path(a.model)
    fused_tmp = None
    if a.lora:
        import tempfile

        from ..merge.merge import merge_lora_into_base
        fused_tmp = tempfile.TemporaryDirectory(prefix="pmetal-fused-")
        merge_lora_into_base(mdir, a.lora, fused_tmp.name, "bfloat16")
        mdir = fused_tmp.name
    try:
        return _quantize_dir(a, mdir)
    finally:
        if fused_tmp is not None:
            fused_tmp.cleanup()


def _quantize_dir(a, mdir: str) -> int:
    if a.format == "fp8":
        from ..models.fp8 import export_fp8_checkpoint
        print(json.dumps(export_fp8_checkpoint(mdir, a.output)))
        return 0
    if a.format == "mlx":
        from ..quant.mlx_affine import quantize_model as quantize_mlx
        # per-weight cost of b-bit groups: b bits + one fp16 scale and bias per group
        bpw = a.target_bpw or ((a.bits + 32.0 / a.group_size) if a.bits else 4.5)
        print(json.dumps(quantize_mlx(mdir, a.output, bpw, a.group_size)))
        return 0
    from ..gguf.convert import quantize_model
    from ..gguf.recipe import DynamicConfig
    dyn = DynamicConfig(kl_calibrate=a.kl_calibrate, target_bpw=a.target_bpw, error_budget=a.kl_threshold) \
        if a.method == "dynamic" else None
    print(json.dumps(quantize_model(mdir, a.output, a.method, a.imatrix, dyn, a.threads)))
    return 0


# ------------------------------------------------------------------------------------------- distill / grpo / rlkd
def _column_args(p, prompt_column: bool = True) -> None:
    """Dataset column options shared by ``train``, ``distill``, ``grpo`` and ``rlkd``."""
    p.add_argument("--text-column", help="dataset field that holds the text")
    p.add_argument("--text-columns", help="comma-separated fields joined into the text")
    p.add_argument("--column-separator", default="\n\n", help="what joins --text-columns (and prompt / response)")
    if prompt_column:
        p.add_argument("--prompt-column", help="dataset field that holds the prompt")
    p.add_argument("--response-column", help="dataset field that holds the response")


DEFAULT_TEXT_KEYS = ("prompt", "question", "text", "instruction")


def record_text(rec, columns=None, key_order=DEFAULT_TEXT_KEYS, with_response: bool = False):
    """The text of one dataset record under the column options. ``with_response`` appends the response column to the
    prompt (full sequences for distillation); without it only the prompt side is read (rollout prompts)."""
    if not isinstance(rec, dict):
        return str(rec)
    sep = getattr(columns, "column_separator", None) or "\n\n"
    names = getattr(columns, "text_columns", None)
    if names:
        parts = [str(rec[k]) for k in (n.strip() for n in names.split(",")) if isinstance(rec.get(k), (str, int, float))]
        if parts:
            return sep.join(parts)
    pc, rc = getattr(columns, "prompt_column", None), getattr(columns, "response_column", None)
    if pc and isinstance(rec.get(pc), str):
        if with_response and rc and isinstance(rec.get(rc), str):
            return rec[pc] + sep + rec[rc]
        return rec[pc]
    tc = getattr(columns, "text_column", None)
    if tc and isinstance(rec.get(tc), str):
        return rec[tc]
    text = next((rec[k] for k in key_order if isinstance(rec.get(k), str)), None)
    if text is not None and with_response:
        resp = next((rec[k] for k in ((rc,) if rc else ()) + ("response", "answer", "output", "completion")
                     if k and isinstance(rec.get(k), str)), None)
        if resp is not None and "text" not in rec:
            return text + sep + resp
    return text


def _read_prompts(path: str, tok, limit=None, key_order=DEFAULT_TEXT_KEYS, columns=None, with_response: bool = False):
    out = []
    with open(path, "r", encoding="utf-8") as fh:
        for line in fh:
            line = line.strip()
            if not line:
                continue
            try:
                text = record_text(json.loads(line), columns, key_order, with_response)
            except json.JSONDecodeError:
                text = line
            if text:
                out.append(tok.encode(text))
            if limit and len(out) >= limit:
                break
    return out


def _distill_args(sp):
    p = sp.add_parser("distill", help="knowledge distillation (online / offline / progressive, TAID)")
    p.add_argument("--teacher", required=True)
    p.add_argument("--student", required=True)
    p.add_argument("-d", "--dataset", required=True)
    p.add_argument("-o", "--output", default="./distill-output")
    p.add_argument("--method", default="online", choices=["online", "offline", "progressive"])
    p.add_argument("--loss-type", default="kl")
    p.add_argument("--alpha", type=float, default=0.5)
    p.add_argument("--temperature", type=float, default=2.0)
    p.add_argument("--learning-rate", type=float, default=2e-5)
    p.add_argument("--max-steps", type=int, default=100)
    p.add_argument("--max-seq-len", type=int, default=1024)
    p.add_argument("--cache-dir", "--offline-cache", dest="cache_dir")
    p.add_argument("--offline", action="store_true", help="same as --method offline: train against cached teacher logits")
    p.add_argument("--offline-generate", action="store_true", help="build the teacher logit cache and stop")
    p.add_argument("--offline-compression", default="topk", choices=["full", "topk", "int8", "int4", "int8_per_token"])
    p.add_argument("--offline-top-k", type=int, default=64)
    p.add_argument("--rationale", action="store_true", help="entropy-weighted KL that stresses reasoning tokens")
    p.add_argument("--rationale-weight", type=float, default=1.0)
    p.add_argument("--epochs", type=int, default=None, help="passes over the dataset (overrides --max-steps)")
    p.add_argument("--batch-size", type=int, default=1, help="sequences per optimiser step are packed one at a time")
    p.add_argument("--eval-dataset", help="report the distillation loss on this dataset at the end")
    p.add_argument("--checkpoint-every", type=int, default=0)
    p.add_argument("--resume", action="store_true", help="continue a LoRA run from the newest checkpoint in the output directory")
    p.add_argument("--log-metrics")
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--lora-r", type=int, default=0, help="train a LoRA adapter on the student instead of all weights")
    p.add_argument("--lora-alpha", type=float, default=None)
    _column_args(p)
    p.add_argument("--device")
    return p


@_command(_distill_args)
def cmd_distill(a) -> int:
    import torch

    from ..distill.trainer import DistillConfig, DistillTrainer
    from ..models.loader import load_pretrained, save_pretrained
    from ..trainer.orchestrator import _portable_model_dir
    a.model = a.student
    s_pdir, t_pdir = _portable_model_dir(a.student), _portable_model_dir(a.teacher)
    if s_pdir is not None:
        # student from the config-driven architectures: portable adapters (or all weights), its own tokenizer
        from ..data.tokenizer import Tokenizer
        from ..models.architectures import load_pretrained as load_portable
        dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
        student = load_portable(s_pdir, torch.bfloat16 if dev.startswith("cuda") else torch.float32, dev)
        tok, sdir = Tokenizer.from_model_dir(s_pdir), s_pdir
    else:
        student, tok, _, _, sdir = _load_for_inference(a)
        dev = str(student.embed_tokens.device)
    if t_pdir is not None:
        from ..models.architectures import load_pretrained as load_portable
        teacher = load_portable(t_pdir, next(student.parameters()).dtype, dev)
    else:
        teacher, _, _ = load_pretrained(a.teacher, dtype=next(student.parameters()).dtype, device=dev)
    teacher.eval()
    for p in teacher.parameters():
        p.requires_grad_(False)
    if a.lora_r > 0 and s_pdir is not None:
        from ..core.config import LoraConfig
        from ..lora.portable import apply_lora_portable
        apply_lora_portable(student, LoraConfig(r=a.lora_r, alpha=a.lora_alpha or 2.0 * a.lora_r))
    elif a.lora_r > 0:
        from ..core.config import LoraConfig
        from ..lora import apply_lora
        apply_lora(student, LoraConfig(r=a.lora_r, alpha=a.lora_alpha or 2.0 * a.lora_r))
        student.to(dev)
    else:
        for p in student.parameters():
            p.requires_grad_(True)
    student.train()
    seqs = [s[: a.max_seq_len] for s in _read_prompts(a.dataset, tok, columns=a, with_response=True) if len(s) > 1]
    if not seqs:
        print("error: no usable sequences in dataset", file=sys.stderr)
        return 2
    method = "offline" if (a.offline or a.offline_generate) else a.method
    steps = a.epochs * len(seqs) if a.epochs else a.max_steps
    markers = None
    if a.rationale:
        ids = [tok.token_to_id(t) for t in ("<think>", "</think>")]
        markers = tuple(ids) if all(i is not None for i in ids) else None
    cache_ready = bool(a.cache_dir) and os.path.exists(os.path.join(a.cache_dir, "metadata.json"))
    cfg = DistillConfig(method=method, loss_type=a.loss_type, alpha=a.alpha, temperature=a.temperature,
                        learning_rate=a.learning_rate, total_steps=steps, cache_dir=a.cache_dir if cache_ready else None,
                        rationale=a.rationale, rationale_weight=a.rationale_weight, reasoning_markers=markers)
    tr = DistillTrainer(student, teacher, cfg)
    if method == "offline":
        if not a.cache_dir:
            print("error: offline distillation needs --offline-cache", file=sys.stderr)
            return 2
        if not cache_ready:
            tr.cache = tr.build_cache(seqs, a.cache_dir, a.offline_compression, a.offline_top_k)
        if a.offline_generate:
            print(json.dumps({"cache": a.cache_dir, "sequences": len(seqs), "compression": a.offline_compression}))
            return 0
    lcfg = None
    if a.lora_r > 0:
        from ..core.config import LoraConfig
        lcfg = LoraConfig(r=a.lora_r, alpha=a.lora_alpha or 2.0 * a.lora_r)
    ckpt_dir = os.path.join(a.output, "checkpoints")
    first = 0
    if s_pdir is not None:
        from ..lora.portable import load_adapter_portable as load_adapter, save_adapter_portable as save_adapter
    else:
        from ..lora.adapter import load_adapter, save_adapter
    if a.resume and lcfg is not None and os.path.isdir(ckpt_dir):
        done = sorted(int(d.split("_")[1]) for d in os.listdir(ckpt_dir) if d.startswith("step_") and d.split("_")[1].isdigit())
        if done:
            load_adapter(student, os.path.join(ckpt_dir, f"step_{done[-1]}"))
            first = tr.step_count = done[-1]
    import random
    order = list(range(len(seqs)))
    random.Random(a.seed).shuffle(order)
    log = open(a.log_metrics, "a", encoding="utf-8") if a.log_metrics else None
    last = {}
    try:
        for step in range(first, steps):
            i = order[step % len(seqs)]
            ids = torch.tensor(seqs[i], dtype=torch.int64)
            last = tr.step(ids, ids.clone(), seq_id=i)
            line = json.dumps({"step": step + 1, **{k: round(v, 5) for k, v in last.items()}})
            if log:
                log.write(line + "\n")
                log.flush()
            if step % 10 == 0:
                print(line, file=sys.stderr)
            if a.checkpoint_every and lcfg is not None and (step + 1) % a.checkpoint_every == 0:
                save_adapter(student, os.path.join(ckpt_dir, f"step_{step + 1}"), lcfg, a.student)
    finally:
        if log:
            log.close()
    extra = {}
    if a.eval_dataset:
        ev = [s[: a.max_seq_len] for s in _read_prompts(a.eval_dataset, tok) if len(s) > 1]
        tr.cache = None
        tot = []
        with torch.no_grad():
            for s_ in ev:
                ids = torch.tensor(s_, dtype=torch.int64)
                with torch.enable_grad():
                    loss, _ = tr.loss(ids.to(tr.device), ids.clone().to(tr.device))
                tot.append(float(loss.detach()))
        extra["eval_loss"] = round(sum(tot) / max(len(tot), 1), 5)
        extra["eval_samples"] = len(ev)
    os.makedirs(a.output, exist_ok=True)
    if lcfg is not None:
        save_adapter(student, a.output, lcfg, a.student)
    elif s_pdir is not None:
        from ..models.architectures import save_pretrained as save_portable
        save_portable(student, a.output, copy_from=sdir)
    else:
        save_pretrained(student, a.output, copy_from=sdir)
    print(json.dumps({"output": a.output, "steps": steps, "resumed_from": first, **last, **extra}))
    return 0


def _grpo_args(sp):
    p = sp.add_parser("grpo", help="GRPO / DAPO reinforcement learning with batched paged rollouts")
    p.add_argument("-m", "--model", required=True)
    p.add_argument("-d", "--dataset", required=True)
    p.add_argument("-o", "--output", default="./grpo-output")
    p.add_argument("--dapo", action="store_true")
    p.add_argument("--num-generations", type=int, default=8)
    p.add_argument("--beta", type=float, default=0.001)
    p.add_argument("--max-completion-length", type=int, default=512)
    p.add_argument("--max-prompt-length", type=int, default=512)
    p.add_argument("--learning-rate", type=float, default=1e-6)
    p.add_argument("--max-steps", type=int, default=None, help="default: --epochs passes over the prompts")
    p.add_argument("--epochs", type=int, default=1)
    p.add_argument("--prompts-per-step", type=int, default=1)
    p.add_argument("--lora-r", type=int, default=16)
    p.add_argument("--lora-alpha", type=float, default=None)
    p.add_argument("--seed", type=int, default=42)
    _column_args(p)
    p.add_argument("--max-seq-len", type=int, default=None,
                   help="cap on prompt + completion tokens: prompts are cut from the left to leave room for the completion")
    p.add_argument("--no-flash-attention", action="store_true", help="PyTorch reference attention instead of the kernels")
    p.add_argument("--reward-model-max-length", type=int, default=2048, help="tokens the reward model reads (cut from the right)")
    p.add_argument("--reward-model-template", help="text template with {prompt} and {completion} for the reward model")
    p.add_argument("--grpo-kv-bits", type=int, choices=[4, 8], default=None,
                   help="rollout key/value cache precision: 8 = int8 blocks, 4 = rotated 4-bit codes (default bf16)")
    p.add_argument("--vlm", action="store_true", help="image-conditioned rollouts (not available: the command stops with a message)")
    p.add_argument("--max-image-size", type=int, default=336, help="with --vlm")
    p.add_argument("--reward", default="format", choices=["format", "length", "accuracy"])
    p.add_argument("--reasoning-rewards", action="store_true", help="XML format reward + answer accuracy reward")
    p.add_argument("--reward-model", help="add the score of this reward model (decoder + scalar head)")
    p.add_argument("--reward-model-weight", type=float, default=1.0)
    p.add_argument("--async-rewards", action="store_true", help="score completions on worker threads")
    p.add_argument("--checkpoint-every", type=int, default=0, help="save the adapter every N steps under checkpoints/")
    p.add_argument("--resume", action="store_true", help="continue from the newest checkpoint in the output directory")
    p.add_argument("--log-metrics", help="append one JSON line per step to this file")
    p.add_argument("--speculative", action="store_true",
                   help="accepted for compatibility: rollouts are generated as one paged batch, which replaces per-stream drafting")
    p.add_argument("--speculative-draft-tokens", type=int, default=4)
    p.add_argument("--teacher", help="with --rlkd-alpha: add a KD term against this teacher (RLKD)")
    p.add_argument("--rlkd-alpha", type=float, default=0.0)
    p.add_argument("--device")
    return p


def _load_reward_model(path: str, dtype, dev, max_length: int = 2048, template=None, tokenizer=None):
    """A frozen scorer for ``--reward-model``: any supported architecture; the scalar head is read from the checkpoint
    (``score.weight`` / ``v_head.weight`` / ``reward_head.weight``), without one the mean read-out logit is the score."""
    from ..models.loader import load_pretrained, read_state_dict
    from ..trainer.orchestrator import _portable_model_dir
    from ..trainer.rewards import ModelReward, RewardModelConfig
    pdir = _portable_model_dir(path)
    if pdir is not None:
        from ..models.architectures import load_pretrained as load_portable
        rm, rdir = load_portable(pdir, dtype, dev), pdir
    else:
        rm, _, rdir = load_pretrained(path, dtype=dtype, device=dev)
    head = None
    if rdir:
        sd = read_state_dict(rdir)
        head = next((sd[k].reshape(-1).to(dev) for k in ("score.weight", "v_head.weight", "reward_head.weight") if k in sd), None)
    rm.eval()
    for p in rm.parameters():
        p.requires_grad_(False)
    if template and tokenizer is None:
        from ..data.tokenizer import Tokenizer
        tokenizer = Tokenizer.from_model_dir(rdir)
    return ModelReward(rm, head, RewardModelConfig(max_length=max_length, template=template), tokenizer)


def _grpo_prompt_cap(a) -> int:
    """Prompt length limit: --max-prompt-length, tightened so that prompt + completion fits --max-seq-len."""
    cap = a.max_prompt_length
    if getattr(a, "max_seq_len", None):
        if a.max_seq_len <= a.max_completion_length:
            raise SystemExit("error: --max-seq-len must exceed --max-completion-length")
        cap = min(cap, a.max_seq_len - a.max_completion_length)
    return cap


def _grpo_portable(a, model_dir: str, lcfg) -> int:
    """``grpo`` on a config-driven architecture: portable LoRA adapters, rollouts on the model's own cache
    (trainer/grpo_portable.py). Reward models, teachers and --resume belong to the llama / qwen path."""
    import random

    import torch

    from ..data.chat_templates import ChatTemplate
    from ..data.inference_config import collect_all_stop_tokens
    from ..data.tokenizer import Tokenizer
    from ..lora.portable import apply_lora_portable, save_adapter_portable
    from ..models.architectures import load_pretrained as load_portable
    from ..trainer.grpo import GrpoConfig
    from ..trainer.grpo_portable import PortableGrpoTrainer
    from ..trainer.rewards import make_reward
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    if getattr(a, "no_flash_attention", False):
        from ..models.architectures import fast
        fast.ROUTES.discard("attention")
    if getattr(a, "grpo_kv_bits", None):
        print("note: --grpo-kv-bits applies to the paged cache of the llama / qwen path; this architecture keeps bf16 "
              "rollout caches", file=sys.stderr)
    model = load_portable(model_dir, torch.bfloat16 if dev.startswith("cuda") else torch.float32, dev)
    apply_lora_portable(model, lcfg)
    model.train()
    tok = Tokenizer.from_model_dir(model_dir)
    eos = collect_all_stop_tokens(model_dir, tok, ChatTemplate.from_model_dir(model_dir).eos())
    kw = dict(num_generations=a.num_generations, beta=a.beta, max_completion_length=a.max_completion_length,
              max_prompt_length=_grpo_prompt_cap(a), learning_rate=a.learning_rate)
    cfg = GrpoConfig.dapo(**kw) if a.dapo else GrpoConfig(**kw)
    reward = make_reward(a.reward, tok)
    if a.reasoning_rewards:
        from ..trainer.rewards import combined_reward
        reward = combined_reward([make_reward("format", tok), make_reward("accuracy", tok, _read_targets(a.dataset))], [1.0, 1.0])
    if a.reward_model:
        from ..trainer.rewards import combined_reward
        reward = combined_reward([reward, _load_reward_model(a.reward_model, next(model.parameters()).dtype, dev,
                                                                 a.reward_model_max_length, a.reward_model_template)],
                                 [1.0, a.reward_model_weight])
    if a.teacher and a.rlkd_alpha > 0:
        from ..trainer.gspo import portable_rlkd_trainer
        from ..trainer.orchestrator import _portable_model_dir
        tdir = _portable_model_dir(a.teacher)
        if tdir is not None:
            teacher = load_portable(tdir, next(model.parameters()).dtype, dev).eval()
        else:
            from ..models.loader import load_pretrained
            teacher = load_pretrained(a.teacher, dtype=next(model.parameters()).dtype, device=dev)[0].eval()
        for p in teacher.parameters():
            p.requires_grad_(False)
        tr = portable_rlkd_trainer(model, cfg, reward, teacher, a.rlkd_alpha, eos_ids=eos, pad_id=tok.pad_token_id or 0)
    else:
        tr = PortableGrpoTrainer(model, cfg, reward, eos_ids=eos, pad_id=tok.pad_token_id or 0)
    keys = ((a.prompt_column,) if a.prompt_column else ()) + ("prompt", "question", "text", "instruction")
    prompts = _read_prompts(a.dataset, tok, key_order=keys, columns=a)
    if not prompts:
        print("error: no prompts in dataset", file=sys.stderr)
        return 2
    random.Random(a.seed).shuffle(prompts)
    steps = a.max_steps if a.max_steps is not None else a.epochs * (-(-len(prompts) // a.prompts_per_step))
    log = open(a.log_metrics, "a", encoding="utf-8") if a.log_metrics else None
    try:
        for step in range(steps):
            batch = [prompts[(step * a.prompts_per_step + j) % len(prompts)] for j in range(a.prompts_per_step)]
            st = tr.step(batch)
            d = st if isinstance(st, dict) else st.__dict__
            line = json.dumps({"step": step + 1, **{k: (round(v, 5) if isinstance(v, float) else v) for k, v in d.items()
                                                    if isinstance(v, (int, float, str, bool))}})
            print(line, file=sys.stderr)
            if log:
                log.write(line + "\n")
                log.flush()
            if a.checkpoint_every and (step + 1) % a.checkpoint_every == 0:
                save_adapter_portable(model, os.path.join(a.output, "checkpoints", f"step_{step + 1}"), lcfg, a.model)
    finally:
        if log:
            log.close()
    save_adapter_portable(model, a.output, lcfg, a.model)
    print(json.dumps({"output": a.output, "steps": steps, "path": "portable"}))
    return 0


@_command(_grpo_args)
def cmd_grpo(a) -> int:
    from ..core.config import LoraConfig
    from ..lora import apply_lora
    from ..lora.adapter import save_adapter
    from ..trainer.grpo import GrpoConfig, GrpoTrainer
    from ..trainer.orchestrator import _portable_model_dir
    from ..trainer.rewards import make_reward
    lcfg = LoraConfig(r=a.lora_r, alpha=a.lora_alpha if getattr(a, 'lora_alpha', None) else 2.0 * a.lora_r)
    if getattr(a, "vlm", False):
        print("error: --vlm (rollouts conditioned on images) is not available; the vision towers load and run "
              "(models/architectures/vision.py, mllama.py) but the GRPO trainers take text prompts only", file=sys.stderr)
        return 2
    pdir = _portable_model_dir(a.model)
    if pdir is not None:
        return _grpo_portable(a, pdir, lcfg)
    if getattr(a, "no_flash_attention", False):
        from ..ops.functional import set_force_reference
        set_force_reference(True)
    model, tok, _, eos, _ = _load_for_inference(a)
    dev = str(model.embed_tokens.device)
    apply_lora(model, lcfg)
    model.to(dev).train()
    kw = dict(num_generations=a.num_generations, beta=a.beta, max_completion_length=a.max_completion_length,
              max_prompt_length=_grpo_prompt_cap(a), learning_rate=a.learning_rate)
    cfg = GrpoConfig.dapo(**kw) if a.dapo else GrpoConfig(**kw)
    reward = make_reward(a.reward, tok)
    if a.reasoning_rewards:
        from ..trainer.rewards import combined_reward
        reward = combined_reward([make_reward("format", tok), make_reward("accuracy", tok, _read_targets(a.dataset))], [1.0, 1.0])
    if a.reward_model:
        from ..trainer.rewards import combined_reward
        reward = combined_reward([reward, _load_reward_model(a.reward_model, next(model.parameters()).dtype, dev,
                                                                 a.reward_model_max_length, a.reward_model_template)],
                                 [1.0, a.reward_model_weight])
    if a.async_rewards:
        reward = _threaded_reward(reward)
    if a.teacher and a.rlkd_alpha > 0:
        from ..models.loader import load_pretrained
        from ..trainer.gspo import RlkdTrainer
        teacher, _, _ = load_pretrained(a.teacher, dtype=next(model.parameters()).dtype, device=dev)
        tr = RlkdTrainer(model, cfg, reward, teacher.eval(), a.rlkd_alpha, eos_ids=eos)
    else:
        tr = GrpoTrainer(model, cfg, reward, eos_ids=eos)
    if getattr(a, "grpo_kv_bits", None):
        # rollouts on a quantised paged cache; log-probabilities are recomputed in bf16, so only sampling sees the codes
        from ..models.generation import Generator
        tr.gen = Generator(model, cache=model.new_cache(8192, quant={8: "int8", 4: "tq4"}[a.grpo_kv_bits]))
    keys = ((a.prompt_column,) if a.prompt_column else ()) + ("prompt", "question", "text", "instruction")
    prompts = _read_prompts(a.dataset, tok, key_order=keys, columns=a)
    if not prompts:
        print("error: no prompts in dataset", file=sys.stderr)
        return 2
    import random
    random.Random(a.seed).shuffle(prompts)
    steps = a.max_steps if a.max_steps is not None else a.epochs * (-(-len(prompts) // a.prompts_per_step))
    ckpt_dir = os.path.join(a.output, "checkpoints")
    first = 0
    if a.resume and os.path.isdir(ckpt_dir):
        from ..lora.adapter import load_adapter
        done = sorted(int(d.split("_")[1]) for d in os.listdir(ckpt_dir) if d.startswith("step_") and d.split("_")[1].isdigit())
        if done:
            load_adapter(model, os.path.join(ckpt_dir, f"step_{done[-1]}"))
            first = done[-1]
    log = open(a.log_metrics, "a", encoding="utf-8") if a.log_metrics else None
    try:
        for step in range(first, steps):
            batch = [prompts[(step * a.prompts_per_step + j) % len(prompts)] for j in range(a.prompts_per_step)]
            if getattr(a, "anneal_alpha", False) and hasattr(tr, "alpha"):
                tr.alpha = a.rlkd_alpha + (a.final_alpha - a.rlkd_alpha) * step / max(steps - 1, 1)
            st = tr.step(batch)
            d = st if isinstance(st, dict) else st.__dict__
            line = json.dumps({"step": step + 1, **{k: (round(v, 5) if isinstance(v, float) else v) for k, v in d.items()
                                                    if isinstance(v, (int, float, str, bool))}})
            print(line, file=sys.stderr)
            if log:
                log.write(line + "\n")
                log.flush()
            if a.checkpoint_every and (step + 1) % a.checkpoint_every == 0:
                save_adapter(model, os.path.join(ckpt_dir, f"step_{step + 1}"), lcfg, a.model)
    finally:
        if log:
            log.close()
    save_adapter(model, a.output, lcfg, a.model)
    print(json.dumps({"output": a.output, "steps": steps, "resumed_from": first}))
    return 0


def _read_targets(path: str):
    """prompt text -> reference answer, from records that carry ``answer`` / ``target`` / ``solution``."""
    out = {}
    with open(path, "r", encoding="utf-8") as fh:
        for line in fh:
            try:
                d = json.loads(line)
            except ValueError:
                continue
            if not isinstance(d, dict):
                continue
            p = next((d[k] for k in ("prompt", "question", "text", "instruction") if isinstance(d.get(k), str)), None)
            t = next((d[k] for k in ("answer", "target", "solution") if d.get(k) is not None), None)
            if p is not None and t is not None:
                out[p] = str(t)
    return out


def _threaded_reward(fn, workers: int = 4):
    """Score slices of the completions on worker threads (reward functions that call tools or models spend their time
    outside the interpreter lock)."""
    from concurrent.futures import ThreadPoolExecutor
    pool = ThreadPoolExecutor(max_workers=workers)

    def wrapped(prompts, completions):
        n = len(completions)
        if n < 2 * workers:
            return fn(prompts, completions)
        cuts = [n * i // workers for i in range(workers + 1)]
        parts = pool.map(lambda i: fn(prompts[cuts[i]:cuts[i + 1]], completions[cuts[i]:cuts[i + 1]]), range(workers))
        return [x for part in parts for x in part]
    return wrapped


# ------------------------------------------------------------------------------------------- eval / bench / cluster
def _eval_args(sp):
    p = sp.add_parser("eval", help="loss / perplexity / token accuracy on a dataset")
    p.add_argument("-m", "--model", required=True)
    p.add_argument("-l", "--lora")
    p.add_argument("-d", "--dataset", required=True)
    p.add_argument("--max-samples", "--num-samples", dest="max_samples", type=int, default=200)
    p.add_argument("--max-seq-len", type=int, default=2048)
    p.add_argument("--json", action="store_true", help="the result is always one JSON line (accepted for compatibility)")
    p.add_argument("--device")
    return p


@_command(_eval_args)
def cmd_eval(a) -> int:
    import math

    import torch

    from ..trainer.orchestrator import _portable_model_dir
    pdir = _portable_model_dir(a.model)
    if pdir is not None:                      # portable architecture: logits straight from the module
        from ..data.tokenizer import Tokenizer
        from ..models.architectures import load_pretrained as load_portable
        dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
        model = load_portable(pdir, torch.bfloat16 if dev.startswith("cuda") else torch.float32, dev).eval()
        if a.lora:
            from ..lora.adapter import load_adapter_config
            from ..lora.portable import apply_lora_portable, load_adapter_portable
            apply_lora_portable(model, load_adapter_config(a.lora))
            load_adapter_portable(model, a.lora)
        tok = Tokenizer.from_model_dir(pdir)
        seqs = [s[: a.max_seq_len] for s in _read_prompts(a.dataset, tok, a.max_samples) if len(s) > 1]
        tot, n, correct = 0.0, 0, 0
        with torch.no_grad():
            for s in seqs:
                ids = torch.tensor([s], dtype=torch.int64, device=dev)
                logits = model(ids)[0, :-1].float()
                tot += float(torch.nn.functional.cross_entropy(logits, ids[0, 1:], reduction="sum"))
                correct += int((logits.argmax(-1) == ids[0, 1:]).sum())
                n += ids.shape[1] - 1
        loss = tot / max(n, 1)
        print(json.dumps({"samples": len(seqs), "tokens": n, "loss": round(loss, 5),
                          "perplexity": round(math.exp(min(loss, 50)), 4), "token_accuracy": round(correct / max(n, 1), 5),
                          "path": "portable"}))
        return 0
    model, tok, _, _, _ = _load_for_inference(a)
    seqs = [s[: a.max_seq_len] for s in _read_prompts(a.dataset, tok, a.max_samples) if len(s) > 1]
    tot, n, correct = 0.0, 0, 0
    dev = model.embed_tokens.device
    with torch.no_grad():
        for s in seqs:
            ids = torch.tensor(s, dtype=torch.int64, device=dev)
            T = ids.numel()
            h = model.forward_hidden(ids, torch.arange(T, dtype=torch.int32, device=dev),
                                     torch.tensor([0, T], dtype=torch.int32, device=dev),
                                     torch.zeros(T, dtype=torch.int32, device=dev))
            logits = h[:-1].float() @ model.head_weight().float().t()
            tot += float(torch.nn.functional.cross_entropy(logits, ids[1:], reduction="sum"))
            correct += int((logits.argmax(-1) == ids[1:]).sum())
            n += T - 1
    loss = tot / max(n, 1)
    print(json.dumps({"samples": len(seqs), "tokens": n, "loss": round(loss, 5), "perplexity": round(math.exp(min(loss, 50)), 4),
                      "token_accuracy": round(correct / max(n, 1), 5)}))
    return 0


def _bench_args(sp):
    p = sp.add_parser("bench", help="kernel corpus / training workload / generation benchmarks")
    p.add_argument("what", nargs="?", default="corpus", choices=["corpus", "workload", "gen"])
    p.add_argument("--case", nargs="*")
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("-m", "--model", default="random:qwen3-0.6b")
    p.add_argument("--batch-size", type=int, default=None, help="workload: packs per step; gen: concurrent sequences")
    p.add_argument("--seq-len", type=int, default=None, help="workload: tokens per pack; gen: prompt length")
    p.add_argument("--json")
    p.add_argument("--device")
    return p


@_command(_bench_args)
def cmd_bench(a) -> int:
    if a.what == "corpus":
        from ..bench import kernels
        iters = a.iters if a.iters is not None else (3 if getattr(a, "quick", False) else 10)
        path = getattr(a, "output", None) or (a.json if isinstance(a.json, str) else None)
        argv = ["--iters", str(iters)] + (["--case"] + a.case if a.case else []) + (["--json", path] if path else [])
        return kernels.main(argv) or 0
    from ..bench import workload
    return workload.main(a) or 0


def _cluster_args(sp):
    p = sp.add_parser("cluster", help="multi-GPU node: status, collective bench, pipeline bench, train, serve")
    p.add_argument("action", choices=["status", "up", "bench", "pipeline-bench", "train", "serve"])
    p.add_argument("--gpus", type=int, default=0)
    p.add_argument("--mb", type=int, default=64)
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--hidden-dim", type=int, default=0, help="pipeline-bench: width of the activation message")
    p.add_argument("--tokens", type=int, default=0, help="pipeline-bench: tokens per activation message")
    p.add_argument("--layers", type=int, default=0, help="accepted for compatibility (the stages exchange activations only)")
    p.add_argument("--vocab", type=int, default=0, help="accepted for compatibility")
    p.add_argument("--timeout", type=float, default=0, help="process-group timeout in seconds")
    p.add_argument("--min-peers", type=int, default=0, help="fail unless this many GPUs besides the first are present")
    p.add_argument("--wait", type=float, default=0, help="up: keep printing snapshots for this many seconds")
    p.add_argument("--status-interval", type=float, default=10, help="up: seconds between snapshots")
    p.add_argument("--json", action="store_true", help="status: one compact JSON line instead of the indented document")
    p.add_argument("--no-discovery", action="store_true", help="status: skip the peer-access / NVLink probe")
    p.add_argument("--gradient-port", type=int, default=0, help="bench: rendezvous port of the worker processes")
    p.add_argument("--activation-port", type=int, default=0, help="pipeline-bench: rendezvous port of the worker processes")
    p.add_argument("--discovery-port", type=int, default=0, help="reported in the status document")
    p.add_argument("--result-port", type=int, default=0, help="reported in the status document")
    p.add_argument("rest", nargs=argparse_remainder())
    return p


def argparse_remainder():
    import argparse
    return argparse.REMAINDER


@_command(_cluster_args)
def cmd_cluster(a) -> int:
    from ..parallel import cluster_cli
    if a.rest:
        # the trailing remainder also swallows this command's own flags when they follow the action
        # (``cluster bench --gpus 2``): pick them out, leave the rest for the launched sub-command
        import argparse
        own = argparse.ArgumentParser(add_help=False)
        for flag, typ in (("--gpus", int), ("--mb", int), ("--iters", int), ("--hidden-dim", int), ("--tokens", int),
                          ("--layers", int), ("--vocab", int), ("--timeout", float), ("--min-peers", int),
                          ("--wait", float), ("--status-interval", float), ("--gradient-port", int),
                          ("--activation-port", int), ("--discovery-port", int), ("--result-port", int)):
            own.add_argument(flag, type=typ, default=None)
        for flag in ("--json", "--no-discovery"):
            own.add_argument(flag, action="store_true", default=None)
        known, rest = own.parse_known_args([x for x in a.rest if x != "--"] if a.action not in ("train", "serve") else [])
        for k, v in vars(known).items():
            if v is not None:
                setattr(a, k, v)
        if a.action not in ("train", "serve"):
            a.rest = rest
    return cluster_cli.run(a) or 0


def _dl_args(sp):
    p = sp.add_parser("download", help="resolve a model from the local Hugging Face cache, or fetch it from the hub")
    p.add_argument("model")
    p.add_argument("--revision", default="main")
    p.add_argument("--token", default=os.environ.get("HF_TOKEN"))
    p.add_argument("--offline", action="store_true", help="never contact the hub")
    return p


@_command(_dl_args)
def cmd_download(a) -> int:
    from ..models.loader import is_hf_id, resolve_model_path
    try:
        print(resolve_model_path(a.model))
        return 0
    except FileNotFoundError as e:
        if a.offline or not is_hf_id(a.model):
            print(f"error: {e}", file=sys.stderr)
            return 1
    from .. import hub
    try:
        print(hub.download_model(a.model, a.revision, a.token))
        return 0
    except hub.HubError as e:
        print(f"error: {e}", file=sys.stderr)
        return 1


def _upload_args(sp):
    p = sp.add_parser("upload", help="upload a model directory to the Hugging Face Hub")
    p.add_argument("path")
    p.add_argument("repo", help="owner/name")
    p.add_argument("--token", default=os.environ.get("HF_TOKEN"))
    p.add_argument("--private", action="store_true")
    return p


@_command(_upload_args)
def cmd_upload(a) -> int:
    from .. import hub
    if not a.token:
        print("error: a token is required (--token or HF_TOKEN)", file=sys.stderr)
        return 2
    try:
        print(json.dumps(hub.upload_model(a.path, a.repo, a.token, a.private)))
        return 0
    except (hub.HubError, ValueError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1


def _ollama_args(sp):
    p = sp.add_parser("ollama", help="write an Ollama Modelfile for a GGUF export")
    p.add_argument("action", choices=["modelfile", "create", "templates"])
    p.add_argument("--gguf", "--base", dest="gguf", help="GGUF file (or model directory) the Modelfile starts FROM")
    p.add_argument("--name", help="create: the Ollama model name to register")
    p.add_argument("--lora", help="adapter directory or file added as ADAPTER")
    p.add_argument("--num-ctx", type=int)
    p.add_argument("--template", default=None, help="default: detected from the model name")
    p.add_argument("--system")
    p.add_argument("--license", help="license text written as the LICENSE block")
    p.add_argument("-o", "--output", default="Modelfile")
    _add_sampling_flags(p, {"temperature": 0.7, "top_k": 40, "top_p": 0.95, "repetition_penalty": 1.1})
    return p


@_command(_ollama_args)
def cmd_ollama(a) -> int:
    from ..utils.ollama import TEMPLATES, write_modelfile
    if a.action == "templates":
        print("\n".join(sorted(TEMPLATES)))
        return 0
    if not a.gguf:
        print("error: --gguf is required", file=sys.stderr)
        return 2
    from ..utils.ollama import detect_template, validate_model_name
    if a.action == "create":
        if not a.name:
            print("error: --name is required", file=sys.stderr)
            return 2
        try:
            validate_model_name(a.name)
        except ValueError as e:
            print(f"error: {e}", file=sys.stderr)
            return 2
    print(write_modelfile(a.gguf, a.output, a.template or detect_template(a.gguf), a.system, a.lora, a.license,
                          temperature=a.temperature, top_k=a.top_k, top_p=a.top_p, repeat_penalty=a.repetition_penalty,
                          num_ctx=a.num_ctx))
    if a.action == "create":
        print(f"To register the model, run:\n  ollama create {a.name} -f {a.output}")
    return 0


def _mcp_args(sp):
    return sp.add_parser("mcp", help="Model Context Protocol server on stdio (tools for training, inference, jobs)")


@_command(_mcp_args)
def cmd_mcp(a) -> int:
    from ..mcp import McpServer
    McpServer().serve_stdio()
    return 0


def _pretrain_args(sp):
    p = sp.add_parser("pretrain", help="full-parameter pre-training on token shards")
    p.add_argument("-m", "--model", help="model directory or random:<preset> for a fresh model")
    p.add_argument("--arch", help="preset name of a fresh model (same as --model random:<name>)")
    p.add_argument("--model-config", help="config.json of a fresh model with random weights")
    p.add_argument("--shards", required=True, help="glob of *.bin token shards")
    p.add_argument("--eval-shards", help="glob of held-out shards")
    p.add_argument("--eval-every", type=int, default=0)
    p.add_argument("--eval-batches", type=int, default=20)
    p.add_argument("-o", "--output", default="./pretrain-output")
    p.add_argument("--seq-len", type=int, default=2048)
    p.add_argument("--micro-batch", "--batch-size", dest="micro_batch", type=int, default=4)
    p.add_argument("--gradient-accumulation-steps", type=int, default=1)
    p.add_argument("--max-steps", "--steps", dest="max_steps", type=int, default=100)
    p.add_argument("--learning-rate", type=float, default=3e-4)
    p.add_argument("--min-lr", type=float, default=3e-5)
    p.add_argument("--lr-schedule", default="cosine")
    p.add_argument("--warmup-steps", type=int, default=10)
    p.add_argument("--weight-decay", type=float, default=0.1)
    p.add_argument("--max-grad-norm", type=float, default=1.0)
    p.add_argument("--z-loss", type=float, default=1e-4)
    p.add_argument("--checkpoint-every", type=int, default=0)
    p.add_argument("--log-every", type=int, default=1)
    p.add_argument("--eos-token-id", type=int, default=None, help="recorded in the saved config of a fresh model")
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--resume", nargs="?", const="auto", help="checkpoint directory, or no value for the newest one under --output")
    p.add_argument("--device")
    p.add_argument("--dp-impl", choices=["fused", "nccl", "overlap"], default="fused",
                   help="gradient exchange on several GPUs: the fused reduce + AdamW kernel over peer memory, one all-reduce "
                        "after backward, or bucketed all-reduces that run while backward continues")
    p.add_argument("--reduce-dtype", choices=["float32", "bfloat16"], default="float32",
                   help="--dp-impl overlap: number format of the gradients on the wire")
    p.add_argument("--bucket-mb", type=float, default=32.0, help="--dp-impl overlap: smallest bucket")
    return p


@_command(_pretrain_args)
def cmd_pretrain(a) -> int:
    import torch

    from ..data.streaming import TokenShardDataset
    from ..models.loader import load_pretrained
    from ..trainer.pretrain import PretrainConfig, PretrainTrainer
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    dctx = None
    if world > 1:
        # every rank reads its own shard of the data: the gradients have to meet before the update, or the replicas
        # drift apart. The process group comes first so that each rank builds its model on its own GPU
        from ..parallel.dp import DistContext
        dctx = DistContext.from_env()
        if torch.cuda.is_available() and not a.device:
            a.device = f"cuda:{int(os.environ.get('LOCAL_RANK', '0'))}"
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    if dctx is not None and dev.startswith("cuda") and a.dp_impl == "fused":
        from ..parallel.fused_dp import FusedDataParallel
        dctx = FusedDataParallel()
    torch.manual_seed(a.seed)
    if a.model_config:
        from ..models.config import ModelArgs
        from ..models.decoder import DecoderLM
        with open(a.model_config, "r", encoding="utf-8") as fh:
            margs = ModelArgs.from_dict(json.load(fh))
        model = DecoderLM(margs, dtype=torch.float32, device=dev).init_weights(0.02, a.seed)
    else:
        name = a.model or (f"random:{a.arch}" if a.arch else None)
        if not name:
            print("error: one of --model, --arch or --model-config is required", file=sys.stderr)
            return 2
        model, _, _ = load_pretrained(name, dtype=torch.float32, device=dev, seed=a.seed)
    if a.eos_token_id is not None and hasattr(model.cfg, "eos_token_id"):
        model.cfg.eos_token_id = a.eos_token_id
    cfg = PretrainConfig(learning_rate=a.learning_rate, min_lr=a.min_lr, warmup_steps=a.warmup_steps, max_steps=a.max_steps,
                         weight_decay=a.weight_decay, max_grad_norm=a.max_grad_norm, z_loss_coef=a.z_loss, seq_len=a.seq_len,
                         micro_batch=a.micro_batch, gradient_accumulation_steps=a.gradient_accumulation_steps,
                         lr_scheduler=a.lr_schedule, checkpoint_every=a.checkpoint_every, output=a.output)
    tr = PretrainTrainer(model.train(), cfg, dist=dctx, overlap_reduce=a.dp_impl == "overlap",
                         reduce_dtype=torch.bfloat16 if a.reduce_dtype == "bfloat16" else None, bucket_mb=a.bucket_mb)
    resume = a.resume
    if resume == "auto":
        done = sorted((int(d.split("_")[1]), d) for d in (os.listdir(a.output) if os.path.isdir(a.output) else [])
                      if d.startswith("step_") and d.split("_")[1].isdigit())
        resume = os.path.join(a.output, done[-1][1]) if done else None
    if resume:
        tr.load_checkpoint(resume)
    ds = TokenShardDataset(a.shards, a.seq_len, rank, world, seed=a.seed, loop=True)      # epochs roll over until --steps
    ev = TokenShardDataset(a.eval_shards, a.seq_len, rank, world) if a.eval_shards else None

    def on_step(st):
        if st.get("step", 0) % max(a.log_every, 1) == 0 or "eval_loss" in st:
            print(json.dumps(st), file=sys.stderr)
    last = tr.run(ds, on_step=on_step, eval_dataset=ev, eval_every=a.eval_every, eval_batches=a.eval_batches)
    if ev is not None and "eval_loss" not in last:
        last = {**last, **tr.evaluate(ev, a.eval_batches)}
    if dctx is not None:
        dctx.gather_optimizer_state(tr.opt)          # sharded moments (fused path) back to full size before writing
    if rank == 0:
        tr.save_checkpoint(os.path.join(a.output, "final"))
        print(json.dumps({"output": a.output, "resumed_from": resume, **last}))
    if dctx is not None:
        from ..parallel.dp import shutdown_process_group
        dctx.barrier()
        shutdown_process_group()
    return 0


def _embed_args(sp):
    p = sp.add_parser("embed-train", help="contrastive fine-tuning of an embedding model (InfoNCE / triplet / CoSENT)")
    p.add_argument("-m", "--model", required=True)
    p.add_argument("-d", "--dataset", required=True, help="JSONL with anchor/positive[/negative][/label]")
    p.add_argument("-o", "--output", default="./embed-output")
    p.add_argument("--loss", default="infonce", choices=["infonce", "triplet", "cosent"])
    p.add_argument("--batch-size", type=int, default=8)
    p.add_argument("--max-steps", type=int, default=None, help="default: --epochs passes over the dataset")
    p.add_argument("--epochs", type=int, default=1)
    p.add_argument("--learning-rate", type=float, default=2e-5)
    p.add_argument("--weight-decay", type=float, default=0.0)
    p.add_argument("--temperature", type=float, default=0.05, help="InfoNCE temperature")
    p.add_argument("--margin", type=float, default=0.5, help="triplet margin")
    p.add_argument("--pooling", default="mean", choices=["mean", "last", "cls", "first"])
    p.add_argument("--no-normalize", action="store_true", help="do not scale embeddings to unit length")
    p.add_argument("--max-seq-len", type=int, default=512)
    p.add_argument("--log-every", type=int, default=10)
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--lora-r", type=int, default=16)
    p.add_argument("--device")
    return p


@_command(_embed_args)
def cmd_embed_train(a) -> int:
    from ..core.config import LoraConfig
    from ..lora import apply_lora
    from ..lora.adapter import save_adapter
    from ..trainer.embedding import EmbeddingConfig, EmbeddingTrainer
    from ..trainer.orchestrator import _portable_model_dir
    lcfg = LoraConfig(r=a.lora_r, alpha=2.0 * a.lora_r)
    pdir = _portable_model_dir(a.model)
    if pdir is not None:
        # encoders (BERT / RoBERTa) and config-driven decoders: adapters on their projections, or every weight with --lora-r 0
        import torch

        from ..data.tokenizer import Tokenizer
        from ..lora.portable import apply_lora_portable, save_adapter_portable
        from ..models.architectures import load_pretrained as load_portable, save_pretrained as save_portable
        dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
        model = load_portable(pdir, torch.float32 if a.lora_r == 0 or not dev.startswith("cuda") else torch.bfloat16, dev)
        tok = Tokenizer.from_model_dir(pdir)
        if a.lora_r > 0:
            lcfg.target_modules = ["q_proj", "k_proj", "v_proj", "o_proj", "query", "key", "value", "dense"]
            apply_lora_portable(model, lcfg)
        else:
            for p_ in model.parameters():
                p_.requires_grad_(True)
        model.train()

        def save():
            if a.lora_r > 0:
                save_adapter_portable(model, a.output, lcfg, a.model)
            else:
                save_portable(model, a.output, copy_from=pdir)
    else:
        model, tok, _, _, _ = _load_for_inference(a)
        dev = str(model.embed_tokens.device)
        apply_lora(model, lcfg)
        model.to(dev).train()

        def save():
            save_adapter(model, a.output, lcfg, a.model)
    rows = []
    with open(a.dataset, "r", encoding="utf-8") as fh:
        for line in fh:
            if line.strip():
                rows.append(json.loads(line))
    import random
    random.Random(a.seed).shuffle(rows)
    pooling = {"cls": "first"}.get(a.pooling, a.pooling)
    tr = EmbeddingTrainer(model, EmbeddingConfig(loss=a.loss, pooling=pooling, temperature=a.temperature, margin=a.margin,
                                                 learning_rate=a.learning_rate, max_length=a.max_seq_len,
                                                 weight_decay=a.weight_decay, normalize=not a.no_normalize))
    steps = a.max_steps if a.max_steps is not None else a.epochs * (-(-len(rows) // a.batch_size))
    last = {}
    for step in range(steps):
        b = [rows[(step * a.batch_size + j) % len(rows)] for j in range(a.batch_size)]
        enc = lambda k: [tok.encode(r[k]) for r in b]        # noqa: E731
        last = tr.step(enc("anchor"), enc("positive"), enc("negative") if "negative" in b[0] else None,
                       [r.get("label", 1.0) for r in b] if a.loss == "cosent" else None)
        if a.log_every and (step + 1) % a.log_every == 0:
            print(json.dumps({"step": step + 1, **{k: round(v, 5) for k, v in last.items()}}), file=sys.stderr)
    save()
    print(json.dumps({"output": a.output, "steps": steps, **last}))
    return 0


# ------------------------------------------------------------------------------------------- rlkd
def _rlkd_args(sp):
    p = sp.add_parser("rlkd", help="GRPO with an added distillation term against a teacher (RLKD)")
    p.add_argument("-m", "--model", required=True)
    p.add_argument("-t", "--teacher", "--teacher-model", dest="teacher", required=True)
    p.add_argument("-d", "--dataset", required=True)
    p.add_argument("-o", "--output", default="./rlkd-output")
    p.add_argument("--alpha", "--distill-alpha", dest="alpha", type=float, default=0.5, help="weight of the KD term")
    p.add_argument("--anneal-alpha", action="store_true", help="move the KD weight linearly to --final-alpha over the run")
    p.add_argument("--final-alpha", type=float, default=0.0)
    p.add_argument("--distill-temperature", type=float, default=1.0,
                   help="accepted for compatibility: the KD term uses the log-probabilities of the sampled tokens")
    p.add_argument("--num-generations", type=int, default=8)
    p.add_argument("--beta", type=float, default=0.001)
    p.add_argument("--max-completion-length", type=int, default=512)
    p.add_argument("--max-prompt-length", type=int, default=512)
    p.add_argument("--learning-rate", type=float, default=1e-6)
    p.add_argument("--max-steps", type=int, default=None, help="default: --epochs passes over the prompts")
    p.add_argument("--epochs", type=int, default=1)
    p.add_argument("--prompts-per-step", type=int, default=1)
    p.add_argument("--lora-r", type=int, default=16)
    p.add_argument("--lora-alpha", type=float, default=None)
    p.add_argument("--seed", type=int, default=42)
    _column_args(p)
    p.add_argument("--max-seq-len", type=int, default=None,
                   help="cap on prompt + completion tokens: prompts are cut from the left to leave room for the completion")
    p.add_argument("--no-flash-attention", action="store_true", help="PyTorch reference attention instead of the kernels")
    p.add_argument("--reward-model-max-length", type=int, default=2048, help="tokens the reward model reads (cut from the right)")
    p.add_argument("--reward-model-template", help="text template with {prompt} and {completion} for the reward model")
    p.add_argument("--grpo-kv-bits", type=int, choices=[4, 8], default=None,
                   help="rollout key/value cache precision: 8 = int8 blocks, 4 = rotated 4-bit codes (default bf16)")
    p.add_argument("--reward", default="format", choices=["format", "length", "accuracy"])
    p.add_argument("--reasoning-rewards", action="store_true", help="XML format reward + answer accuracy reward")
    p.add_argument("--reward-model", help="add the score of this reward model (decoder + scalar head)")
    p.add_argument("--reward-model-weight", type=float, default=1.0)
    p.add_argument("--async-rewards", action="store_true", help="score completions on worker threads")
    p.add_argument("--checkpoint-every", type=int, default=0, help="save the adapter every N steps under checkpoints/")
    p.add_argument("--resume", action="store_true", help="continue from the newest checkpoint in the output directory")
    p.add_argument("--log-metrics", help="append one JSON line per step to this file")
    p.add_argument("--speculative", action="store_true",
                   help="accepted for compatibility: rollouts are generated as one paged batch, which replaces per-stream drafting")
    p.add_argument("--speculative-draft-tokens", type=int, default=4)
    p.add_argument("--device")
    return p


@_command(_rlkd_args)
def cmd_rlkd(a) -> int:
    a.dapo, a.rlkd_alpha = False, a.alpha
    return cmd_grpo(a)


# ------------------------------------------------------------------------------------------- search (offline)
def _search_args(sp):
    p = sp.add_parser("search", help="search models in the local Hugging Face cache, or on the hub with --online")
    p.add_argument("query", nargs="?", default="")
    p.add_argument("--limit", type=int, default=20)
    p.add_argument("--online", action="store_true")
    p.add_argument("--tag")
    p.add_argument("--detailed", action="store_true", help="full fit analysis (memory breakdown, training estimate) per result")
    p.add_argument("--download", action="store_true", help="with --online: download the first result that fits this device")
    p.add_argument("--json", action="store_true", help="the result is always JSON (accepted for compatibility)")
    return p


def local_model_index():
    """[(repo id, snapshot dir, bytes)] of every model in the local hub cache."""
    cache = os.path.join(os.environ.get("HF_HOME", os.path.expanduser("~/.cache/huggingface")), "hub")
    out = []
    if not os.path.isdir(cache):
        return out
    for name in sorted(os.listdir(cache)):
        if not name.startswith("models--"):
            continue
        snaps = os.path.join(cache, name, "snapshots")
        if not os.path.isdir(snaps) or not os.listdir(snaps):
            continue
        snap = os.path.join(snaps, sorted(os.listdir(snaps))[-1])
        size = 0
        for root, _, files in os.walk(snap):
            for f in files:
                try:
                    size += os.path.getsize(os.path.join(root, f))
                except OSError:
                    pass
        out.append((name[len("models--"):].replace("--", "/"), snap, size))
    return out


@_command(_search_args)
def cmd_search(a) -> int:
    from ..utils.sysinfo import estimate_fit
    if getattr(a, "online", False):
        from .. import hub
        try:
            res = hub.search_models(a.query, a.limit, a.tag, os.environ.get("HF_TOKEN"))
        except hub.HubError as e:
            print(f"error: {e}", file=sys.stderr)
            return 1
        out = {"query": a.query, "source": hub.endpoint(), "results": [
            {"id": r.id, "downloads": hub.format_downloads(r.downloads), "likes": r.likes, "pipeline_tag": r.pipeline_tag}
            for r in res]}
        if a.download and res:
            # sizes are only known after a download, so take the results in order and keep the first that fits
            for r in res:
                try:
                    path = hub.download_model(r.id, token=os.environ.get("HF_TOKEN"))
                    fit = estimate_fit(path, 4096, 1, 16, "none")
                except Exception as e:      # noqa: BLE001 - a failed candidate must not end the search
                    out.setdefault("skipped", []).append({"id": r.id, "reason": str(e)[:200]})
                    continue
                if fit.get("fits", True):
                    out["downloaded"] = {"id": r.id, "path": path, "fit": fit if a.detailed else fit.get("fits")}
                    break
        print(json.dumps(out, indent=2))
        return 0
    q = a.query.lower()
    rows = []
    for repo, snap, size in local_model_index():
        if q and q not in repo.lower():
            continue
        row = {"id": repo, "path": snap, "size_gb": round(size / 1e9, 3)}
        try:
            fit = estimate_fit(snap, 4096, 1, 16, "none")
            row["fits"] = fit.get("fits")
            if a.detailed:
                row["fit"] = fit
        except Exception:
            pass
        rows.append(row)
    print(json.dumps({"query": a.query, "source": "local cache", "results": rows[: a.limit]}, indent=2))
    return 0


# ------------------------------------------------------------------------------------------- dflash
def _dflash_args(sp):
    p = sp.add_parser("dflash", help="speculative decoding with a DFlash block-diffusion draft model")
    p.add_argument("-m", "--model", "--target", dest="model", required=True, help="target model directory or random:<preset>")
    p.add_argument("--draft", required=True, help="draft directory (config.json + safetensors) or 'random'")
    p.add_argument("-p", "--prompt", default="Hello")
    p.add_argument("--max-tokens", "--max-new-tokens", dest="max_tokens", type=int, default=64)
    p.add_argument("--block-size", "--speculative-tokens", dest="block_size", type=int, default=0)
    p.add_argument("--temperature", type=float, default=0.0, help="verification is greedy; values above 0 are refused")
    p.add_argument("--no-chat", action="store_true", help="the prompt is used as it is (always the case here)")
    p.add_argument("--json", action="store_true", help="the result is always one JSON line")
    p.add_argument("--draft-fp8", action="store_true", help="accepted for compatibility: the draft runs in the model dtype")
    p.add_argument("--tree-budget", type=int, default=0, help="> 0: tree verification with this many candidate nodes")
    p.add_argument("--device")
    return p


@_command(_dflash_args)
def cmd_dflash(a) -> int:
    import time

    import torch

    from ..models.dflash import DFlashDecoder, load_dflash_pair
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    if a.temperature > 0:
        print("error: block-diffusion drafting verifies greedily; use --temperature 0", file=sys.stderr)
        return 2
    target, draft, tok = load_dflash_pair(a.model, a.draft, dev)
    c = target.c
    prompt = tok.encode(a.prompt) if tok is not None else [min(ord(ch), c.vocab_size - 2) for ch in a.prompt]
    dec = DFlashDecoder(target, draft)
    t0 = time.time()
    if a.tree_budget > 0:
        out = dec.generate_tree(prompt, a.max_tokens, a.tree_budget, a.block_size or None)
    else:
        out = dec.generate(prompt, a.max_tokens, a.block_size or None)
    dt = time.time() - t0
    dec.close()
    print(json.dumps({"tokens": out, "text": tok.decode(out) if tok is not None else None,
                      "tokens_per_s": round(len(out) / max(dt, 1e-9), 2),
                      "avg_acceptance_length": round(dec.stats.avg_acceptance_length, 3),
                      "acceptance_rate": round(dec.stats.acceptance_rate, 3)}))
    return 0


# ------------------------------------------------------------------------------------------- pack-experts
def _pack_args(sp):
    p = sp.add_parser("pack-experts", help="pack the routed experts of a mixture-of-experts checkpoint into per-layer files")
    p.add_argument("-m", "--model", required=True)
    p.add_argument("-o", "--output", required=True)
    p.add_argument("--bits", type=int, default=4, choices=[2, 4])
    p.add_argument("--group-size", type=int, default=64)
    return p


def _expert_record(hidden: int, inter: int, group: int, bits: int) -> dict:
    """Byte layout of one expert inside ``layer_XX.bin``: gate, up, down, each as packed uint32 weights, bf16 scales and
    bf16 biases (crates/pmetal-models/src/expert_layout.rs:62-140)."""
    pf = 32 // bits
    comps, off = {}, 0
    for name, rows, cols in (("gate", inter, hidden), ("up", inter, hidden), ("down", hidden, inter)):
        for field, size, shape in ((f"{name}_weight", rows * (cols // pf) * 4, [rows, cols // pf]),
                                   (f"{name}_scales", rows * (cols // group) * 2, [rows, cols // group]),
                                   (f"{name}_biases", rows * (cols // group) * 2, [rows, cols // group])):
            comps[field] = {"offset": off, "size": size, "shape": shape}
            off += size
    return comps


def pack_experts(sd, out_dir: str, bits: int = 4, group_size: int = 64, model_name: str = "") -> dict:
    """Write ``layer_XX.bin`` (expert E starts at byte ``E * expert_size``) and ``layout.json`` for every layer with routed
    experts; weights are affine group-quantised on the fly (quant/mlx_affine.py). Both the stacked
    (``...experts.gate_up_proj`` [E, 2I, H]) and the per-expert (``...experts.E.{gate,up,down}_proj.weight``) checkpoint
    layouts are understood (crates/pmetal/src/pack_experts.rs)."""
    import re

    import torch

    from ..quant.mlx_affine import quantize_affine
    os.makedirs(out_dir, exist_ok=True)
    per = re.compile(r"^(?:model\.)?layers\.(\d+)\.(?:mlp|block_sparse_moe)\.experts\.(\d+)\.(gate_proj|up_proj|down_proj|w1|w2|w3)\.weight$")
    stacked = re.compile(r"^(?:model\.)?layers\.(\d+)\.(?:mlp|block_sparse_moe)\.experts\.(gate_up_proj|down_proj)$")
    role = {"gate_proj": "gate", "w1": "gate", "up_proj": "up", "w3": "up", "down_proj": "down", "w2": "down"}
    layers = {}
    for k, v in sd.items():
        m = per.match(k)
        if m:
            layers.setdefault(int(m.group(1)), {}).setdefault(int(m.group(2)), {})[role[m.group(3)]] = v
            continue
        m = stacked.match(k)
        if m:
            ex = layers.setdefault(int(m.group(1)), {})
            for e in range(v.shape[0]):
                if m.group(2) == "gate_up_proj":
                    half = v.shape[1] // 2
                    ex.setdefault(e, {})["gate"], ex[e]["up"] = v[e, :half], v[e, half:]
                else:
                    ex.setdefault(e, {})["down"] = v[e]
    if not layers:
        raise ValueError("no routed experts found in the checkpoint")
    first = next(iter(next(iter(layers.values())).values()))
    inter, hidden = first["gate"].shape
    record = _expert_record(hidden, inter, group_size, bits)
    expert_size = record["down_biases"]["offset"] + record["down_biases"]["size"]
    num_experts = max(len(ex) for ex in layers.values())
    for layer, ex in sorted(layers.items()):
        with open(os.path.join(out_dir, f"layer_{layer:02d}.bin"), "wb") as fh:
            for e in range(num_experts):
                buf = bytearray(expert_size)
                for name in ("gate", "up", "down"):
                    w, sc, bi = quantize_affine(ex[e][name].float(), bits, group_size)
                    for field, t in ((f"{name}_weight", w), (f"{name}_scales", sc.to(torch.bfloat16)),
                                     (f"{name}_biases", bi.to(torch.bfloat16))):
                        raw = t.contiguous().view(torch.uint8).numpy().tobytes()
                        c = record[field]
                        assert len(raw) == c["size"], (field, len(raw), c["size"])
                        buf[c["offset"]:c["offset"] + c["size"]] = raw
                fh.write(buf)
    layout = {"model_name": model_name, "num_layers": len(layers), "num_experts": num_experts, "hidden_dim": hidden,
              "intermediate_dim": inter, "group_size": group_size, "bits": "Four" if bits == 4 else "Two",
              "expert_size": expert_size, "moe_layer_indices": sorted(layers), "record": record}
    with open(os.path.join(out_dir, "layout.json"), "w", encoding="utf-8") as fh:
        json.dump(layout, fh, indent=1)
    return layout


def read_packed_expert(pack_dir: str, layer: int, expert: int):
    """One expert's {gate, up, down} matrices (fp32, dequantised) from a packed directory."""
    import numpy as np
    import torch

    from ..quant.mlx_affine import dequantize_affine
    with open(os.path.join(pack_dir, "layout.json"), "r", encoding="utf-8") as fh:
        lay = json.load(fh)
    bits = 4 if lay["bits"] == "Four" else 2
    with open(os.path.join(pack_dir, f"layer_{layer:02d}.bin"), "rb") as fh:
        fh.seek(expert * lay["expert_size"])
        raw = fh.read(lay["expert_size"])
    out = {}
    for name in ("gate", "up", "down"):
        parts = {}
        for field, dt in (("weight", torch.int32), ("scales", torch.bfloat16), ("biases", torch.bfloat16)):
            c = lay["record"][f"{name}_{field}"]
            arr = np.frombuffer(raw, dtype=np.uint8, count=c["size"], offset=c["offset"]).copy()
            parts[field] = torch.from_numpy(arr).view(dt).reshape(c["shape"])
        out[name] = dequantize_affine(parts["weight"], parts["scales"], parts["biases"], bits, lay["group_size"])
    return out


@_command(_pack_args)
def cmd_pack_experts(a) -> int:
    from ..models.loader import read_state_dict
    lay = pack_experts(read_state_dict(a.model), a.output, a.bits, a.group_size, os.path.basename(os.path.normpath(a.model)))
    print(json.dumps({"output": a.output, "layers": lay["num_layers"], "experts": lay["num_experts"],
                      "expert_size": lay["expert_size"]}))
    return 0


# ------------------------------------------------------------------------------------------- dashboard / tui
def _dash_args(sp):
    p = sp.add_parser("dashboard", help="follow a job-event file (--log-events output) and print progress lines")
    p.add_argument("events", nargs="?", help="JSON-lines event file")
    p.add_argument("-m", "--metrics-file", help="a --log-metrics file (one JSON object per step) instead of an event file")
    p.add_argument("--once", action="store_true", help="print the summary of what is there and exit")
    p.add_argument("--interval", type=float, default=1.0)
    p.set_defaults(func=cmd_dashboard)
    p = sp.add_parser("tui", help="terminal application: forms for every job kind, job runner, live monitor; with an "
                                  "event file it follows that file like `dashboard`")
    p.add_argument("events", nargs="?", help="JSON-lines event file to follow instead of opening the application")
    p.add_argument("--once", action="store_true")
    p.add_argument("--interval", type=float, default=1.0)
    p.add_argument("--keys", default=None,
                   help="scripted keys separated by commas (names: tab, enter, up, down, esc ... or single characters); "
                        "the application applies them, waits for the jobs it started and prints the last frame")
    p.add_argument("--workdir", default=None, help="where job logs and event files go (default: a temporary directory)")
    p.set_defaults(func=cmd_tui)
    p = sp.add_parser("gui", help="browser front end: job forms, runner and live monitor served over HTTP")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=8090)
    p.add_argument("--workdir", default=None, help="where job logs and event files go (default: a temporary directory)")
    p.set_defaults(func=cmd_gui)
    return p


def cmd_gui(a) -> int:
    from ..gui import serve_gui
    return serve_gui(a.host, a.port, a.workdir)


def cmd_tui(a) -> int:
    if a.events:
        return cmd_dashboard(a)
    from ..tui import JobRunner, TuiApp, run
    app = TuiApp(runner=JobRunner(workdir=a.workdir))
    keys = None
    if a.keys is not None:
        keys = [k if k != "comma" else "," for k in a.keys.split(",") if k != ""]
    return run(app, keys=keys)


def summarise_events(lines) -> dict:
    """Fold job events into {job_id: {kind, state, step, loss, tokens_per_s, ...}}."""
    jobs = {}
    for ln in lines:
        ln = ln.strip()
        if not ln:
            continue
        try:
            ev = json.loads(ln)
        except ValueError:
            continue
        if isinstance(ev, dict) and "event" not in ev and "step" in ev:
            # a plain metrics line (--log-metrics): the file is one job
            j = jobs.setdefault("metrics", {"state": "running", "kind": "metrics"})
            for k in ("step", "loss", "lr", "tokens_per_s", "tok_per_s", "grad_norm", "eval_loss", "reward", "kl"):
                if k in ev:
                    j[k] = ev[k]
            continue
        j = jobs.setdefault(ev.get("job_id", "?"), {"state": "running"})
        kind = ev.get("event")
        if kind == "started":
            j["kind"] = ev.get("kind")
        elif kind == "metric":
            pl = ev.get("payload") or {}
            for k in ("step", "loss", "lr", "tokens_per_s", "tok_per_s", "grad_norm", "eval_loss"):
                if k in pl:
                    j[k] = pl[k]
        elif kind in ("finished", "completed"):
            j["state"] = "finished"
        elif kind in ("failed", "error"):
            j["state"], j["error"] = "failed", ev.get("message") or (ev.get("payload") or {}).get("message")
        elif kind == "cancelled":
            j["state"] = "cancelled"
    return jobs


def cmd_dashboard(a) -> int:
    import time
    if getattr(a, "metrics_file", None):
        a.events = a.metrics_file
    if not a.events:
        print("error: an event file or --metrics-file is needed", file=sys.stderr)
        return 2
    seen = 0
    lines = []
    while True:
        if os.path.exists(a.events):
            with open(a.events, "r", encoding="utf-8") as fh:
                lines = fh.readlines()
        if len(lines) != seen or a.once:
            seen = len(lines)
            for job, st in summarise_events(lines).items():
                print(json.dumps({"job": job, **st}), flush=True)
        if a.once or all(s["state"] != "running" for s in summarise_events(lines).values()) and lines:
            return 0
        time.sleep(a.interval)


cmd_dashboard._register = lambda sp: _dash_args(sp)


# ------------------------------------------------------------------------------------------- bench-* aliases
def _bench_alias_args(sp):
    for name, what in (("bench-corpus", "corpus"), ("bench-workload", "workload"), ("bench-gen", "gen")):
        p = sp.add_parser(name, help=f"same as: bench {what}")
        p.add_argument("--case", nargs="*")
        p.add_argument("--iters", type=int, default=None)
        p.add_argument("-m", "--model", default="random:qwen3-0.6b")
        p.add_argument("--json", nargs="?", const=True, default=None,
                       help="the result is always printed as JSON; with a path it is also written there")
        p.add_argument("-o", "--output", help="write the JSON report to this file")
        p.add_argument("--device")
        p.add_argument("--experts-dir", help="stream the routed experts from this `pack-experts` directory")
        if what == "corpus":
            p.add_argument("--quick", action="store_true", help="fewer iterations per kernel case")
        else:
            from ..bench.workload import PRESETS
            p.add_argument("--preset", choices=sorted(PRESETS), help="named set of the shape options below")
            p.add_argument("--dataset", help="JSON-lines file to take prompts and training documents from (default: synthetic tokens)")
            p.add_argument("--prompt-samples", type=int, default=None, help="prompts in the inference part")
            p.add_argument("--max-prompt-tokens", type=int, default=None, help="cut prompts to this length (0: 1024)")
            p.add_argument("--inference-context", choices=["auto", "prompt", "text-prefix"], default="auto",
                           help="with --dataset: prompts are the prompt column only, or a prefix of the whole record (auto)")
            p.add_argument("--decode-steps", type=int, default=None)
            p.add_argument("--inference-warmup-passes", type=int, default=None, help="untimed passes per session")
            p.add_argument("--inference-session-repeats", type=int, default=None, help="independent sessions (fresh cache)")
            p.add_argument("--inference-repeats", type=int, default=None, help="timed passes per session")
            p.add_argument("--train-samples", type=int, default=None, help="sequences per training step")
            p.add_argument("--train-steps", type=int, default=None)
            p.add_argument("--batch-size", type=int, default=None)
            p.add_argument("--max-seq-len", "--seq-len", dest="seq_len", type=int, default=None)
        p.set_defaults(func=cmd_bench, what=what)
    p = sp.add_parser("bench-gdn", help="gated delta rule layer: projections and the recurrent update, backend against backend")
    p.add_argument("-m", "--model", help="Qwen3-Next style checkpoint directory to take the layer shapes from")
    p.add_argument("--stage", choices=["input-proj", "out-proj", "prefill"], default="prefill",
                   help="input-proj: the four input projections, one concatenated GEMM against four; out-proj: the output "
                        "projection; prefill: the recurrent update, chunked against token by token")
    p.add_argument("--layer", type=int, default=None, help="accepted for compatibility: all GDN layers share one shape")
    p.add_argument("--batch-size", type=int, default=1)
    p.add_argument("--seq-len", type=int, default=None, help="tokens (same as --tokens)")
    p.add_argument("--tokens", type=int, default=512)
    p.add_argument("--heads", type=int, default=8)
    p.add_argument("--warmup-iterations", type=int, default=2)
    p.add_argument("--benchmark-iterations", type=int, default=5)
    p.add_argument("--json", action="store_true", help="the result is always JSON")
    p.add_argument("-o", "--output", help="write the JSON report to this file")
    p.add_argument("--device")
    p.set_defaults(func=cmd_bench_gdn)
    p = sp.add_parser("bench-ffi", help="cost of one call into the native host library")
    p.add_argument("--calls", type=int, default=200000)
    p.set_defaults(func=cmd_bench_ffi)
    p = sp.add_parser("bench-skinny", help="few-row linear layers: mat-vec and narrow-tile GEMM kernels against cuBLAS")
    p.set_defaults(func=lambda a: __import__("pmetal_b200.bench.skinny", fromlist=["main"]).main(args=a))
    p = sp.add_parser("bench-decode", help="short decode runs for profiling; --phases prints per-phase device times of "
                                           "the whole-step decode kernel")
    from ..bench.decode_trace import add_arguments as _decode_trace_args
    _decode_trace_args(p)
    p.set_defaults(func=lambda a: __import__("pmetal_b200.bench.decode_trace", fromlist=["main"]).main(args=a))
    return p


def cmd_bench_gdn(a) -> int:
    import time

    import torch

    from ..models.gdn import gdn_chunked, gdn_recurrent
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    shape = {"hidden_size": 2048, "linear_num_key_heads": 16, "linear_num_value_heads": 32, "linear_key_head_dim": 128,
             "linear_value_head_dim": 128}
    if a.model and os.path.isfile(os.path.join(a.model, "config.json")):
        with open(os.path.join(a.model, "config.json"), "r", encoding="utf-8") as fh:
            cfg = json.load(fh)
        cfg = cfg.get("text_config") or cfg
        shape.update({k: cfg[k] for k in shape if cfg.get(k)})
    T = (a.seq_len or a.tokens) * max(1, a.batch_size)

    def timed(fn):
        for _ in range(max(0, a.warmup_iterations)):
            fn()
        if dev.startswith("cuda"):
            torch.cuda.synchronize()
        ts = []
        for _ in range(max(1, a.benchmark_iterations)):
            t0 = time.perf_counter()
            y = fn()
            if dev.startswith("cuda"):
                torch.cuda.synchronize()
            ts.append(time.perf_counter() - t0)
        ts.sort()
        return {"ms": round(ts[len(ts) // 2] * 1e3, 3)}, y

    g = torch.Generator().manual_seed(0)
    dt = torch.bfloat16 if dev.startswith("cuda") else torch.float32
    res = {}

    def lin(x, w):
        """The projection as the models run it: the tensor-core GEMM of this package on a GPU."""
        from ..ops import functional as ops
        if x.is_cuda and ops.use_native(x) and w.shape[0] % 8 == 0 and w.shape[1] % 8 == 0:
            return ops.lora_linear(x, w, None, None, None, (w.shape[0],), 0, 0.0, None)
        return torch.nn.functional.linear(x, w)

    if a.stage == "prefill":
        H, d = a.heads, 64
        q, k = (torch.nn.functional.normalize(torch.randn(T, H, d, generator=g), dim=-1).to(dev) for _ in range(2))
        v = torch.randn(T, H, d, generator=g).to(dev)
        gate, beta = torch.rand(T, H, generator=g).mul(0.2).add(0.8).to(dev), torch.rand(T, H, generator=g).to(dev)
        res["recurrent"], y0 = timed(lambda: gdn_recurrent(q, k, v, gate, beta)[0])
        for chunk in (32, 64, 128):
            res[f"chunked_{chunk}"], y = timed(lambda c=chunk: gdn_chunked(q, k, v, gate, beta, chunk=c)[0])
            res[f"chunked_{chunk}"]["max_abs_diff"] = float((y - y0).abs().max())
        res["chunked"] = res["chunked_64"]
        out = {"stage": a.stage, "tokens": T, "heads": H, "device": dev, **res, "max_abs_diff": res["chunked_64"]["max_abs_diff"]}
    else:
        hid = shape["hidden_size"]
        kd = shape["linear_num_key_heads"] * shape["linear_key_head_dim"]
        vd = shape["linear_num_value_heads"] * shape["linear_value_head_dim"]
        nv = shape["linear_num_value_heads"]
        if a.stage == "input-proj":
            dims = {"qkv": 2 * kd + vd, "z": vd, "b": nv, "a": nv}
            x = torch.randn(T, hid, generator=g).to(dev, dt)
            ws = {n: (torch.randn(o, hid, generator=g) * 0.02).to(dev, dt) for n, o in dims.items()}
            cat = torch.cat(list(ws.values()), 0)
            res["separate"], ys = timed(lambda: torch.cat([lin(x, w) for w in ws.values()], -1))
            res["concatenated"], yc = timed(lambda: lin(x, cat))
            res["max_abs_diff"] = float((ys.float() - yc.float()).abs().max())
            flops = 2.0 * T * hid * sum(dims.values())
        else:
            x = torch.randn(T, vd, generator=g).to(dev, dt)
            w = (torch.randn(hid, vd, generator=g) * 0.02).to(dev, dt)
            res["linear"], _ = timed(lambda: lin(x, w))
            flops = 2.0 * T * hid * vd
        for r in res.values():
            if isinstance(r, dict):
                r["tflops"] = round(flops / (r["ms"] * 1e-3) / 1e12, 3)
        out = {"stage": a.stage, "tokens": T, "device": dev, "shape": shape, **res}
    print(json.dumps(out))
    if a.output:
        with open(a.output, "w", encoding="utf-8") as fh:
            json.dump(out, fh, indent=2)
    return 0


def cmd_bench_ffi(a) -> int:
    import time

    from ..gguf import native
    from ..gguf.types import GgmlType
    fn = native.lib().pm_gguf_block_elems
    t0 = time.perf_counter()
    for _ in range(a.calls):
        fn(int(GgmlType.Q4K))
    dt = time.perf_counter() - t0
    print(json.dumps({"calls": a.calls, "ns_per_call": round(dt / a.calls * 1e9, 1)}))
    return 0


cmd_bench_gdn._register = lambda sp: _bench_alias_args(sp)
