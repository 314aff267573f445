"""LoRA on the portable architectures: wrapping, adapter files, merge, and the training orchestrator's portable path."""
import json
import os

import pytest
import torch

tf = pytest.importorskip("transformers")

from pmetal_b200.core.config import LoraConfig
from pmetal_b200.lora import portable as P
from pmetal_b200.models.architectures import build_model, load_pretrained


def _tiny_gemma_dir(tmp_path):
    """A tiny Gemma 3 checkpoint with a byte-level tokenizer, written the way the hub lays a model out."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    torch.manual_seed(0)
    cfg = tf.Gemma3TextConfig(vocab_size=300, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2,
                              num_key_value_heads=1, head_dim=16, sliding_window=8, max_position_embeddings=128)
    hf = tf.Gemma3ForCausalLM(cfg)
    d = tmp_path / "gemma"
    hf.save_pretrained(str(d), safe_serialization=True)
    vocab = {chr(i) if 32 <= i < 127 else f"<0x{i:02X}>": i for i in range(256)}
    vocab.update({"<pad>": 256, "<eos>": 257, "<bos>": 258})
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<pad>"))
    tok.pre_tokenizer = pre_tokenizers.Split("", "isolated")
    tok.save(str(d / "tokenizer.json"))
    (d / "tokenizer_config.json").write_text(json.dumps({"eos_token": "<eos>", "pad_token": "<pad>", "bos_token": "<bos>"}))
    return str(d)


def test_wrap_save_load_merge(tmp_path):
    d = _tiny_gemma_dir(tmp_path)
    model = load_pretrained(d, torch.float32).eval()
    ids = torch.randint(0, 256, (2, 12), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        base = model(ids)
    cfg = LoraConfig(r=4, alpha=8.0, target_modules=["q_proj", "v_proj", "down_proj"])
    P.apply_lora_portable(model, cfg)
    mods = P.lora_modules(model)
    assert set(mods) == {f"layers.{i}.{s}" for i in range(2) for s in ("self_attn.q_proj", "self_attn.v_proj", "mlp.down_proj")}
    assert all(p.requires_grad == ("lora_" in n) for n, p in model.named_parameters())
    with torch.no_grad():
        assert torch.allclose(model(ids), base, atol=1e-6)                       # B = 0: the adapted model is the base model
        for m in mods.values():
            m.lora_b.normal_(std=0.05)
        tuned = model(ids)
    assert not torch.allclose(tuned, base, atol=1e-4)
    P.save_adapter_portable(model, str(tmp_path / "ad"), cfg, d)
    sd = __import__("pmetal_b200.utils.safetensors_io", fromlist=["x"]).load_file(str(tmp_path / "ad" / "lora_weights.safetensors"))
    assert sd["layers.0.self_attn.q_proj.lora_a"].shape == (4, 32) and sd["layers.1.mlp.down_proj.lora_b"].shape == (32, 4)
    fresh = P.apply_lora_portable(load_pretrained(d, torch.float32).eval(), cfg)
    assert P.load_adapter_portable(fresh, str(tmp_path / "ad")) == 6
    with torch.no_grad():
        assert torch.allclose(fresh(ids), tuned, atol=1e-5)
        merged = P.merge_lora_portable(fresh)
        assert not P.lora_modules(merged) and torch.allclose(merged(ids), tuned, atol=1e-4)
    # the adapter file is in the common format: the fuse command folds it into the checkpoint
    from pmetal_b200.cli.main import main
    assert main(["fuse", "-m", d, "-l", str(tmp_path / "ad"), "-o", str(tmp_path / "fused"), "--dtype", "float32"]) == 0
    with torch.no_grad():
        assert torch.allclose(load_pretrained(str(tmp_path / "fused"), torch.float32).eval()(ids), tuned, atol=1e-4)


def test_dora_and_trainer_reduce_the_loss():
    from pmetal_b200.models.architectures.generic import GenericDecoderLM
    torch.manual_seed(0)
    cfg = tf.LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2,
                         num_key_value_heads=1, max_position_embeddings=64).to_dict()
    model = GenericDecoderLM.from_hf_config(cfg).init_weights(0.05, 0)
    lc = LoraConfig(r=4, alpha=8.0, target_modules=["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"],
                    use_dora=True)
    P.apply_lora_portable(model, lc)
    assert any(n.endswith("magnitude") for n, _ in model.named_parameters())
    tr = P.PortableLoraTrainer(model, learning_rate=5e-3, warmup_steps=2, total_steps=40, loraplus_ratio=4.0)
    ids = torch.randint(0, 64, (4, 16), generator=torch.Generator().manual_seed(2))
    losses = [tr.step(ids, ids.clone())["loss"] for _ in range(40)]
    assert losses[-1] < 0.8 * losses[0]
    with pytest.raises(ValueError):
        P.apply_lora_portable(GenericDecoderLM.from_hf_config(cfg), LoraConfig(r=2, target_modules=["nothing"]))


def test_train_command_takes_the_portable_path_for_gemma(tmp_path, capsys):
    from pmetal_b200.cli.main import main
    d = _tiny_gemma_dir(tmp_path)
    data = tmp_path / "d.jsonl"
    data.write_text("".join(json.dumps({"text": "the cat sat on the mat and looked at the dog"}) + "\n" for _ in range(8)))
    out = str(tmp_path / "out")
    assert main(["train", "-m", d, "-d", str(data), "-o", out, "--lora-r", "4", "--lora-alpha", "8", "--learning-rate", "5e-3",
                 "--batch-size", "4", "--max-steps", "6", "--warmup-steps", "0", "--device", "cpu", "--dtype", "float32",
                 "--log-metrics", str(tmp_path / "m.jsonl"), "--no-adaptive-lr"]) == 0
    summary = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert summary["path"] == "portable" and summary["steps"] == 6
    assert os.path.exists(os.path.join(out, "lora_weights.safetensors"))
    assert json.load(open(os.path.join(out, "adapter_config.json")))["r"] == 4
    steps = [json.loads(l) for l in open(tmp_path / "m.jsonl") if '"step"' in l]
    assert len(steps) == 6 and steps[-1]["loss"] < steps[0]["loss"]


def test_portable_path_accumulates_micro_batches_and_resumes(tmp_path, capsys):
    """16 samples, batch 2, accumulation 4, one epoch: two optimiser steps that together see every token of the data;
    a second run with --resume continues the step count and the optimiser instead of starting over."""
    from pmetal_b200.cli.main import main
    d = _tiny_gemma_dir(tmp_path)
    data = tmp_path / "d.jsonl"
    rows = ["the cat sat on the mat " * (1 + i % 3) for i in range(16)]
    data.write_text("".join(json.dumps({"text": r}) + "\n" for r in rows))
    out = str(tmp_path / "out")
    args = ["train", "-m", d, "-d", str(data), "-o", out, "--lora-r", "4", "--lora-alpha", "8", "--batch-size", "2",
            "--gradient-accumulation-steps", "4", "--epochs", "1", "--warmup-steps", "0", "--device", "cpu", "--dtype",
            "float32", "--log-metrics", str(tmp_path / "m.jsonl"), "--no-adaptive-lr", "--no-sequence-packing"]
    assert main(args) == 0
    summary = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    steps = [json.loads(l) for l in open(tmp_path / "m.jsonl") if '"step"' in l]
    assert summary["steps"] == 2 and len(steps) == 2
    from pmetal_b200.data.dataset import TrainingDataset
    from pmetal_b200.data.tokenizer import Tokenizer
    ds = TrainingDataset.from_file_tokenized(str(data), Tokenizer.from_model_dir(d), 2048, "auto", None, None, None)
    assert summary["tokens"] == sum(len(x) for x in ds.samples)        # nothing skipped, nothing seen twice
    state = torch.load(os.path.join(out, "portable_trainer_state.pt"), weights_only=True)
    assert state["step"] == 2 and state["trainer"]["step"] == 2
    assert main(args + ["--resume", "--max-steps", "3"]) == 0
    summary = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert summary["steps"] == 3
    state = torch.load(os.path.join(out, "portable_trainer_state.pt"), weights_only=True)
    assert state["trainer"]["step"] == 3 and state["trainer"]["optimizer"]["state"]


def test_infer_command_runs_portable_models_with_adapter_and_quantised_cache(tmp_path, capsys):
    from pmetal_b200.cli.main import main
    d = _tiny_gemma_dir(tmp_path)
    assert main(["infer", "-m", d, "-p", "hello", "--max-tokens", "5", "--greedy", "--json", "--device", "cpu"]) == 0
    a = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert a["path"] == "portable" and a["prompt_tokens"] == 5 and a["generated_tokens"] <= 5
    assert main(["infer", "-m", d, "-p", "hello", "--max-tokens", "5", "--greedy", "--json", "--kv-quant", "--device", "cpu"]) == 0
    b = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert b["generated_tokens"] == a["generated_tokens"]
    model = load_pretrained(d, torch.float32)
    cfg = LoraConfig(r=2, alpha=4.0, target_modules=["q_proj"])
    P.apply_lora_portable(model, cfg)
    P.save_adapter_portable(model, str(tmp_path / "ad"), cfg, d)
    assert main(["infer", "-m", d, "-l", str(tmp_path / "ad"), "-p", "hello", "--max-tokens", "5", "--greedy", "--json",
                 "--device", "cpu"]) == 0
    c = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert c["text"] == a["text"]                                                  # a fresh adapter (B = 0) changes nothing


def test_eval_command_on_a_portable_model_sees_the_adapter(tmp_path, capsys):
    from pmetal_b200.cli.main import main
    d = _tiny_gemma_dir(tmp_path)
    data = tmp_path / "d.jsonl"
    data.write_text("".join(json.dumps({"text": "the cat sat on the mat and looked at the dog"}) + "\n" for _ in range(8)))
    out = str(tmp_path / "out")
    assert main(["train", "-m", d, "-d", str(data), "-o", out, "--lora-r", "4", "--learning-rate", "1e-2", "--batch-size", "4",
                 "--max-steps", "12", "--warmup-steps", "0", "--device", "cpu", "--dtype", "float32", "--no-adaptive-lr"]) == 0
    capsys.readouterr()
    assert main(["eval", "-m", d, "-d", str(data), "--device", "cpu"]) == 0
    base = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert main(["eval", "-m", d, "-l", out, "-d", str(data), "--device", "cpu"]) == 0
    tuned = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert base["path"] == "portable" and tuned["loss"] < base["loss"]


def test_qblora_starts_at_the_base_and_balances_gradients():
    torch.manual_seed(0)
    base = torch.nn.Linear(32, 24, bias=False)
    x = torch.randn(5, 32)
    g = torch.Generator().manual_seed(1)
    ad = P.QBLoraLinear(base, 32, 24, r=4, scale=2.0, input_proj_dim=16, output_proj_dim=12, rank_multiplier=2.0, generator=g)
    assert ad.r == 8 and ad.lora_a.shape == (8, 16) and ad.lora_b.shape == (12, 8) and len(ad.trainable_parameters()) == 4
    assert torch.allclose(ad(x), base(x)) and not base.weight.requires_grad
    with torch.no_grad():
        ad.lora_b.normal_(std=0.1)
    want = base(x) + 2.0 * ((((x @ ad.p_in) @ ad.lora_a.t()) @ ad.lora_b.t()) @ ad.p_out)
    assert torch.allclose(ad(x), want, atol=1e-5)
    ad(x).sum().backward()
    g1 = ad.lora_a.grad.clone()
    ad.zero_grad()
    ad.gradient_scale = 0.5
    y = ad(x)
    assert torch.allclose(y, want, atol=1e-5)                                  # the forward value does not change
    y.sum().backward()
    assert torch.allclose(ad.lora_a.grad, 0.5 * g1, atol=1e-6)
    fixed = P.QBLoraLinear(torch.nn.Linear(32, 24), 32, 24, 4, 1.0, 16, None, learnable_projections=False)
    assert len(fixed.trainable_parameters()) == 2 and fixed.p_in_fixed.shape == (32, 16)


@pytest.mark.parametrize("family,extra", [("cohere", dict(logit_scale=0.25)), ("gemma2", dict(final_logit_softcapping=20.0)),
                                          ("granite", dict(logits_scaling=4.0)), ("llama", {})])
def test_trainer_loss_without_materialised_logits_matches_forward(family, extra):
    """The fused read-out + cross entropy (logit scale, soft cap) equals the loss on the model's own logits, value and gradient."""
    import torch
    from pmetal_b200.lora import portable as P
    from pmetal_b200.models.architectures.generic import GenericDecoderLM, arch_config_from_hf
    cfg = dict(model_type=family, vocab_size=96, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
               num_attention_heads=4, num_key_value_heads=2, head_dim=8, max_position_embeddings=64)
    cfg.update(extra)
    torch.manual_seed(0)
    m = GenericDecoderLM(arch_config_from_hf(cfg)).init_weights(0.2, 0)
    P.apply_lora_portable(m, LoraConfig(r=4, alpha=8.0, target_modules=["q_proj", "v_proj", "down_proj"]))
    tr = P.PortableLoraTrainer(m, total_steps=4)
    assert m.loss_head() is not None
    ids = torch.randint(0, 96, (3, 17))
    labels = ids.clone()
    labels[:, :4] = -100
    a = tr.loss(ids, labels)
    ga = torch.autograd.grad(a, [p for p in m.parameters() if p.requires_grad], allow_unused=True)
    b = P.causal_lm_loss(m(ids), labels)
    gb = torch.autograd.grad(b, [p for p in m.parameters() if p.requires_grad], allow_unused=True)
    assert abs(float(a) - float(b)) < 1e-5 * max(1.0, abs(float(b)))
    for x, y in zip(ga, gb):
        if x is not None:
            assert torch.allclose(x, y, atol=1e-6, rtol=1e-4)


def test_serve_command_answers_http_for_a_portable_family(tmp_path):
    """``serve -m <gemma directory>`` picks the sequential engine and answers the OpenAI routes."""
    import signal
    import subprocess
    import sys
    import time
    import urllib.request
    d = _tiny_gemma_dir(tmp_path)
    port = 18437
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.Popen([sys.executable, "-m", "pmetal_b200.cli.main", "serve", "-m", d, "--device", "cpu", "--port", str(port),
                          "--max-slots", "4"], cwd=root, start_new_session=True, stdout=subprocess.PIPE,
                         stderr=subprocess.STDOUT, text=True)
    try:
        up = False
        for _ in range(240):
            try:
                urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=1).read()
                up = True
                break
            except Exception:
                if p.poll() is not None:
                    break
                time.sleep(0.5)
        assert up, "server did not come up: " + (p.stdout.read()[-2000:] if p.poll() is not None else "")
        outs = []
        for _ in range(2):
            req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/completions",
                                         data=json.dumps({"prompt": "hello", "max_tokens": 6, "temperature": 0}).encode(),
                                         headers={"Content-Type": "application/json"})
            outs.append(json.loads(urllib.request.urlopen(req, timeout=120).read()))
        assert outs[0]["usage"]["completion_tokens"] <= 6 and outs[0]["usage"]["prompt_tokens"] >= 5
        assert outs[0]["choices"][0]["text"] == outs[1]["choices"][0]["text"]
        models = json.loads(urllib.request.urlopen(f"http://127.0.0.1:{port}/v1/models", timeout=10).read())
        assert models["data"][0]["id"] == "gemma"
    finally:
        os.killpg(p.pid, signal.SIGINT)
        try:
            p.communicate(timeout=60)
        except subprocess.TimeoutExpired:
            os.killpg(p.pid, signal.SIGKILL)
            p.communicate()


def test_grpo_on_a_portable_family_updates_the_adapters_and_keeps_the_reference(tmp_path, capsys):
    import math
    from pmetal_b200.lora.portable import lora_modules
    from pmetal_b200.trainer.grpo import GrpoConfig, mod7_length_reward
    from pmetal_b200.trainer.grpo_portable import PortableGrpoTrainer
    d = _tiny_gemma_dir(tmp_path)
    model = load_pretrained(d, torch.float32)
    P.apply_lora_portable(model, LoraConfig(r=4, alpha=8.0, target_modules=["q_proj", "v_proj", "down_proj"]))
    with torch.no_grad():
        for m in lora_modules(model).values():
            m.lora_b.normal_(0, 0.05)
    cfg = GrpoConfig(num_generations=4, max_completion_length=6, beta=0.05, learning_rate=1e-2, top_k=0, top_p=1.0)
    tr = PortableGrpoTrainer(model, cfg, mod7_length_reward, eos_ids=[257], pad_id=256, logprob_batch=5)
    prompts = [torch.randint(0, 256, (7,)).tolist() for _ in range(3)]
    before = {k: m.lora_b.detach().clone() for k, m in lora_modules(model).items()}
    base_w = {k: m.base.weight.detach().clone() for k, m in lora_modules(model).items()}
    st = tr.step(prompts)
    assert math.isfinite(st.loss) and 0 < st.completion_tokens <= 3 * 4 * 6 and st.kl >= 0.0
    assert any(not torch.equal(before[k], m.lora_b) for k, m in lora_modules(model).items())
    assert all(torch.equal(base_w[k], m.base.weight) for k, m in lora_modules(model).items())
    # reference log-probabilities are those of the base model: the adapters are switched off and back on
    seqs, plens = [prompts[0] + [5, 6, 7]], [len(prompts[0])]
    ref_lp, _ = tr._completion_logps(tr.ref, seqs, plens, grad=False)
    pol_lp, _ = tr._completion_logps(tr.policy, seqs, plens, grad=False)
    assert not torch.allclose(pol_lp, ref_lp)                     # the policy itself is scored with its adapters on
    scales = [m.scale for m in lora_modules(model).values()]
    assert all(s != 0.0 for s in scales)
    plain = load_pretrained(d, torch.float32).eval()
    with torch.no_grad():
        lg = plain(torch.tensor(seqs))[0]
    want = torch.log_softmax(lg[len(prompts[0]) - 1:-1].float(), -1).gather(-1, torch.tensor([5, 6, 7])[:, None])[:, 0]
    assert torch.allclose(ref_lp, want, atol=1e-5)
    # the command takes the same path for a portable model directory
    from pmetal_b200.cli.main import main
    data = tmp_path / "p.jsonl"
    data.write_text("\n".join(json.dumps({"prompt": f"question {i}"}) for i in range(3)))
    out = str(tmp_path / "grpo")
    assert main(["grpo", "-m", d, "-d", str(data), "-o", out, "--max-steps", "1", "--num-generations", "2",
                 "--max-completion-length", "4", "--lora-r", "4", "--device", "cpu", "--reward", "length"]) == 0
    assert os.path.exists(os.path.join(out, "adapter_config.json"))
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["path"] == "portable"


def test_distill_command_with_portable_student_and_teacher(tmp_path, capsys):
    """``distill`` between config-driven models: LoRA student (adapter written in the portable format) and full-parameter
    student (a loadable model directory)."""
    from pmetal_b200.cli.main import main
    d = _tiny_gemma_dir(tmp_path)
    data = tmp_path / "p.jsonl"
    data.write_text("\n".join(json.dumps({"prompt": f"question {i} about things"}) for i in range(4)))
    out = str(tmp_path / "kd")
    assert main(["distill", "--teacher", d, "--student", d, "-d", str(data), "-o", out, "--max-steps", "2", "--lora-r", "4",
                 "--device", "cpu"]) == 0
    j = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert j["steps"] == 2 and os.path.exists(os.path.join(out, "lora_weights.safetensors"))
    m = load_pretrained(d, torch.float32)
    P.apply_lora_portable(m, P.load_adapter_config(out) if hasattr(P, "load_adapter_config") else LoraConfig(r=4, alpha=8.0))
    assert P.load_adapter_portable(m, out) > 0
    out2 = str(tmp_path / "kd_full")
    assert main(["distill", "--teacher", d, "--student", d, "-d", str(data), "-o", out2, "--max-steps", "2", "--lora-r", "0",
                 "--device", "cpu", "--loss-type", "reverse_kl", "--learning-rate", "1e-3"]) == 0
    tuned = load_pretrained(out2, torch.float32).eval()
    base = load_pretrained(d, torch.float32).eval()
    ids = torch.randint(0, 256, (1, 9))
    with torch.no_grad():
        assert not torch.allclose(tuned(ids), base(ids))          # the weights moved and the directory loads


def test_qlora_on_a_portable_family(tmp_path, capsys):
    """Packed base projections: close to the full-precision model, adapters train, merging gives plain matrices back, and
    ``train --quantization nf4`` runs the whole path for a Gemma directory."""
    from pmetal_b200.lora.portable import QuantLinear, quantize_base_portable
    d = _tiny_gemma_dir(tmp_path)
    full = load_pretrained(d, torch.float32).eval()
    model = load_pretrained(d, torch.float32)
    saved = quantize_base_portable(model, "nf4", 64, double_quant=True)
    packed = [m for m in model.modules() if isinstance(m, QuantLinear)]
    assert saved > 0 and len(packed) == 2 * 7 and not isinstance(model.lm_head if hasattr(model, "lm_head") else None, QuantLinear)
    ids = torch.randint(0, 256, (2, 11), generator=torch.Generator().manual_seed(3))
    with torch.no_grad():
        a, b = full(ids), model.eval()(ids)
    assert (a - b).norm() / a.norm() < 0.35                      # 4-bit weights of a random tiny model: close, not equal
    P.apply_lora_portable(model, LoraConfig(r=4, alpha=8.0, target_modules=["q_proj", "v_proj", "down_proj"]))
    assert all(isinstance(m.base, QuantLinear) for m in P.lora_modules(model).values())
    tr = P.PortableLoraTrainer(model.train(), learning_rate=2e-2, total_steps=30)
    losses = [tr.step(ids, ids.clone())["loss"] for _ in range(30)]
    assert losses[-1] < 0.97 * losses[0]
    with torch.no_grad():
        tuned = model.eval()(ids)
    P.merge_lora_portable(model)
    assert not P.lora_modules(model)
    with torch.no_grad():
        assert torch.allclose(model(ids), tuned, atol=1e-4)
    from pmetal_b200.cli.main import main
    data = tmp_path / "t.jsonl"
    data.write_text("".join(json.dumps({"text": "hello world " * 6}) + "\n" for _ in range(8)))
    out = str(tmp_path / "qlora")
    assert main(["train", "--model", d, "--dataset", str(data), "--output", out, "--max-steps", "2", "--lora-r", "4",
                 "--quantization", "nf4", "--device", "cpu", "--dtype", "float32"]) == 0
    assert os.path.exists(os.path.join(out, "lora_weights.safetensors"))


def test_packed_rows_equal_separate_documents_and_train_command_packs(tmp_path, capsys):
    """Documents packed into one row (positions restart, attention inside each document) give the loss of the documents run
    one by one; the train command packs by default for a Gemma directory."""
    from pmetal_b200.data.dataloader import PackedDataLoader
    from pmetal_b200.data.packing import Sample
    d = _tiny_gemma_dir(tmp_path)
    model = load_pretrained(d, torch.float32)
    P.apply_lora_portable(model, LoraConfig(r=4, alpha=8.0, target_modules=["q_proj", "v_proj"]))
    with torch.no_grad():
        for m in P.lora_modules(model).values():
            m.lora_b.normal_(0, 0.05)
    tr = P.PortableLoraTrainer(model, total_steps=2)
    g = torch.Generator().manual_seed(5)
    docs = [torch.randint(0, 256, (n,), generator=g).tolist() for n in (9, 14, 6, 11)]
    loader = PackedDataLoader([Sample(x, list(x)) for x in docs], 24, packs_per_batch=2, shuffle=False)
    assert len(loader.packs) == 2                                  # two rows of 24 hold the 40 tokens
    batch = next(iter(loader))
    ids, labels = batch.input_ids.view(2, 24), batch.labels.view(2, 24)
    packed = tr.loss(ids, labels, batch.position_ids.view(2, 24).long(), batch.seq_start.view(2, 24).long())
    tot, cnt = 0.0, 0
    for x in docs:
        t = torch.tensor([x])
        n = len(x) - 1
        tot += float(tr.loss(t, t.clone())) * n
        cnt += n
    assert abs(float(packed) - tot / cnt) < 1e-4
    from pmetal_b200.cli.main import main
    data = tmp_path / "t.jsonl"
    data.write_text("".join(json.dumps({"text": "hello world " * (2 + i % 3)}) + "\n" for i in range(12)))
    out = str(tmp_path / "packed")
    assert main(["train", "--model", d, "--dataset", str(data), "--output", out, "--max-steps", "2", "--lora-r", "4",
                 "--device", "cpu", "--dtype", "float32", "--batch-size", "2", "--gradient-accumulation-steps", "1"]) == 0
    j = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert j["path"] == "portable" and j["steps"] == 2 and os.path.exists(os.path.join(out, "lora_weights.safetensors"))


def test_infer_command_with_a_draft_for_a_portable_target(tmp_path, capsys):
    from pmetal_b200.cli.main import main
    d = _tiny_gemma_dir(tmp_path)
    assert main(["infer", "-m", d, "-p", "hello", "--max-tokens", "8", "--greedy", "--json", "--device", "cpu"]) == 0
    plain = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert main(["infer", "-m", d, "-p", "hello", "--max-tokens", "8", "--greedy", "--json", "--device", "cpu",
                 "--draft-model", d]) == 0
    spec = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert spec["speculative"] and spec["text"] == plain["text"] and spec["acceptance_rate"] == 1.0


def test_python_api_loads_generates_streams_and_saves_a_portable_model(tmp_path):
    import pmetal_b200 as pm
    d = _tiny_gemma_dir(tmp_path)
    m = pm.Model.load(d, device="cpu")
    assert m.portable
    text = m.generate("hello", max_tokens=6, temperature=0)
    assert isinstance(text, str)
    assert "".join(m.stream("hello", max_tokens=6, temperature=0)) == text
    out = str(tmp_path / "copy")
    m.save(out)
    again = pm.Model.load(out, device="cpu")
    assert again.generate("hello", max_tokens=6, temperature=0) == text
    assert pm.infer(d, "hello", max_tokens=3, temperature=0) == m.generate("hello", max_tokens=3, temperature=0)


def test_rlkd_command_on_a_portable_policy_with_a_portable_teacher(tmp_path, capsys):
    from pmetal_b200.cli.main import main
    d = _tiny_gemma_dir(tmp_path)
    data = tmp_path / "p.jsonl"
    data.write_text("\n".join(json.dumps({"prompt": f"question {i}"}) for i in range(3)))
    out = str(tmp_path / "rlkd")
    assert main(["rlkd", "-m", d, "--teacher", d, "-d", str(data), "-o", out, "--max-steps", "1", "--num-generations", "2",
                 "--max-completion-length", "4", "--lora-r", "4", "--device", "cpu", "--reward", "length", "--alpha", "0.5",
                 "--log-metrics", str(tmp_path / "m.jsonl")]) == 0
    assert os.path.exists(os.path.join(out, "adapter_config.json"))
    line = json.loads(open(tmp_path / "m.jsonl").read().strip().splitlines()[-1])
    assert "kd_loss" in line and "rl_loss" in line and line["kd_loss"] >= 0.0


def _tiny_bert_dir(tmp_path):
    from tokenizers import Tokenizer, models, pre_tokenizers
    torch.manual_seed(0)
    cfg = tf.BertConfig(vocab_size=300, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
                        max_position_embeddings=64)
    d = tmp_path / "bert"
    tf.BertModel(cfg).save_pretrained(str(d), safe_serialization=True)
    vocab = {chr(i) if 32 <= i < 127 else f"<0x{i:02X}>": i for i in range(256)}
    vocab.update({"[PAD]": 256, "[SEP]": 257, "[CLS]": 258})
    tok = Tokenizer(models.WordLevel(vocab, unk_token="[PAD]"))
    tok.pre_tokenizer = pre_tokenizers.Split("", "isolated")
    tok.save(str(d / "tokenizer.json"))
    (d / "tokenizer_config.json").write_text(json.dumps({"pad_token": "[PAD]", "sep_token": "[SEP]", "cls_token": "[CLS]"}))
    return str(d)


def test_embedding_training_on_an_encoder_and_a_portable_decoder(tmp_path, capsys):
    """InfoNCE on a BERT encoder (all weights, then adapters) and on a Gemma decoder: the loss falls, the command writes
    a model directory or an adapter."""
    from pmetal_b200.cli.main import main
    from pmetal_b200.trainer.embedding import EmbeddingConfig, EmbeddingTrainer
    bert = _tiny_bert_dir(tmp_path)
    enc = load_pretrained(bert, torch.float32)
    for p in enc.parameters():
        p.requires_grad_(True)
    tr = EmbeddingTrainer(enc.train(), EmbeddingConfig(learning_rate=2e-3, pooling="cls"))
    g = torch.Generator().manual_seed(1)
    anchors = [torch.randint(0, 256, (n,), generator=g).tolist() for n in (6, 9, 4, 7)]
    positives = [a[::-1] for a in anchors]
    first = tr.step(anchors, positives)["loss"]
    for _ in range(20):
        last = tr.step(anchors, positives)["loss"]
    assert last < 0.7 * first
    e = tr.encode(anchors)
    assert e.shape == (4, 32) and torch.allclose(e.norm(dim=-1), torch.ones(4), atol=1e-5)
    gem = load_pretrained(_tiny_gemma_dir(tmp_path), torch.float32)
    P.apply_lora_portable(gem, LoraConfig(r=4, alpha=8.0, target_modules=["q_proj", "v_proj", "o_proj"]))
    t2 = EmbeddingTrainer(gem.train(), EmbeddingConfig(learning_rate=2e-2, pooling="last"))
    a0 = t2.step(anchors, positives)["loss"]
    for _ in range(25):
        b0 = t2.step(anchors, positives)["loss"]
    assert b0 < a0
    data = tmp_path / "pairs.jsonl"
    data.write_text("".join(json.dumps({"anchor": f"query {i}", "positive": f"answer {i}"}) + "\n" for i in range(8)))
    out = str(tmp_path / "emb_full")
    assert main(["embed-train", "-m", bert, "-d", str(data), "-o", out, "--max-steps", "3", "--batch-size", "4", "--lora-r", "0",
                 "--device", "cpu", "--pooling", "mean", "--learning-rate", "1e-3"]) == 0
    assert os.path.exists(os.path.join(out, "model.safetensors")) and os.path.exists(os.path.join(out, "config.json"))
    tuned = load_pretrained(out, torch.float32)
    assert not torch.equal(tuned.encoder.layer[0].attention.self.query.weight,
                           load_pretrained(bert, torch.float32).encoder.layer[0].attention.self.query.weight)
    out2 = str(tmp_path / "emb_lora")
    assert main(["embed-train", "-m", bert, "-d", str(data), "-o", out2, "--max-steps", "2", "--batch-size", "4", "--lora-r", "4",
                 "--device", "cpu"]) == 0
    assert os.path.exists(os.path.join(out2, "lora_weights.safetensors"))
