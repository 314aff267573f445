"""Embedding objectives, token shards, pre-training with checkpoint resume, MCP protocol, Python API (CPU)."""
import io
import json
import math
import os

import numpy as np
import pytest
import torch

from pmetal_b200.data.streaming import ShardWriter, TokenShardDataset
from pmetal_b200.trainer import embedding as E


def tiny(seed=0, vocab=97):
    from pmetal_b200.models.config import ModelArgs
    from pmetal_b200.models.decoder import DecoderLM
    cfg = ModelArgs(vocab_size=vocab, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                    num_attention_heads=2, num_key_value_heads=1, head_dim=16)
    return DecoderLM(cfg).init_weights(0.1, seed)


def test_contrastive_losses():
    a = torch.nn.functional.normalize(torch.tensor([[1.0, 0.0], [0.0, 1.0]]), dim=-1)
    assert float(E.info_nce(a, a, 0.05)) < 1e-6
    assert float(E.info_nce(a, a.flip(0), 0.05)) > 10
    assert float(E.triplet_loss(a, a, a.flip(0), 0.5)) == 0.0
    assert float(E.triplet_loss(a, a.flip(0), a, 0.5)) == pytest.approx(1.5)
    cos_ok = E.cosent_loss(a, torch.stack([a[1], a[1]]), torch.tensor([0.0, 1.0]))      # cos 0 (label 0) < cos 1 (label 1)
    cos_bad = E.cosent_loss(a, torch.stack([a[0], a[0]]), torch.tensor([0.0, 1.0]))     # order violated
    assert float(cos_ok) < float(cos_bad)
    h = torch.arange(12, dtype=torch.float32).reshape(6, 2)
    p = E.pool(h, [0, 2, 6], "mean", normalize=False)
    assert torch.allclose(p, torch.stack([h[:2].mean(0), h[2:].mean(0)]))
    assert torch.allclose(E.pool(h, [0, 2, 6], "last", False), torch.stack([h[1], h[5]]))


def test_embedding_trainer_improves():
    torch.manual_seed(0)
    tr = E.EmbeddingTrainer(tiny(1), E.EmbeddingConfig(learning_rate=1e-2, temperature=1.0))
    anchors = [[1, 2, 3], [40, 41, 42, 43], [1, 2, 5], [40, 41, 45]]
    positives = [[1, 2, 4], [40, 41, 44], [1, 2, 6], [40, 41, 46]]
    a = tr.step(anchors, positives)["loss"]
    for _ in range(10):
        b = tr.step(anchors, positives)["loss"]
    assert b < a
    e = tr.encode(anchors)
    assert e.shape == (4, 32) and torch.allclose(e.norm(dim=-1), torch.ones(4), atol=1e-5)


def test_token_shards(tmp_path):
    p = str(tmp_path / "s0.bin")
    with ShardWriter(p) as w:
        w.add_document(list(range(100)))
        w.add_document(list(range(100, 130)))
    assert os.path.getsize(p) == 130 * 4
    ds = TokenShardDataset(str(tmp_path / "*.bin"), 16, shuffle=False)
    wins = list(ds)
    assert len(wins) == 8 and wins[0].tolist() == list(range(16)) and ds.total_tokens() == 130
    assert ds.documents(0).tolist() == [0, 100, 130]
    r0 = [w[0] for w in TokenShardDataset(str(tmp_path / "*.bin"), 16, 0, 2, shuffle=True, seed=1)]
    r1 = [w[0] for w in TokenShardDataset(str(tmp_path / "*.bin"), 16, 1, 2, shuffle=True, seed=1)]
    assert sorted(r0 + r1) == [i * 16 for i in range(8)] and not set(r0) & set(r1)
    with pytest.raises(FileNotFoundError):
        TokenShardDataset(str(tmp_path / "none*.bin"), 16)


def test_pretrain_loss_falls_and_checkpoint_resumes(tmp_path):
    from pmetal_b200.ops.functional import linear_cross_entropy_z
    from pmetal_b200.trainer.pretrain import PretrainConfig, PretrainTrainer
    torch.manual_seed(0)
    cfg = PretrainConfig(learning_rate=5e-3, min_lr=5e-3, warmup_steps=0, max_steps=6, micro_batch=2, seq_len=16,
                         z_loss_coef=1e-3, lr_scheduler="constant")
    data = [np.arange(i, i + 16) % 97 for i in range(40)]
    tr = PretrainTrainer(tiny(2), cfg)
    first = tr.train_step(data[:2])
    last = tr.run(iter(data))
    assert last["loss"] < first["loss"] and last["z_loss"] > 0 and tr.step_count == 6
    tot, ce, z = linear_cross_entropy_z(torch.zeros(3, 4), torch.zeros(5, 4), torch.tensor([1, -100, 2]), 0.5)
    assert float(z) == pytest.approx(math.log(5) ** 2) and float(ce) == pytest.approx(math.log(5))
    assert float(tot) == pytest.approx(math.log(5) + 0.5 * math.log(5) ** 2)
    ck = str(tmp_path / "ck")
    tr.save_checkpoint(ck)
    tr2 = PretrainTrainer(tiny(3), cfg)
    tr2.load_checkpoint(ck)
    assert tr2.step_count == 6 and torch.allclose(tr2.opt.flat_p, tr.opt.flat_p) and torch.allclose(tr2.opt.flat_m, tr.opt.flat_m)
    a, b = tr.train_step(data[2:4]), tr2.train_step(data[2:4])
    assert a["loss"] == pytest.approx(b["loss"], rel=1e-5)


def test_mcp_protocol(tmp_path):
    from pmetal_b200.mcp import McpServer
    srv = McpServer()
    msgs = [{"jsonrpc": "2.0", "id": 1, "method": "initialize", "params": {}},
            {"jsonrpc": "2.0", "method": "notifications/initialized"},
            {"jsonrpc": "2.0", "id": 2, "method": "tools/list"},
            {"jsonrpc": "2.0", "id": 3, "method": "tools/call", "params": {"name": "set_learning_rate",
                                                                           "arguments": {"output_dir": str(tmp_path), "lr": 1e-5}}},
            {"jsonrpc": "2.0", "id": 4, "method": "tools/call", "params": {"name": "job_status", "arguments": {"id": "nope"}}},
            {"jsonrpc": "2.0", "id": 5, "method": "tools/call", "params": {"name": "infer", "arguments": {}}},
            {"jsonrpc": "2.0", "id": 6, "method": "bogus"}]
    fin = io.StringIO("\n".join(json.dumps(m) for m in msgs) + "\nnot json\n")
    fout = io.StringIO()
    srv.serve_stdio(fin, fout)
    out = [json.loads(l) for l in fout.getvalue().splitlines()]
    by_id = {o["id"]: o for o in out}
    assert by_id[1]["result"]["serverInfo"]["name"] == "pmetal-b200"
    names = {t["name"] for t in by_id[2]["result"]["tools"]}
    assert {"start_train", "start_grpo", "job_status", "infer", "set_learning_rate", "graceful_stop"} <= names and len(names) >= 20
    assert by_id[3]["result"]["isError"] is False
    assert json.load(open(tmp_path / ".lr_control.json")) == {"command": "set_lr", "lr": 1e-5}
    assert by_id[4]["result"]["isError"] is True and by_id[5]["result"]["isError"] is True
    assert by_id[6]["error"]["code"] == -32601 and by_id[None]["error"]["code"] == -32700
    # the reference server's tool names are all present, and the dataset tools run through the command line
    reference_names = {"device_info", "search_models", "download_model", "list_local_models", "model_fit", "memory",
                       "generate", "train", "pretrain", "distill", "grpo", "rlkd", "embed_train", "list_jobs", "job_status",
                       "job_logs", "stop_job", "run_cli", "start_cli_job", "dataset_analyze", "dataset_preview",
                       "dataset_validate", "dataset_download", "dataset_convert", "dataset_filter", "dataset_split",
                       "dataset_merge", "dataset_sample", "dataset_template", "dataset_prepare", "quantize", "fuse_lora",
                       "merge_models", "pack_experts", "eval_perplexity", "benchmark", "bench_train", "bench_gen",
                       "bench_corpus", "start_serve", "tokenize", "dflash", "ollama_create", "ollama_modelfile",
                       "job_set_lr", "job_reduce_lr", "job_reset_lr", "job_save_checkpoint", "job_graceful_stop",
                       "model_info", "chat"}
    assert reference_names <= names
    src = tmp_path / "d.jsonl"
    src.write_text("".join(json.dumps({"text": f"t{i}"}) + "\n" for i in range(10)))
    call = lambda name, args: srv.tools[name]["fn"](args)
    assert call("dataset_sample", {"input": str(src), "output": str(tmp_path / "o.jsonl"), "num": 3}) == {"sampled": 3}
    assert call("dataset_validate", {"path": str(src)})["valid"] == 10
    assert call("dataset_merge", {"inputs": [str(src), str(src)], "output": str(tmp_path / "m.jsonl")})["merged"] == 20
    assert "chatml" in call("run_cli", {"argv": ["dataset", "formats"]})["templates"]


def test_python_api_generate(tmp_path):
    import pmetal_b200 as pm
    from pmetal_b200.models.loader import save_pretrained
    d = str(tmp_path / "m")
    save_pretrained(tiny(4, vocab=300), d)
    m = pm.Model.load(d, device="cpu")
    text = m.generate("hello", max_tokens=4, temperature=0)
    assert isinstance(text, str)
    assert "".join(m.stream("hello", max_tokens=4, temperature=0)) == text


def test_masked_diffusion_lm_training_and_sampling():
    import math

    import torch

    from pmetal_b200.models.architectures.generic import GenericDecoderLM
    from pmetal_b200.trainer.diffusion import (BidirectionalLM, DiffusionConfig, DiffusionSampler, DiffusionTrainer,
                                               diffusion_loss, forward_process, noise_alpha)
    assert noise_alpha("linear", 0.25) == 0.75 and abs(noise_alpha("cosine", 1.0)) < 1e-6 and noise_alpha("polynomial2", 0.5) == 0.25
    g = torch.Generator().manual_seed(0)
    x0 = torch.randint(0, 50, (4, 200))
    xt, mask = forward_process(x0, 0.3, 63, g)
    assert 0.2 < mask.float().mean() < 0.4 and (xt[mask] == 63).all() and torch.equal(xt[~mask], x0[~mask])
    elig = torch.zeros_like(mask)
    elig[:, 100:] = True
    _, m2 = forward_process(x0, 0.9, 63, g, elig)
    assert not m2[:, :100].any() and m2[:, 100:].float().mean() > 0.8
    logits = torch.zeros(1, 3, 5)
    logits[0, 1, 2] = 10.0
    tg = torch.tensor([[0, 2, -100]])
    mk = torch.tensor([[True, True, True]])
    plain = diffusion_loss(logits, tg, mk, 0.5, use_elbo=False)
    assert abs(float(plain) - (math.log(5) + 0.0002) / 2) < 1e-2          # position 0 uniform, position 1 certain, 2 ignored
    assert abs(float(diffusion_loss(logits, tg, mk, 0.5, True)) - 2 * float(plain)) < 1e-5
    assert float(diffusion_loss(logits, tg, torch.zeros_like(mk), 0.5)) == 0.0
    torch.manual_seed(0)
    lm = GenericDecoderLM.from_hf_config(dict(model_type="llama", vocab_size=64, hidden_size=64, intermediate_size=96,
                                              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2)).init_weights(0.05, 0)
    model = BidirectionalLM(lm)
    ids = torch.randint(0, 60, (1, 12))
    a = model(ids)
    ids2 = ids.clone()
    ids2[0, -1] = (ids2[0, -1] + 1) % 60
    assert not torch.allclose(a[0, 0], model(ids2)[0, 0])                 # position 0 sees the last token: no causal mask
    assert torch.allclose(lm(ids)[0, 0], lm(ids2)[0, 0])                   # and the wrapper leaves the causal model intact
    cfg = DiffusionConfig(mask_token_id=63, num_inference_steps=6, use_elbo_loss=False)
    tr = DiffusionTrainer(model, cfg, lr=3e-3)
    data = torch.arange(16)[None].repeat(8, 1) % 60                         # one memorisable pattern
    losses = [tr.train_step(data)["loss"] for _ in range(60)]
    assert sum(losses[-5:]) / 5 < 0.6 * sum(losses[:5]) / 5
    ev = tr.evaluate([data])
    assert ev["perplexity"] < 30
    for strategy in ("low_confidence", "random", "semi_autoregressive"):
        cfg.remasking, cfg.block_size = strategy, 2
        out = DiffusionSampler(cfg).sample(model, list(range(6)), 8)
        assert len(out) == 8 and all(0 <= t < 64 for t in out) and 63 not in out
    cfg.remasking = "low_confidence"
    out = DiffusionSampler(cfg).sample(model, list(range(6)), 8)
    assert sum(int(t == 6 + i) for i, t in enumerate(out)) >= 4              # it continues the memorised pattern


def test_dflash_draft_training_step_learns():
    import torch

    from pmetal_b200.models.architectures.generic import GenericDecoderLM
    from pmetal_b200.models.dflash import DFlashConfig, DFlashDraftModel
    from pmetal_b200.trainer.diffusion import DFlashDraftTrainer, dflash_train_step
    torch.manual_seed(0)
    target = GenericDecoderLM.from_hf_config(dict(model_type="qwen3", vocab_size=64, hidden_size=64, intermediate_size=96,
                                                  num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                                                  head_dim=16)).init_weights(0.05, 1).eval()
    dc = DFlashConfig.from_dict(dict(hidden_size=64, num_hidden_layers=1, intermediate_size=96, num_attention_heads=4,
                                     num_key_value_heads=2, head_dim=16, vocab_size=64, block_size=4,
                                     dflash_config=dict(target_layer_ids=[0, 2], mask_token_id=63)))
    draft = DFlashDraftModel(dc)
    toks = (torch.arange(24)[None] * 3) % 60
    out = dflash_train_step(target, draft, toks, 10)
    assert out["block"] == (10, 4) and out["loss"].requires_grad and 3.0 < float(out["loss"].detach()) < 6.0
    assert all(p.grad is None for p in target.parameters())
    tr = DFlashDraftTrainer(target, draft, lr=3e-3)
    losses = [tr.train_step(toks)["loss"] for _ in range(120)]
    assert sum(losses[-10:]) < 0.8 * sum(losses[:10])


def test_python_api_exports_and_trainer_object(tmp_path):
    import pmetal_b200 as pm
    for name in ("LoraConfig", "TrainingConfig", "GenerationConfig", "DataLoaderConfig", "Dtype", "Quantization", "LoraBias",
                 "LrSchedulerType", "OptimizerType", "DatasetFormat", "ModelArchitecture", "download_model", "download_file",
                 "Model", "Tokenizer", "Trainer", "ProgressCallback", "LoggingCallback", "MetricsJsonCallback", "finetune", "infer"):
        assert getattr(pm, name) is not None and name in pm.__all__
    assert pm.LrSchedulerType.COSINE == "cosine" and str(pm.Quantization.NF4) == "nf4"
    assert pm.ModelArchitecture.from_config({"model_type": "qwen3_moe"}) is pm.ModelArchitecture.QWEN3_MOE
    assert pm.GenerationConfig(temperature=0.3, max_tokens=5).temperature == 0.3
    data = tmp_path / "d.jsonl"
    data.write_text("".join(json.dumps({"text": "the cat sat on the mat " * 4}) + "\n" for _ in range(8)))
    seen = []

    class Watch:                                                     # a plain object: only the methods it has are called
        def on_step_end_with_metrics(self, m):
            seen.append(m.step)
    tcfg = pm.TrainingConfig(learning_rate=1e-3, max_steps=2, gradient_accumulation_steps=1, warmup_steps=0)
    tr = pm.Trainer("random:tiny-qwen3", pm.LoraConfig(r=4, alpha=8.0), tcfg, str(data), output=str(tmp_path / "out"))
    tr.add_callback(Watch())
    tr.set_sequence_packing(True)
    tr.set_metal_fused_optimizer(False)
    tr.job.device, tr.job.dtype, tr.job.adaptive_lr = "cpu", "float32", False
    res = tr.train()
    assert seen == [1, 2] and os.path.exists(tmp_path / "out" / "lora_weights.safetensors") and "Trainer(" in repr(tr)
    assert isinstance(res, dict)


def test_token_stream_position_resumes_exactly(tmp_path):
    with ShardWriter(str(tmp_path / "s.bin")) as w:
        w.add_document(list(range(1000)))
    full = TokenShardDataset(str(tmp_path / "s.bin"), 10, seed=3, loop=True)
    it = iter(full)
    seq = [next(it)[0] for _ in range(250)]                              # 100 windows per epoch: runs into the third epoch
    assert full.state_dict()["epoch"] == 2 and sorted(seq[:100]) == sorted(seq[100:200]) and seq[:100] != seq[100:200]
    a = TokenShardDataset(str(tmp_path / "s.bin"), 10, seed=3, loop=True)
    ia = iter(a)
    head = [next(ia)[0] for _ in range(130)]
    b = TokenShardDataset(str(tmp_path / "s.bin"), 10, seed=3, loop=True)
    b.load_state_dict(a.state_dict())
    ib = iter(b)
    assert head + [next(ib)[0] for _ in range(120)] == seq
    with pytest.raises(ValueError):
        TokenShardDataset(str(tmp_path / "s.bin"), 20, seed=3).load_state_dict(a.state_dict())
    assert len(list(TokenShardDataset(str(tmp_path / "s.bin"), 10))) == 100       # single pass without loop
