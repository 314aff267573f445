"""End-to-end parity of the native training step with the fp32 PyTorch path."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _build(dtype, device):
    from pmetal_b200.core.config import LoraConfig
    from pmetal_b200.lora import apply_lora
    from pmetal_b200.models.config import ModelArgs
    from pmetal_b200.models.decoder import DecoderLM
    cfg = ModelArgs(vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                    num_attention_heads=2, num_key_value_heads=1, head_dim=128)
    m = DecoderLM(cfg).init_weights(0.05, 0)
    apply_lora(m, LoraConfig(r=16, alpha=32, target_modules=["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj",
                                                             "up_proj", "down_proj"]), seed=1)
    with torch.no_grad():
        g = torch.Generator().manual_seed(2)
        for _, _, fl in m.fused_linears():
            fl.lora_b.copy_(torch.randn(fl.lora_b.shape, generator=g) * 0.05)
    m = m.to(device)
    for n, p in m.named_parameters():
        if "lora_" not in n:
            p.data = p.data.to(dtype)
    return m


def _batch(T, vocab, device):
    from pmetal_b200.data.dataloader import synthetic_documents
    from pmetal_b200.data.packing import PackerConfig, SequencePacker, collate_packs
    docs = synthetic_documents(12, 20, 300, vocab, seed=3)
    packs = SequencePacker(PackerConfig(max_length=T)).pack(docs)
    return collate_packs(packs[:1], T).to(device)


def test_model_loss_and_grads_match_reference():
    from pmetal_b200.ops import functional as F
    from pmetal_b200.ops import native
    assert native.available(), native.load_error()
    dev = torch.device("cuda")
    m = _build(torch.bfloat16, dev)
    m.prepare_for_training()
    ref = _build(torch.float32, dev)
    b = _batch(1024, 2048, dev)
    loss = m.loss(b.input_ids, b.labels, b.position_ids, b.cu_seqlens, b.seq_start)
    loss.backward()
    native.check_status()
    with F.force_reference():
        rl = ref.loss(b.input_ids, b.labels, b.position_ids, b.cu_seqlens, b.seq_start)
        rl.backward()
    assert abs(loss.item() - rl.item()) < 3e-2 * abs(rl.item()), (loss.item(), rl.item())
    worst = 0.0
    for (n, p), (_, q) in zip(m.named_parameters(), ref.named_parameters()):
        if p.grad is None:
            continue
        num = (p.grad.float() - q.grad.float()).norm().item()
        den = q.grad.float().norm().item() + 1e-8
        worst = max(worst, num / den)
        assert num / den < 8e-2, f"{n}: relative grad error {num / den:.4f}"
    print("worst relative grad error", worst)


def test_training_loop_reduces_loss():
    from pmetal_b200.core.config import TrainingConfig
    from pmetal_b200.ops import native
    from pmetal_b200.trainer.loop import TrainingLoop
    dev = torch.device("cuda")
    m = _build(torch.bfloat16, dev)
    m.prepare_for_training()
    loop = TrainingLoop(m, TrainingConfig(learning_rate=1e-3, gradient_accumulation_steps=1, warmup_steps=0,
                                          lr_scheduler="constant", max_grad_norm=1.0))
    b = _batch(1024, 2048, dev)
    losses = []
    for _ in range(8):
        loss, gn = loop.train_step(b)
        losses.append(float(loss))
    native.check_status()
    assert losses[-1] < losses[0], losses
