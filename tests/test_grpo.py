import math

import pytest

import torch

from pmetal_b200.core.config import LoraConfig
from pmetal_b200.lora import apply_lora
from pmetal_b200.models.config import preset
from pmetal_b200.models.decoder import DecoderLM
from pmetal_b200.trainer.grpo import GrpoConfig, GrpoTrainer, group_advantages, grpo_loss, mod7_length_reward


def test_group_advantages_sample_std_and_floor():
    adv = group_advantages([1.0, 2.0, 3.0, 5.0, 5.0, 5.0], 2, True)
    assert abs(adv[0] + 1.0) < 1e-9 and abs(adv[2] - 1.0) < 1e-9      # sample std of (1,2,3) is 1
    assert adv[3:] == [0.0, 0.0, 0.0]                                    # zero variance -> floor, numerator 0
    raw = group_advantages([1.0, 3.0], 1, False)
    assert raw == [-1.0, 1.0]


def test_grpo_loss_forms():
    cfg = GrpoConfig(beta=0.5)
    lp = torch.log(torch.tensor([0.5, 0.25, 0.5]))
    old = torch.log(torch.tensor([0.25, 0.25, 0.5]))
    ref = torch.log(torch.tensor([0.5, 0.5, 0.5]))
    adv = torch.tensor([1.0, 1.0, -1.0])
    mask = torch.ones(3)
    seq = torch.tensor([0, 0, 1])
    loss, kl, pol = grpo_loss(lp, old, ref, adv, mask, seq, 2, cfg)
    # ratios 2 (clipped to 1.2), 1, 1 -> token losses -1.2, -1, +1
    assert abs(pol.item() - (-1.2 - 1.0 + 1.0) / 3) < 1e-6
    r = math.log(0.5 / 0.25)
    assert abs(kl.item() - (math.exp(r) - 1 - r) / 3) < 1e-6
    assert abs(loss.item() - (pol.item() + 0.5 * kl.item())) < 1e-6
    cfg2 = GrpoConfig(beta=0.0, loss_type="dr_grpo")
    _, _, pol2 = grpo_loss(lp, old, None, adv, mask, seq, 2, cfg2)
    assert abs(pol2.item() - ((-1.2 - 1.0) / 2 + 1.0) / 2) < 1e-6


def test_grpo_step_runs_and_updates_policy():
    torch.manual_seed(0)
    m = DecoderLM(preset("tiny-qwen3")).init_weights(0.05, 0)
    apply_lora(m, LoraConfig(r=4, alpha=8))
    with torch.no_grad():
        for _, _, fl in m.fused_linears():
            if fl.lora_b is not None:
                fl.lora_b.normal_(0, 0.02)
    ref = DecoderLM(preset("tiny-qwen3")).init_weights(0.05, 0).eval()
    cfg = GrpoConfig(num_generations=4, max_completion_length=12, beta=0.04, learning_rate=1e-3, top_k=0, top_p=1.0)
    tr = GrpoTrainer(m, cfg, mod7_length_reward, reference=ref, kv_blocks=64)
    before = tr.opt.flat_p.clone()
    prompts = [torch.randint(0, 1024, (10,)).tolist() for _ in range(3)]
    st = tr.step(prompts)
    assert st.completion_tokens == 3 * 4 * 12 and math.isfinite(st.loss)
    assert not torch.equal(before, tr.opt.flat_p)
    assert tr.gen.cache.num_free() == 64
    st2 = GrpoTrainer(m, GrpoConfig.dapo(num_generations=4, max_completion_length=6), mod7_length_reward,
                      kv_blocks=64, optimizer=tr.opt).step(prompts)
    assert st2.skipped_groups >= 0


def test_model_reward_strategies_batching_and_families():
    """Packed scoring of several sequences equals scoring them one by one; score head and mean-logit strategies, last
    token and mean pooling, truncation, and a config-driven scorer."""
    from pmetal_b200.trainer.rewards import ModelReward, RewardModelConfig
    torch.manual_seed(0)
    m = DecoderLM(preset("tiny-qwen3")).init_weights(0.05, 0).eval()
    head = torch.randn(m.cfg.hidden_size)
    prompts = [torch.randint(0, 1024, (n,)).tolist() for n in (5, 9, 3, 7)]
    comps = [torch.randint(0, 1024, (n,)).tolist() for n in (4, 2, 6, 1)]
    for cfg in (RewardModelConfig(batch_size=3), RewardModelConfig(use_last_token=False, batch_size=2)):
        packed = ModelReward(m, head, cfg)(prompts, comps)
        single = [ModelReward(m, head, RewardModelConfig(use_last_token=cfg.use_last_token, batch_size=1))([p], [c])[0]
                  for p, c in zip(prompts, comps)]
        assert all(abs(a - b) < 1e-4 for a, b in zip(packed, single))
    r = ModelReward(m)
    assert r.strategy == "mean_logits" and len(r(prompts, comps)) == 4
    cut = ModelReward(m, head, RewardModelConfig(max_length=6))(prompts[:1], comps[:1])[0]
    want = ModelReward(m, head)([prompts[0][:5]], [comps[0][:1]])[0]
    assert abs(cut - want) < 1e-4
    from pmetal_b200.models.architectures.generic import GenericDecoderLM, arch_config_from_hf
    g = GenericDecoderLM(arch_config_from_hf(dict(model_type="gemma2", vocab_size=1024, hidden_size=32, intermediate_size=64,
                                                  num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=2, head_dim=8,
                                                  max_position_embeddings=64))).init_weights(0.1, 0).eval()
    vals = ModelReward(g, torch.randn(32))(prompts, comps)
    assert len(vals) == 4 and all(math.isfinite(v) for v in vals)
    with pytest.raises(ValueError):
        ModelReward(m, head, RewardModelConfig(template="{prompt} => {completion}"))
