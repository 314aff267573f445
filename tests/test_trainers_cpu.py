"""CPU tests of the preference / RL / distillation objectives and their trainers on a tiny model."""
import math

import pytest
import torch

from pmetal_b200.distill import losses as DL
from pmetal_b200.distill.offline import LogitCache, LogitCompressor
from pmetal_b200.distill.taid import TaidConfig, TaidDistiller
from pmetal_b200.trainer import gspo as G
from pmetal_b200.trainer import ppo as P
from pmetal_b200.trainer import preference as PR


def tiny(seed=0, vocab=97):
    from pmetal_b200.models.config import ModelArgs
    from pmetal_b200.models.decoder import DecoderLM
    cfg = ModelArgs(vocab_size=vocab, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                    num_attention_heads=2, num_key_value_heads=1, head_dim=16)
    return DecoderLM(cfg).init_weights(0.1, seed)


def test_dpo_family_losses():
    pw, pl = torch.tensor([-5.0, -4.0]), torch.tensor([-6.0, -3.0])
    rw, rl = torch.tensor([-5.5, -4.5]), torch.tensor([-5.5, -3.5])
    c = PR.PreferenceConfig(beta=0.5)
    loss, cw, cl = PR.dpo_loss(pw, pl, rw, rl, c)
    logits = 0.5 * ((pw - rw) - (pl - rl))
    assert torch.allclose(loss, torch.nn.functional.softplus(-logits).mean())
    assert torch.allclose(cw, 0.5 * (pw - rw))
    c.label_smoothing = 0.1
    ls, _, _ = PR.dpo_loss(pw, pl, rw, rl, c)
    want = (torch.nn.functional.softplus(-logits) * 0.9 + torch.nn.functional.softplus(logits) * 0.1).mean()
    assert torch.allclose(ls, want)
    for kind, fn in (("ipo", lambda x: (x - 1.0) ** 2), ("hinge", lambda x: torch.clamp(1 - x, min=0)),
                     ("robust", lambda x: torch.nn.functional.softplus(-x) + 0.5 * torch.clamp(0.5 - x, min=0))):
        l2, _, _ = PR.dpo_loss(pw, pl, rw, rl, PR.PreferenceConfig(beta=0.5, loss_type=kind))
        assert torch.allclose(l2, fn(logits).mean()), kind
    s, _, _ = PR.dpo_loss(pw, pl, None, None, PR.PreferenceConfig.simpo())
    assert torch.allclose(s, torch.nn.functional.softplus(-(2.5 * (pw - pl) - 0.5)).mean())
    total, sft, ratio = PR.orpo_loss(torch.tensor([-0.5]), torch.tensor([-1.5]), 0.1)
    lo = lambda x: x - math.log(1 - math.exp(x))       # noqa: E731
    assert abs(float(ratio) - math.log(1 + math.exp(-(lo(-0.5) - lo(-1.5))))) < 1e-5
    assert abs(float(total) - (0.5 + 0.1 * float(ratio))) < 1e-6
    k = PR.kto_loss(torch.tensor([1.0, -1.0]), torch.tensor([True, False]), 0.2, 0.1, 0.3, 1.0, 2.0)
    want = (torch.sigmoid(torch.tensor(0.2 - 0.1)) + 2 * torch.sigmoid(torch.tensor(-0.3 - 0.2))) / 2
    assert torch.allclose(k, want)


def test_preference_trainers_reduce_loss():
    torch.manual_seed(0)
    policy, ref = tiny(1), tiny(1)
    for p in ref.parameters():
        p.requires_grad_(False)
    pairs = [PR.PreferencePair([1, 2, 3], [10, 11, 12, 13], [20, 21]), PR.PreferencePair([4, 5], [30, 31], [40, 41, 42])]
    tr = PR.PreferenceTrainer(policy, PR.PreferenceConfig(beta=0.5, learning_rate=5e-3), ref)
    first = tr.step(pairs)
    for _ in range(15):
        last = tr.step(pairs)
    assert abs(first["loss"] - math.log(2)) < 1e-4         # policy == reference at the start
    assert last["loss"] < first["loss"] and last["reward_accuracy"] == 1.0
    for cfg in (PR.PreferenceConfig.simpo(learning_rate=5e-3), PR.PreferenceConfig.orpo(learning_rate=5e-3)):
        t2 = PR.PreferenceTrainer(tiny(2), cfg)
        a = t2.step(pairs)["loss"]
        for _ in range(10):
            b = t2.step(pairs)["loss"]
        assert b < a
    kt = PR.KtoTrainer(tiny(3), PR.KtoConfig(beta=0.5, learning_rate=5e-3), tiny(3))
    ex = [PR.KtoExample([1, 2], [5, 6, 7], True), PR.KtoExample([1, 2], [8, 9], False)]
    a = kt.step(ex)["loss"]
    for _ in range(10):
        b = kt.step(ex)["loss"]
    assert b < a


def test_online_dpo_builds_pairs_and_steps():
    torch.manual_seed(0)
    pol = tiny(4)
    tr = PR.OnlineDpoTrainer(pol, PR.PreferenceConfig(beta=0.1, learning_rate=1e-3),
                             reward_fn=lambda ps, cs: [float(sum(c) % 7) for c in cs], reference=None,
                             max_new_tokens=6, kv_blocks=64)
    out = tr.step_online([[1, 2, 3], [4, 5, 6, 7]])
    assert "loss" in out and out["pairs"] <= 2


def test_gae_and_ppo_losses():
    r = torch.tensor([0.0, 0.0, 1.0])
    v = torch.tensor([0.5, 0.4, 0.3])
    d = torch.tensor([0.0, 0.0, 1.0])
    adv, ret = P.compute_gae(r, v, d, gamma=0.9, lam=0.8)
    d2 = 1.0 - 0.3
    d1 = 0.9 * 0.3 - 0.4
    d0 = 0.9 * 0.4 - 0.5
    a2 = d2
    a1 = d1 + 0.9 * 0.8 * a2
    a0 = d0 + 0.9 * 0.8 * a1
    assert torch.allclose(adv, torch.tensor([a0, a1, a2]), atol=1e-6)
    assert torch.allclose(ret, adv + v)
    lp, old = torch.tensor([-1.0, -2.0]), torch.tensor([-1.5, -1.5])
    loss, ratio = P.ppo_policy_loss(lp, old, torch.tensor([1.0, -1.0]), 0.2)
    want = -(min(math.exp(0.5), 1.2) * 1.0 + min(-math.exp(-0.5), -0.8)) / 2
    assert abs(float(loss) - want) < 1e-6
    vl = P.ppo_value_loss(torch.tensor([1.0]), torch.tensor([0.0]), torch.tensor([2.0]), 0.2)
    assert abs(float(vl) - 0.5 * max(1.0, (0.2 - 2.0) ** 2)) < 1e-6
    k = P.AdaptiveKl(0.1, 1.0)
    assert k.update(2.0) == pytest.approx(0.15) and k.update(0.1) == pytest.approx(0.1)


def test_ppo_trainer_runs():
    torch.manual_seed(0)
    tr = P.PpoTrainer(tiny(5), P.PpoConfig(ppo_epochs=2, max_completion_length=5, learning_rate=1e-3),
                      reward_fn=lambda ps, cs: [1.0 if len(c) > 2 else 0.0 for c in cs], reference=tiny(5), kv_blocks=64)
    out = tr.step([[1, 2, 3], [4, 5]])
    assert math.isfinite(out["loss"]) and "value_loss" in out


def test_gspo_dapo_objectives_and_trainers():
    adv = G.gspo_advantages([1.0, 2.0, 6.0, 3.0], [1, 1, 1, 1], 4, G.GspoConfig(whiten=False, length_normalize_rewards=False))
    assert adv == [1.0 - 2.5, 2.0 - 2.5, 5.0 if 6.0 - 2.5 > 5 else 3.5, 0.5]
    adv = G.gspo_advantages([10.0, 0.0], [10, 1], 2, G.GspoConfig(whiten=False, baseline="mean"))
    assert adv == [0.5, -0.5]
    d = G.dapo_advantages([1.0, 0.0, 1.0, 0.0], 4)
    assert d == [1.0, -1.0, 1.0, -1.0]
    lp, old = torch.tensor([0.0, 0.0]), torch.tensor([-1.0, 1.0])
    l = G.dapo_token_loss(lp, old, torch.tensor([1.0, 1.0]), 0.0, 0.28)
    assert abs(float(l) + (1.28 + math.exp(-1)) / 2) < 1e-6
    loss, pol, kl = G.gspo_loss(torch.tensor([-1.0, -2.0, -3.0]), torch.tensor([1.0, 1.0, -1.0]), torch.tensor([0, 0, 1]), 2,
                                G.GspoConfig(token_weighting="sequence", beta=0.0))
    assert abs(float(pol) - ((1.0 + 2.0) / 2 - 3.0) / 2) < 1e-6
    torch.manual_seed(0)
    from pmetal_b200.trainer.grpo import GrpoConfig
    gc = GrpoConfig(num_generations=2, max_completion_length=4, learning_rate=1e-3, beta=0.0)
    tr = G.GspoTrainer(tiny(6), G.GspoConfig(num_generations=2, beta=0.0), lambda ps, cs: [float(len(c)) for c in cs],
                       grpo_cfg=gc, kv_blocks=64)
    assert math.isfinite(tr.step([[1, 2, 3]])["loss"])
    rk = G.RlkdTrainer(tiny(7), gc, lambda ps, cs: [float(sum(c) % 3) for c in cs], teacher=tiny(8), alpha=0.5, kv_blocks=64)
    out = rk.step([[1, 2, 3], [4, 5]])
    assert math.isfinite(out["loss"]) and out["kd_loss"] >= 0


def test_distill_losses_basic_properties():
    torch.manual_seed(0)
    s, t = torch.randn(3, 5, 50), torch.randn(3, 5, 50)
    for name, fn in DL.LOSSES.items():
        same = fn(t, t)
        diff = fn(s, t)
        assert float(same) <= 1e-5 + (0.7 if name == "logistic_ranking" else 0) or name == "soft_ce", name
        assert float(diff) > float(same) - 1e-6, name
    assert abs(float(DL.kl_divergence(s, t, 1.0)) -
               float((t.softmax(-1) * (t.log_softmax(-1) - s.log_softmax(-1))).sum(-1).mean())) < 1e-5
    js = DL.jensen_shannon(s, t, 1.0)
    assert 0 < float(js) <= math.log(2) + 1e-5
    assert abs(float(DL.gkd(s, t, 1.0, beta=0.0)) - float(DL.kl_divergence(s, t, 1.0))) < 1e-6
    mask = torch.zeros(3, 5, dtype=torch.bool)
    mask[0, 0] = True
    one = DL.kl_divergence(s[:1, :1], t[:1, :1], 2.0)
    assert abs(float(DL.kl_divergence(s, t, 2.0, mask)) - float(one)) < 1e-6
    assert float(DL.universal_logit(torch.randn(2, 30), torch.randn(2, 40))) > 0
    assert float(DL.hidden_state_loss(torch.ones(2, 4), torch.ones(2, 4), "cosine")) < 1e-6
    h = DL.hidden_state_loss(torch.ones(2, 3), torch.ones(2, 4), "mse", proj=torch.ones(4, 3) / 3)
    assert float(h) < 1e-10
    # the fused entry point falls back to the dense formulas on CPU and agrees with them
    hs, ht = torch.randn(7, 16), torch.randn(7, 16)
    ws, wt = torch.randn(50, 16), torch.randn(50, 16)
    f = DL.fused_kd_loss(hs, ws, ht, wt, None, 2.0, "kl")
    assert abs(float(f) - float(DL.kl_divergence(hs @ ws.t(), ht @ wt.t(), 2.0))) < 1e-5


def test_taid_schedule_and_loss():
    t = TaidDistiller(TaidConfig(initial_alpha=0.9, final_alpha=0.5, schedule="linear"))
    assert t.base_alpha(0, 100) == pytest.approx(0.9) and t.base_alpha(100, 100) == pytest.approx(0.5)
    assert TaidDistiller(TaidConfig(schedule="cosine")).base_alpha(50, 100) == pytest.approx(0.7)
    assert TaidDistiller(TaidConfig(schedule="step")).base_alpha(30, 100) == pytest.approx(0.9 - 0.4 * 0.33)
    torch.manual_seed(0)
    tl, sl = torch.randn(2, 4, 30), torch.randn(2, 4, 30, requires_grad=True)
    loss, a = t.loss(tl, sl, 10, 100)
    loss.backward()
    assert float(loss.detach()) > 0 and 0.1 <= a <= 0.99 and sl.grad.abs().sum() > 0
    easy, _ = t.loss(tl, tl.clone(), 10, 100)
    assert float(easy) < 1e-5


def test_logit_cache_round_trip(tmp_path):
    torch.manual_seed(0)
    x = torch.randn(6, 200) * 3
    for method, tol in (("full", 0), ("int8", 0.06), ("int4", 1.0), ("int8_per_token", 0.06)):
        y = LogitCompressor.decompress(LogitCompressor(method).compress(x))
        assert y.shape == x.shape and float((y - x).abs().max()) <= tol + 1e-6, method
    y = LogitCompressor.decompress(LogitCompressor("topk", 20).compress(x))
    assert torch.allclose(y.softmax(-1).sum(-1), torch.ones(6), atol=1e-4)
    top = x.topk(20, -1)
    assert torch.allclose(y.gather(-1, top.indices), top.values)
    assert torch.allclose(y.softmax(-1).gather(-1, top.indices), x.softmax(-1).gather(-1, top.indices), atol=1e-5)
    c = LogitCache(str(tmp_path / "cache"), "topk", 16)
    c.cache_sequence(0, x)
    c.save_metadata()
    c2 = LogitCache.load(str(tmp_path / "cache"))
    assert c2.has_sequence(0) and not c2.has_sequence(1) and c2.meta.vocab_size == 200
    assert c2.load_sequence(0).shape == x.shape and c2.stats(0)["compressed_bytes"] > 0


def test_distill_trainer_online_offline_progressive(tmp_path):
    from pmetal_b200.distill.trainer import DistillConfig, DistillTrainer
    torch.manual_seed(0)
    student, teacher = tiny(10), tiny(11)
    for p in teacher.parameters():
        p.requires_grad_(False)
    ids = torch.randint(0, 97, (24,))
    tr = DistillTrainer(student, teacher, DistillConfig(learning_rate=5e-3, loss_type="kl", alpha=1.0))
    a = tr.step(ids, ids.clone())
    for _ in range(12):
        b = tr.step(ids, ids.clone())
    assert b["soft"] < a["soft"]
    cache = tr.build_cache([ids.tolist()], str(tmp_path / "lc"), "topk", 32)
    assert cache.has_sequence(0)
    off = DistillTrainer(tiny(12), teacher, DistillConfig(method="offline", cache_dir=str(tmp_path / "lc"), learning_rate=1e-3))
    assert math.isfinite(off.step(ids, ids.clone(), seq_id=0)["loss"])
    prog = DistillTrainer(tiny(13), teacher, DistillConfig(method="progressive", total_steps=4, temperature=4.0,
                                                           final_temperature=1.0, loss_type="js"))
    temps = [prog.step(ids, ids.clone())["temperature"] for _ in range(5)]
    assert temps[0] == 4.0 and temps[-1] == 1.0
    td = DistillTrainer(tiny(14), teacher, DistillConfig(loss_type="taid", total_steps=10))
    assert "taid_alpha" in td.step(ids, ids.clone())


def test_preference_trainers_on_a_config_driven_architecture():
    """DPO with a frozen reference copy, SimPO and KTO drive a Gemma-style model through the padded log-probability path."""
    from pmetal_b200.models.architectures.generic import GenericDecoderLM, arch_config_from_hf

    def gemma(seed):
        cfg = dict(model_type="gemma2", vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                   num_attention_heads=4, num_key_value_heads=2, head_dim=8, max_position_embeddings=64,
                   final_logit_softcapping=30.0)
        torch.manual_seed(seed)
        m = GenericDecoderLM(arch_config_from_hf(cfg)).init_weights(0.2, seed)
        for p in m.parameters():
            p.requires_grad_(True)
        return m

    policy, ref = gemma(1), gemma(1)
    for p in ref.parameters():
        p.requires_grad_(False)
    pairs = [PR.PreferencePair([1, 2, 3], [10, 11, 12, 13], [20, 21]), PR.PreferencePair([4, 5], [30, 31], [40, 41, 42])]
    tr = PR.PreferenceTrainer(policy, PR.PreferenceConfig(beta=0.5, learning_rate=5e-3), ref)
    first = tr.step(pairs)
    for _ in range(15):
        last = tr.step(pairs)
    assert abs(first["loss"] - math.log(2)) < 1e-4 and last["loss"] < first["loss"] and last["reward_accuracy"] == 1.0
    t2 = PR.PreferenceTrainer(gemma(2), PR.PreferenceConfig.simpo(learning_rate=5e-3))
    a = t2.step(pairs)["loss"]
    for _ in range(10):
        b = t2.step(pairs)["loss"]
    assert b < a
    kt = PR.KtoTrainer(gemma(3), PR.KtoConfig(beta=0.5, learning_rate=5e-3), gemma(3))
    ex = [PR.KtoExample([1, 2], [5, 6, 7], True), PR.KtoExample([1, 2], [8, 9], False)]
    a = kt.step(ex)["loss"]
    for _ in range(10):
        b = kt.step(ex)["loss"]
    assert b < a
