"""BigVGAN vocoder: activation formulas, anti-aliasing filters, generator / discriminator shapes, mel features, losses."""
import math

import torch

from pmetal_b200 import vocoder as V


def _tiny():
    return V.BigVGANConfig(num_mels=20, upsample_rates=[4, 2], upsample_kernel_sizes=[8, 4], upsample_initial_channel=16,
                           resblock_kernel_sizes=[3, 7], resblock_dilation_sizes=[[1, 3], [1, 3]], sampling_rate=8000,
                           n_fft=128, hop_size=8, win_size=128, fmax=4000)


def test_snake_and_filter():
    x = torch.linspace(-2, 2, 11)[None, None].repeat(1, 3, 1)
    s = V.Snake(3, logscale=True, beta=True)
    with torch.no_grad():
        s.alpha.copy_(torch.tensor([0.0, math.log(2.0), 0.0]))
        s.beta.copy_(torch.tensor([0.0, 0.0, math.log(4.0)]))
    y = s(x)
    assert torch.allclose(y[0, 0], x[0, 0] + torch.sin(x[0, 0]) ** 2, atol=1e-6)
    assert torch.allclose(y[0, 1], x[0, 1] + torch.sin(2 * x[0, 1]) ** 2, atol=1e-6)
    assert torch.allclose(y[0, 2], x[0, 2] + torch.sin(x[0, 2]) ** 2 / 4, atol=1e-6)
    f = V.kaiser_sinc_filter(0.25, 0.3, 12)
    assert abs(float(f.sum()) - 1) < 1e-6 and torch.allclose(f, f.flip(0), atol=1e-7)
    # identity activation between the resamplers: a slow sine comes back almost unchanged, length preserved
    aa = V.AntiAliasedActivation(torch.nn.Identity())
    t = torch.arange(256).float()
    sig = torch.sin(2 * math.pi * t / 64)[None, None]
    out = aa(sig)
    assert out.shape == sig.shape and (out - sig)[..., 16:-16].abs().max() < 0.02


def test_generator_and_discriminators():
    torch.manual_seed(0)
    cfg = _tiny()
    g = V.BigVGAN(cfg)
    mel = torch.randn(2, 20, 12)
    wav = g(mel)
    assert wav.shape == (2, 1, 12 * cfg.total_upsample) and wav.abs().max() <= 1
    names = set(g.state_dict())
    assert {"conv_pre.weight", "ups.0.0.weight", "resblocks.0.convs1.1.weight", "resblocks.3.activations.2.act.alpha",
            "activation_post.act.beta", "conv_post.weight"} <= names
    assert V.BigVGANConfig.v2_24khz_100band().total_upsample == 256 == V.BigVGANConfig().hop_size
    mpd = V.MultiPeriodDiscriminator((2, 3), channels=(4, 8))
    mrd = V.MultiResolutionDiscriminator(((64, 16, 64), (32, 8, 32)), channels=4)
    for d in (mpd, mrd):
        outs = d(wav)
        assert len(outs) == 2 and all(o.dim() == 2 and len(f) >= 3 for o, f in outs)


def test_mel_features_and_losses():
    assert abs(V.hz_to_mel(1000.0) - 15.0) < 1e-6 and abs(V.mel_to_hz(V.hz_to_mel(4321.0)) - 4321.0) < 1e-2
    assert abs(V.hz_to_mel(700.0, htk=True) - 2595 * math.log10(2)) < 1e-4
    fb = V.mel_filterbank(8000, 128, 20, 0, 4000)
    assert fb.shape == (20, 65) and (fb >= 0).all() and (fb.sum(1) > 0).all()
    cfg = _tiny()
    t = torch.arange(800).float()
    tone = torch.sin(2 * math.pi * 1000 * t / 8000)[None]
    mel = V.mel_spectrogram(tone, cfg)
    assert mel.shape == (1, 20, 800 // 8)
    peak = int(mel[0, :, 20].argmax())
    centre = V.mel_to_hz(V.hz_to_mel(0) + (V.hz_to_mel(4000) - V.hz_to_mel(0)) * (peak + 1) / 21)
    assert abs(centre - 1000) < 250                                    # the tone lands in the band near 1 kHz
    ones = [(torch.ones(2, 3), [torch.ones(2, 3)])]
    zeros = [(torch.zeros(2, 3), [torch.zeros(2, 3)])]
    assert float(V.generator_adversarial_loss(ones)) == 0 and float(V.generator_adversarial_loss(zeros)) == 1
    assert float(V.discriminator_adversarial_loss(ones, zeros)) == 0 and float(V.discriminator_adversarial_loss(zeros, ones)) == 2
    assert float(V.feature_matching_loss(ones, zeros)) == 2.0
    assert float(V.mel_reconstruction_loss(tone, tone, cfg)) == 0
    assert float(V.multi_scale_mel_loss(tone, tone * 0.5, cfg)) > 0


def test_adversarial_training_step_runs_and_mel_loss_falls():
    torch.manual_seed(0)
    cfg = _tiny()
    g = V.BigVGAN(cfg)
    ds = [V.MultiPeriodDiscriminator((2, 3), channels=(4, 8)), V.MultiResolutionDiscriminator(((64, 16, 64),), channels=4)]
    og = torch.optim.AdamW(g.parameters(), 2e-3)
    od = torch.optim.AdamW([p for d in ds for p in d.parameters()], 2e-3)
    t = torch.arange(96 * 8).float()
    real = (0.5 * torch.sin(2 * math.pi * 440 * t / 8000))[None, None]
    mel = V.mel_spectrogram(real[:, 0], cfg)
    first = last = None
    for step in range(12):
        fake = g(mel)
        od.zero_grad()
        V.discriminator_loss(real, fake, ds).backward()
        od.step()
        og.zero_grad()
        loss, parts = V.generator_loss(real, g(mel), ds, cfg)
        loss.backward()
        og.step()
        first = parts["mel"] if first is None else first
        last = parts["mel"]
    assert last < first
