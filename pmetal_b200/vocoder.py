"""BigVGAN neural vocoder: mel spectrogram -> waveform generator, the period / resolution discriminators used to train
it, mel utilities and the GAN losses (crates/pmetal-vocoder/src/{generator/mod,nn/amp_block,nn/activation,
discriminator/mpd,discriminator/mrd,audio/mel,audio/stft,loss/mod}.rs).

Generator: ``conv_pre`` lifts the mel bands to ``upsample_initial_channel``; every stage is a transposed convolution
(stride = upsample rate, channels halve) followed by the mean of three anti-aliased multi-periodicity (AMP) residual
blocks with kernel sizes (3, 7, 11) and dilations (1, 3, 5); a final periodic activation, ``conv_post`` and ``tanh``.
The periodic activation is Snake, x + sin^2(alpha x) / alpha, or SnakeBeta with a separate magnitude 1 / beta, with
log-scale parameters; it is applied at twice the sample rate between a Kaiser-windowed sinc up-sampler and
down-sampler so that the harmonics it creates do not alias."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class BigVGANConfig:
    num_mels: int = 100
    upsample_rates: List[int] = field(default_factory=lambda: [4, 4, 2, 2, 2, 2])
    upsample_kernel_sizes: List[int] = field(default_factory=lambda: [8, 8, 4, 4, 4, 4])
    upsample_initial_channel: int = 1536
    resblock_kernel_sizes: List[int] = field(default_factory=lambda: [3, 7, 11])
    resblock_dilation_sizes: List[List[int]] = field(default_factory=lambda: [[1, 3, 5]] * 3)
    activation: str = "snakebeta"
    snake_logscale: bool = True
    sampling_rate: int = 24000
    n_fft: int = 1024
    hop_size: int = 256
    win_size: int = 1024
    fmin: int = 0
    fmax: int = 12000

    @classmethod
    def v2_24khz_100band(cls) -> "BigVGANConfig":
        return cls()

    @classmethod
    def v2_44khz_128band(cls) -> "BigVGANConfig":
        return cls(num_mels=128, upsample_rates=[4, 4, 2, 2, 2, 2], sampling_rate=44100, n_fft=2048, hop_size=512,
                   win_size=2048, fmax=22050)

    @property
    def total_upsample(self) -> int:
        return math.prod(self.upsample_rates)


# ------------------------------------------------------------------------------------------------ activations
class Snake(nn.Module):
    def __init__(self, channels: int, logscale: bool = True, beta: bool = False):
        super().__init__()
        init = torch.zeros(channels) if logscale else torch.ones(channels)
        self.alpha = nn.Parameter(init.clone())
        if beta:
            self.beta = nn.Parameter(init.clone())
        self.logscale, self.has_beta = logscale, beta

    def forward(self, x):                                   # x [B, C, T]
        a = self.alpha[None, :, None]
        b = self.beta[None, :, None] if self.has_beta else a
        if self.logscale:
            a, b = torch.exp(a), torch.exp(b)
        return x + torch.sin(x * a).pow(2) / (b + 1e-9)


def kaiser_sinc_filter(cutoff: float, half_width: float, kernel_size: int) -> torch.Tensor:
    """Low-pass FIR prototype: Kaiser window (attenuation from the transition width) times a sinc, unit DC gain."""
    half = kernel_size // 2
    delta_f = 4 * half_width
    A = 2.285 * (half - 1) * math.pi * delta_f + 7.95
    beta = 0.1102 * (A - 8.7) if A > 50 else (0.5842 * (A - 21) ** 0.4 + 0.07886 * (A - 21) if A >= 21 else 0.0)
    window = torch.kaiser_window(kernel_size, beta=beta, periodic=False, dtype=torch.float64)
    t = torch.arange(-half, half, dtype=torch.float64) + 0.5 if kernel_size % 2 == 0 else torch.arange(kernel_size, dtype=torch.float64) - half
    filt = 2 * cutoff * window * torch.sinc(2 * cutoff * t)
    return (filt / filt.sum()).float()


class AntiAliasedActivation(nn.Module):
    """Up-sample x2 -> activation -> down-sample x2 with Kaiser-sinc filters (12 taps, as the published models)."""

    def __init__(self, act: nn.Module, ratio: int = 2, kernel_size: int = 12):
        super().__init__()
        self.act, self.ratio, self.k = act, ratio, kernel_size
        filt = kaiser_sinc_filter(0.5 / ratio, 0.6 / ratio, kernel_size)
        self.register_buffer("filter", filt[None, None], persistent=False)

    def _up(self, x):
        B, C, T = x.shape
        r, k = self.ratio, self.k
        pad = k // r - 1
        x = F.pad(x, (pad, pad), mode="replicate")
        y = r * F.conv_transpose1d(x, self.filter.expand(C, 1, k), stride=r, groups=C)
        left = pad * r + (k - r) // 2
        right = pad * r + (k - r + 1) // 2
        return y[..., left:y.shape[-1] - right]

    def _down(self, x):
        C, r, k = x.shape[1], self.ratio, self.k
        x = F.pad(x, (k // 2 - int(k % 2 == 0), k // 2), mode="replicate")
        return F.conv1d(x, self.filter.expand(C, 1, k), stride=r, groups=C)

    def forward(self, x):
        return self._down(self.act(self._up(x)))


def _pad(k: int, d: int) -> int:
    return (k * d - d) // 2


class AMPBlock(nn.Module):
    def __init__(self, channels: int, kernel: int, dilations: Sequence[int], cfg: BigVGANConfig):
        super().__init__()
        self.convs1 = nn.ModuleList([nn.Conv1d(channels, channels, kernel, dilation=d, padding=_pad(kernel, d)) for d in dilations])
        self.convs2 = nn.ModuleList([nn.Conv1d(channels, channels, kernel, padding=_pad(kernel, 1)) for _ in dilations])
        beta = cfg.activation == "snakebeta"
        self.activations = nn.ModuleList([AntiAliasedActivation(Snake(channels, cfg.snake_logscale, beta))
                                          for _ in range(2 * len(dilations))])

    def forward(self, x):
        for i, (c1, c2) in enumerate(zip(self.convs1, self.convs2)):
            x = x + c2(self.activations[2 * i + 1](c1(self.activations[2 * i](x))))
        return x


class BigVGAN(nn.Module):
    def __init__(self, cfg: Optional[BigVGANConfig] = None):
        super().__init__()
        self.cfg = cfg = cfg or BigVGANConfig()
        ch = cfg.upsample_initial_channel
        self.conv_pre = nn.Conv1d(cfg.num_mels, ch, 7, padding=3)
        self.ups = nn.ModuleList()
        self.resblocks = nn.ModuleList()
        for i, (r, k) in enumerate(zip(cfg.upsample_rates, cfg.upsample_kernel_sizes)):
            out = ch // 2
            self.ups.append(nn.ModuleList([nn.ConvTranspose1d(ch, out, k, r, padding=(k - r) // 2)]))
            for ks, ds in zip(cfg.resblock_kernel_sizes, cfg.resblock_dilation_sizes):
                self.resblocks.append(AMPBlock(out, ks, ds, cfg))
            ch = out
        self.activation_post = AntiAliasedActivation(Snake(ch, cfg.snake_logscale, cfg.activation == "snakebeta"))
        self.conv_post = nn.Conv1d(ch, 1, 7, padding=3, bias=False)

    def forward(self, mel: torch.Tensor) -> torch.Tensor:
        """mel [B, num_mels, frames] -> waveform [B, 1, frames * prod(upsample_rates)] in [-1, 1]."""
        x = self.conv_pre(mel)
        nk = len(self.cfg.resblock_kernel_sizes)
        for i, up in enumerate(self.ups):
            x = up[0](x)
            x = sum(self.resblocks[i * nk + j](x) for j in range(nk)) / nk
        return torch.tanh(self.conv_post(self.activation_post(x)))

    @torch.no_grad()
    def generate(self, mel: torch.Tensor) -> torch.Tensor:
        return self.forward(mel)[:, 0]


# ------------------------------------------------------------------------------------------------ mel features
def hz_to_mel(f: float, htk: bool = False) -> float:
    if htk:
        return 2595.0 * math.log10(1.0 + f / 700.0)
    f_sp, min_log_hz = 200.0 / 3, 1000.0
    min_log_mel, logstep = min_log_hz / f_sp, math.log(6.4) / 27.0
    return min_log_mel + math.log(f / min_log_hz) / logstep if f >= min_log_hz else f / f_sp


def mel_to_hz(m: float, htk: bool = False) -> float:
    if htk:
        return 700.0 * (10.0 ** (m / 2595.0) - 1.0)
    f_sp, min_log_hz = 200.0 / 3, 1000.0
    min_log_mel, logstep = min_log_hz / f_sp, math.log(6.4) / 27.0
    return min_log_hz * math.exp(logstep * (m - min_log_mel)) if m >= min_log_mel else f_sp * m


def mel_filterbank(sr: int, n_fft: int, n_mels: int, fmin: float, fmax: float, htk: bool = False) -> torch.Tensor:
    """[n_mels, n_fft / 2 + 1] triangular filters with Slaney area normalisation."""
    freqs = torch.linspace(0, sr / 2, n_fft // 2 + 1)
    lo, hi = hz_to_mel(fmin, htk), hz_to_mel(fmax, htk)
    pts = torch.tensor([mel_to_hz(lo + (hi - lo) * i / (n_mels + 1), htk) for i in range(n_mels + 2)])
    fb = torch.zeros(n_mels, freqs.numel())
    for i in range(n_mels):
        l, c, r = pts[i], pts[i + 1], pts[i + 2]
        fb[i] = torch.clamp(torch.minimum((freqs - l) / (c - l), (r - freqs) / (r - c)), min=0) * (2.0 / (r - l))
    return fb


def mel_spectrogram(audio: torch.Tensor, cfg: BigVGANConfig, n_fft=None, hop=None, win=None, n_mels=None) -> torch.Tensor:
    """audio [B, T] -> log-compressed mel [B, n_mels, frames] (reflect padding, Hann window, magnitude, log clamp 1e-5)."""
    n_fft, hop, win = n_fft or cfg.n_fft, hop or cfg.hop_size, win or cfg.win_size
    n_mels = n_mels or cfg.num_mels
    pad = (n_fft - hop) // 2
    x = F.pad(audio[:, None], (pad, pad), mode="reflect")[:, 0]
    spec = torch.stft(x, n_fft, hop, win, torch.hann_window(win, device=audio.device), center=False, return_complex=True)
    mag = torch.sqrt(spec.real.pow(2) + spec.imag.pow(2) + 1e-9)
    fb = mel_filterbank(cfg.sampling_rate, n_fft, n_mels, cfg.fmin, min(cfg.fmax, cfg.sampling_rate // 2)).to(audio.device)
    return torch.log(torch.clamp(fb @ mag, min=1e-5))


# ------------------------------------------------------------------------------------------------ discriminators
class PeriodDiscriminator(nn.Module):
    def __init__(self, period: int, channels: Sequence[int] = (32, 128, 512, 1024, 1024)):
        super().__init__()
        self.period = period
        convs, cin = [], 1
        for i, c in enumerate(channels):
            convs.append(nn.Conv2d(cin, c, (5, 1), (3 if i < len(channels) - 1 else 1, 1), padding=(2, 0)))
            cin = c
        self.convs = nn.ModuleList(convs)
        self.conv_post = nn.Conv2d(cin, 1, (3, 1), 1, padding=(1, 0))

    def forward(self, x) -> Tuple[torch.Tensor, List[torch.Tensor]]:          # x [B, 1, T]
        B, C, T = x.shape
        if T % self.period:
            x = F.pad(x, (0, self.period - T % self.period), mode="reflect")
        x = x.view(B, C, -1, self.period)
        feats = []
        for conv in self.convs:
            x = F.leaky_relu(conv(x), 0.1)
            feats.append(x)
        x = self.conv_post(x)
        feats.append(x)
        return x.flatten(1), feats


class MultiPeriodDiscriminator(nn.Module):
    def __init__(self, periods: Sequence[int] = (2, 3, 5, 7, 11), channels: Sequence[int] = (32, 128, 512, 1024, 1024)):
        super().__init__()
        self.discriminators = nn.ModuleList([PeriodDiscriminator(p, channels) for p in periods])

    def forward(self, x):
        return [d(x) for d in self.discriminators]


class ResolutionDiscriminator(nn.Module):
    def __init__(self, n_fft: int, hop: int, win: int, channels: int = 32):
        super().__init__()
        self.res = (n_fft, hop, win)
        self.convs = nn.ModuleList([nn.Conv2d(1, channels, (3, 9), padding=(1, 4)),
                                    nn.Conv2d(channels, channels, (3, 9), (1, 2), padding=(1, 4)),
                                    nn.Conv2d(channels, channels, (3, 9), (1, 2), padding=(1, 4)),
                                    nn.Conv2d(channels, channels, (3, 9), (1, 2), padding=(1, 4)),
                                    nn.Conv2d(channels, channels, (3, 3), padding=(1, 1))])
        self.conv_post = nn.Conv2d(channels, 1, (3, 3), padding=(1, 1))

    def forward(self, x):
        n_fft, hop, win = self.res
        pad = (n_fft - hop) // 2
        a = F.pad(x, (pad, pad), mode="reflect")[:, 0]
        spec = torch.stft(a, n_fft, hop, win, torch.hann_window(win, device=x.device), center=False, return_complex=True)
        h = torch.sqrt(spec.real.pow(2) + spec.imag.pow(2) + 1e-9)[:, None]
        feats = []
        for conv in self.convs:
            h = F.leaky_relu(conv(h), 0.1)
            feats.append(h)
        h = self.conv_post(h)
        feats.append(h)
        return h.flatten(1), feats


class MultiResolutionDiscriminator(nn.Module):
    def __init__(self, resolutions: Sequence[Tuple[int, int, int]] = ((1024, 120, 600), (2048, 240, 1200), (512, 50, 240)),
                 channels: int = 32):
        super().__init__()
        self.discriminators = nn.ModuleList([ResolutionDiscriminator(*r, channels=channels) for r in resolutions])

    def forward(self, x):
        return [d(x) for d in self.discriminators]


# ------------------------------------------------------------------------------------------------ losses
def generator_adversarial_loss(fake_outputs) -> torch.Tensor:
    """Least-squares GAN: sum over discriminators of mean((1 - D(G(z)))^2)."""
    return sum(torch.mean((1 - o) ** 2) for o, _ in fake_outputs)


def discriminator_adversarial_loss(real_outputs, fake_outputs) -> torch.Tensor:
    return sum(torch.mean((1 - r) ** 2) + torch.mean(f ** 2) for (r, _), (f, _) in zip(real_outputs, fake_outputs))


def feature_matching_loss(real_outputs, fake_outputs) -> torch.Tensor:
    loss = 0.0
    for (_, rf), (_, ff) in zip(real_outputs, fake_outputs):
        for a, b in zip(rf, ff):
            loss = loss + torch.mean(torch.abs(a.detach() - b))
    return 2.0 * loss


def mel_reconstruction_loss(real: torch.Tensor, fake: torch.Tensor, cfg: BigVGANConfig) -> torch.Tensor:
    return F.l1_loss(mel_spectrogram(fake, cfg), mel_spectrogram(real, cfg))


def multi_scale_mel_loss(real, fake, cfg: BigVGANConfig,
                         scales: Sequence[Tuple[int, int]] = ((32, 5), (64, 10), (128, 20), (256, 40), (512, 80), (1024, 160), (2048, 320))):
    """L1 between log-mels at several window sizes (n_fft, n_mels); windows longer than the clip are skipped."""
    loss, used = 0.0, 0
    for n_fft, n_mels in scales:
        if n_fft > real.shape[-1]:
            continue
        hop = n_fft // 4
        loss = loss + F.l1_loss(mel_spectrogram(fake, cfg, n_fft, hop, n_fft, n_mels), mel_spectrogram(real, cfg, n_fft, hop, n_fft, n_mels))
        used += 1
    return loss / max(used, 1)


def generator_loss(real, fake, discriminators: Sequence[nn.Module], cfg: BigVGANConfig, lambda_mel: float = 45.0):
    """Adversarial + feature matching over all discriminators + weighted mel reconstruction. real / fake [B, 1, T]."""
    adv, fm = 0.0, 0.0
    for d in discriminators:
        ro, fo = d(real), d(fake)
        adv = adv + generator_adversarial_loss(fo)
        fm = fm + feature_matching_loss(ro, fo)
    mel = mel_reconstruction_loss(real[:, 0], fake[:, 0], cfg)
    return adv + fm + lambda_mel * mel, dict(adv=float(adv.detach()), fm=float(fm.detach()), mel=float(mel.detach()))


def discriminator_loss(real, fake, discriminators: Sequence[nn.Module]) -> torch.Tensor:
    return sum(discriminator_adversarial_loss(d(real), d(fake.detach())) for d in discriminators)
