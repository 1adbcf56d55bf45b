"""Keyword spotting on Google Speech Commands with a spiking convolutional network over log-mel frames (the reference's
``examples/speechcommands.py``): waveform -> power spectrogram -> mel filter bank (+ first-order delta) -> three dilated
convolutions along time, each followed by BatchNorm and a multi-step LIF layer run over the FRAME axis (time of the audio is
the simulation time) -> linear read-out of the firing rates.

``--synthetic`` replaces the dataset by tones whose pitch depends on the class, so the script runs without torchaudio or a
download; with the real data ``datasets.SpeechCommands`` (which needs torchaudio to decode the files) is used.

    python -m spikingjelly_b200.activation_based.examples.speechcommands --synthetic --max-steps 20
"""
from __future__ import annotations

import argparse
import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.data import TensorDataset

from .. import functional, layer, neuron, surrogate
from . import _common as C

SAMPLE_RATE = 16000


def hz_to_mel(f: torch.Tensor) -> torch.Tensor:
    return 2595.0 * torch.log10(1.0 + f / 700.0)


def mel_to_hz(m: torch.Tensor) -> torch.Tensor:
    return 700.0 * (10.0 ** (m / 2595.0) - 1.0)


def mel_filter_bank(n_freqs: int, n_mels: int, f_min: float, f_max: float, sample_rate: int) -> torch.Tensor:
    """Triangular filters, ``[n_freqs, n_mels]`` (HTK mel scale)."""
    freqs = torch.linspace(0, sample_rate / 2, n_freqs)
    pts = mel_to_hz(torch.linspace(float(hz_to_mel(torch.tensor(f_min))), float(hz_to_mel(torch.tensor(f_max))), n_mels + 2))
    up = (freqs[:, None] - pts[None, :-2]) / (pts[1:-1] - pts[:-2])[None]
    down = (pts[None, 2:] - freqs[:, None]) / (pts[2:] - pts[1:-1])[None]
    return torch.clamp(torch.minimum(up, down), min=0.0)


class LogMelDelta(nn.Module):
    """Waveform ``[N, samples]`` -> ``[N, 2, frames, n_mels]``: log-mel energies and their first difference along time."""

    def __init__(self, n_fft: int = 512, hop: int = 160, n_mels: int = 40, f_min: float = 20.0, f_max: float = 4000.0):
        super().__init__()
        self.n_fft, self.hop = n_fft, hop
        self.register_buffer("window", torch.hann_window(n_fft), persistent=False)
        self.register_buffer("fb", mel_filter_bank(n_fft // 2 + 1, n_mels, f_min, f_max, SAMPLE_RATE), persistent=False)

    def forward(self, wav: torch.Tensor) -> torch.Tensor:
        spec = torch.stft(wav, self.n_fft, self.hop, window=self.window, return_complex=True).abs().pow(2)     # [N, F, frames]
        mel = torch.log(spec.transpose(1, 2) @ self.fb + 1e-6)                                                  # [N, frames, mels]
        delta = F.pad(mel[:, 1:] - mel[:, :-1], (0, 0, 1, 0))
        return torch.stack([mel, delta], dim=1)


class SpeechNet(nn.Module):
    def __init__(self, n_mels: int, classes: int, channels: int = 64, backend: str = "torch"):
        super().__init__()
        def block(cin, dilation):
            return nn.Sequential(
                layer.Conv2d(cin, channels, kernel_size=(4, 3), dilation=(dilation, 1), padding=(0, 1), bias=False, step_mode="s"),
                layer.BatchNorm2d(channels, step_mode="s"))
        self.convs = nn.ModuleList([block(2, 1), block(channels, 4), block(channels, 16)])
        self.lifs = nn.ModuleList(neuron.LIFNode(tau=10.0 / 7.0, surrogate_function=surrogate.ATan(), detach_reset=True,
                                                 step_mode="m", backend=backend) for _ in range(3))
        self.fc = nn.Linear(channels * n_mels, classes)

    def forward(self, feats: torch.Tensor) -> torch.Tensor:            # [N, 2, frames, mels]
        x = feats
        for conv, lif in zip(self.convs, self.lifs):
            y = conv(x)                                                 # [N, C, frames', mels]: frames are the time axis
            s = lif(y.permute(2, 0, 1, 3).contiguous())                 # LIF over frames: [T = frames', N, C, mels]
            x = s.permute(1, 2, 0, 3)
        rate = x.mean(2)                                                # firing rate over time: [N, C, mels]
        return self.fc(rate.flatten(1))


def synthetic_speech(n: int, classes: int, seed: int = 0, samples: int = SAMPLE_RATE) -> TensorDataset:
    g = torch.Generator().manual_seed(seed)
    y = torch.randint(0, classes, (n,), generator=g)
    t = torch.arange(samples) / SAMPLE_RATE
    f0 = 300.0 + 250.0 * y.float()
    wav = torch.sin(2 * math.pi * f0[:, None] * t[None]) * 0.5 + 0.05 * torch.randn(n, samples, generator=g)
    return TensorDataset(wav, y)


def main(argv=None) -> dict:
    p = C.add_common_args(argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter))
    p.add_argument("--classes", type=int, default=12)
    p.add_argument("--channels", type=int, default=64)
    p.add_argument("--n-mels", type=int, default=40)
    a = p.parse_args(argv)
    device = C.pick_device(a.device)
    if a.synthetic:
        a.classes = min(a.classes, 6)
        train_set, test_set = synthetic_speech(256, a.classes, 0), synthetic_speech(64, a.classes, 1)
    else:
        from ...datasets import SpeechCommands
        words = ["yes", "no", "up", "down", "left", "right", "on", "off", "stop", "go"]
        label_dict = {w: i for i, w in enumerate(words)}
        label_dict.update({"_silence_": 10, "_unknown_": 11})

        def fix_length(wav):
            wav = torch.as_tensor(wav).float().flatten()[:SAMPLE_RATE]
            return F.pad(wav, (0, SAMPLE_RATE - wav.numel()))
        train_set = SpeechCommands(label_dict, a.data_dir, silence_cnt=2300, split="train", transform=fix_length, download=True)
        test_set = SpeechCommands(label_dict, a.data_dir, silence_cnt=260, split="test", transform=fix_length, download=True)
        a.classes = 12
    train, test = C.loaders(train_set, test_set, a)
    front = LogMelDelta(n_mels=a.n_mels).to(device)
    net = SpeechNet(a.n_mels, a.classes, a.channels, C.pick_backend(device, a.backend)).to(device)

    def forward(net, wav):
        with torch.no_grad():
            feats = front(wav)
            feats = (feats - feats.mean(dim=(2, 3), keepdim=True)) / (feats.std(dim=(2, 3), keepdim=True) + 1e-5)
        return net(feats)

    return C.run_epochs(net, train, test, forward, lambda out, y: F.cross_entropy(out, y), a, device)


if __name__ == "__main__":
    main()
