#!/usr/bin/env python
"""SpikeZIP-TF conversion of a quantised ViT-Small (patch 16, 384 wide, 12 blocks, 6 heads, LSQ-style quantisers of
``--level`` levels): logits of the QANN against the time-summed logits of the converted SNN, and the time of both.
Counterpart of the reference's ``benchmark/benchmark_ann2snn_spikezip_vit_qann.py``, which loads a trained checkpoint and
ImageNet; here the weights are random, the quantiser steps are calibrated on one synthetic batch, and the images are
synthetic, so the figures are parity and time, not accuracy.

    python benchmark/benchmark_ann2snn_spikezip_vit_qann.py [--impl ours|reference] [--step-mode m|s] [--time-steps 64]
"""
import argparse
import json
import sys
import time
from pathlib import Path

import torch
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, str(Path(__file__).resolve().parent))
import _arms  # noqa: E402


class Quan(nn.Module):
    def __init__(self, level: int, sym: bool):
        super().__init__()
        self.level, self.sym = int(level), bool(sym)
        self.register_buffer("pos_max", torch.tensor(float(level // 2 - 1 if sym else level - 1)))
        self.register_buffer("neg_min", torch.tensor(float(-level // 2 if sym else 0)))
        self.s = nn.Parameter(torch.tensor(1.0))

    def forward(self, x):
        return torch.clamp(torch.floor(x / self.s + 0.5), min=self.neg_min, max=self.pos_max) * self.s


class QAttention(nn.Module):
    def __init__(self, dim, heads, level):
        super().__init__()
        self.num_heads, self.head_dim = heads, dim // heads
        self.scale, self.level, self.is_softmax = self.head_dim ** -0.5, level, True
        self.qkv = nn.Linear(dim, dim * 3)
        self.quan_q, self.quan_k, self.quan_v = Quan(level, True), Quan(level, True), Quan(level, True)
        self.attn_drop, self.proj_drop = nn.Dropout(0.0), nn.Dropout(0.0)
        self.proj, self.quan_proj = nn.Linear(dim, dim), Quan(level, True)
        self.attn_quan, self.after_attn_quan = Quan(level, False), Quan(level, True)

    def forward(self, x):
        b, l, c = x.shape
        q, k, v = self.qkv(x).reshape(b, l, 3, self.num_heads, self.head_dim).permute(2, 0, 3, 1, 4).unbind(0)
        p = self.attn_quan(F.softmax(self.quan_q(q) * self.scale @ self.quan_k(k).transpose(-2, -1), dim=-1))
        y = self.after_attn_quan(p @ self.quan_v(v)).transpose(1, 2).reshape(b, l, c)
        return self.quan_proj(self.proj(y))


class QMLP(nn.Module):
    def __init__(self, dim, hidden, level):
        super().__init__()
        self.fc1 = nn.Linear(dim, hidden)
        self.act = nn.Sequential(Quan(level, False), nn.ReLU())
        self.fc2 = nn.Sequential(nn.Linear(hidden, dim), Quan(level, True))

    def forward(self, x):
        return self.fc2(self.act(self.fc1(x)))


class QBlock(nn.Module):
    def __init__(self, dim, heads, ratio, level):
        super().__init__()
        self.norm1 = nn.Sequential(nn.LayerNorm(dim, eps=1e-6), Quan(level, True))
        self.attn = QAttention(dim, heads, level)
        self.norm2 = nn.Sequential(nn.LayerNorm(dim, eps=1e-6), Quan(level, True))
        self.mlp = QMLP(dim, dim * ratio, level)

    def forward(self, x):
        x = x + self.attn(self.norm1(x))
        return x + self.mlp(self.norm2(x))


class PatchEmbed(nn.Module):
    def __init__(self, dim, level, patch):
        super().__init__()
        self.proj = nn.Sequential(nn.Conv2d(3, dim, patch, stride=patch), Quan(level, True))

    def forward(self, x):
        return self.proj(x)


class QViT(nn.Module):
    def __init__(self, level=32, dim=384, depth=12, heads=6, image=224, patch=16, classes=1000):
        super().__init__()
        self.patch_embed = PatchEmbed(dim, level, patch)
        n = (image // patch) ** 2
        self.cls_token = nn.Parameter(torch.randn(1, 1, dim) * 0.02)
        self.pos_embed = nn.Parameter(torch.randn(1, n + 1, dim) * 0.02)
        self.pos_drop = nn.Dropout(0.0)
        self.blocks = nn.Sequential(*[QBlock(dim, heads, 4, level) for _ in range(depth)])
        self.norm = nn.Sequential(nn.LayerNorm(dim, eps=1e-6), Quan(level, True))
        self.head = nn.Linear(dim, classes)

    def forward(self, x):
        x = self.patch_embed.proj(x).flatten(2).transpose(1, 2)
        x = self.pos_drop(torch.cat((self.cls_token.expand(x.shape[0], -1, -1), x), dim=1) + self.pos_embed)
        return self.head(self.norm(self.blocks(x))[:, 0])


def calibrate(model: nn.Module, x: torch.Tensor) -> None:
    """One forward pass in which every quantiser sets its step from the range of the tensor it is about to quantise."""
    def hook(q, inputs):
        v = inputs[0].detach()
        top = v.abs().max() if q.sym else v.max().clamp_min(1e-6)
        q.s.data.copy_(top / q.pos_max.clamp_min(1.0))
    handles = [m.register_forward_pre_hook(hook) for m in model.modules() if isinstance(m, Quan)]
    with torch.no_grad():
        model(x)
    for h in handles:
        h.remove()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--time-steps", type=int, default=64)
    ap.add_argument("--level", type=int, default=32)
    ap.add_argument("--batch-size", type=int, default=2)
    ap.add_argument("--batches", type=int, default=2)
    ap.add_argument("--step-mode", choices=("m", "s"), default="m")
    ap.add_argument("--dim", type=int, default=384)
    ap.add_argument("--depth", type=int, default=12)
    ap.add_argument("--heads", type=int, default=6)
    ap.add_argument("--image-size", type=int, default=224)
    ap.add_argument("--parity-atol", type=float, default=1e-4)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()
    try:
        arm = _arms.load(a.impl)
        functional, ann2snn = arm.get("functional"), arm.get("ann2snn")
    except Exception as exc:
        return _arms.unavailable(a.impl, exc)
    dev = torch.device(a.device)
    torch.manual_seed(a.seed)
    qann = QViT(a.level, a.dim, a.depth, a.heads, a.image_size).to(dev).eval()
    images = [torch.randn(a.batch_size, 3, a.image_size, a.image_size, device=dev) for _ in range(a.batches)]
    calibrate(qann, images[0])
    snn = ann2snn.ModuleConverter(recipe=ann2snn.SpikeZIPTFQANNRecipe(time_steps=a.time_steps, model_family="vit"), device=dev).convert(qann).eval()
    functional.set_step_mode(snn, a.step_mode)
    if a.impl == "reference" and dev.type == "cuda" and arm.fast_backend == "triton":
        functional.set_backend(snn, "triton", instance=arm.get("neuron").STBIFNeuron)
    sync = (lambda: torch.cuda.synchronize(dev)) if dev.type == "cuda" else (lambda: None)

    def run_snn(x):
        functional.reset_net(snn)
        seq = torch.zeros(a.time_steps, *x.shape, device=dev)
        seq[0] = x
        if a.step_mode == "m":
            return snn(seq).sum(0)
        return torch.stack([snn(s) for s in seq]).sum(0)

    t_q = t_s = 0.0
    worst, mismatched, agree, total = 0.0, 0, 0, 0
    with torch.inference_mode():
        run_snn(images[0])                               # kernels compiled / caches warm
        qann(images[0])
        for x in images:
            sync(); t0 = time.perf_counter(); want = qann(x); sync(); t_q += time.perf_counter() - t0
            sync(); t0 = time.perf_counter(); got = run_snn(x); sync(); t_s += time.perf_counter() - t0
            d = (got - want).abs()
            worst = max(worst, d.max().item())
            mismatched += int((d > a.parity_atol).sum())
            agree += int((got.argmax(-1) == want.argmax(-1)).sum())
            total += x.shape[0]
    print(json.dumps({"impl": a.impl, "device": str(dev), "step_mode": a.step_mode, "time_steps": a.time_steps, "level": a.level,
                      "samples": total, "qann_ms_per_batch": round(t_q / a.batches * 1e3, 2), "snn_ms_per_batch": round(t_s / a.batches * 1e3, 2),
                      "logit_max_abs_diff": worst, "logits_off_by_more_than_atol": mismatched, "top1_agreement": agree / total}))


if __name__ == "__main__":
    main()
