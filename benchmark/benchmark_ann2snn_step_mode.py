#!/usr/bin/env python
"""Converted-SNN inference: a Python loop of single steps against one multi-step call, for the rate-coding recipe (a
Conv-BN-ReLU-AvgPool classifier) and the STA transformer recipe (a pre-norm transformer classifier).  Counterpart of the
reference's ``benchmark/benchmark_ann2snn_rate_coding_step_mode.py`` and ``benchmark_ann2snn_sta_step_mode.py``: the two
paths must agree (``--atol`` / ``--rtol``) before either is timed.

    python benchmark/benchmark_ann2snn_step_mode.py --recipe rate|sta [--impl ours|reference] [--device cuda]
"""
import argparse
import copy
import json
import sys
import time
from pathlib import Path

import torch
import torch.nn as nn

sys.path.insert(0, str(Path(__file__).resolve().parent))
import _arms  # noqa: E402


class ConvClassifier(nn.Module):
    def __init__(self, in_channels, channels, image_size, depth, hidden, classes):
        super().__init__()
        blocks, c, size = [], in_channels, image_size
        for _ in range(depth):
            blocks += [nn.Conv2d(c, channels, 3, padding=1, bias=False), nn.BatchNorm2d(channels), nn.ReLU(), nn.AvgPool2d(2)]
            c, size = channels, size // 2
        self.features = nn.Sequential(*blocks)
        self.flatten = nn.Flatten()
        self.fc0, self.relu, self.fc1 = nn.Linear(c * size * size, hidden), nn.ReLU(), nn.Linear(hidden, classes)

    def forward(self, x):
        return self.fc1(self.relu(self.fc0(self.flatten(self.features(x)))))


class Block(nn.Module):
    def __init__(self, dim, heads, mlp):
        super().__init__()
        self.norm1 = nn.LayerNorm(dim)
        self.attn = nn.MultiheadAttention(dim, heads, dropout=0.0, batch_first=True)
        self.norm2 = nn.LayerNorm(dim)
        self.fc1, self.act, self.fc2 = nn.Linear(dim, mlp), nn.GELU(), nn.Linear(mlp, dim)

    def forward(self, x):
        y = self.norm1(x)
        attn, _ = self.attn(y, y, y, need_weights=False)
        x = x + attn
        return x + self.fc2(self.act(self.fc1(self.norm2(x))))


class TransformerClassifier(nn.Module):
    def __init__(self, input_dim, dim, depth, heads, mlp, classes):
        super().__init__()
        self.token_proj = nn.Linear(input_dim, dim)
        self.blocks = nn.ModuleList(Block(dim, heads, mlp) for _ in range(depth))
        self.head_norm, self.head = nn.LayerNorm(dim), nn.Linear(dim, classes)

    def forward(self, x):
        x = self.token_proj(x)
        for b in self.blocks:
            x = b(x)
        return self.head(self.head_norm(x.mean(dim=1)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--recipe", choices=["rate", "sta"], default="rate")
    ap.add_argument("--sta-mode", default="equivalent", help="STATransformerRecipe mode (equivalent | spiking_encoder | spiking_affine)")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--time-steps", type=int, default=16)
    ap.add_argument("--batch-size", type=int, default=None, help="default 64 (rate) / 32 (sta)")
    ap.add_argument("--batches-per-epoch", type=int, default=None, help="default 64 (rate) / 32 (sta)")
    ap.add_argument("--epochs", type=int, default=5)
    ap.add_argument("--warmup-epochs", type=int, default=1)
    ap.add_argument("--calibration-batches", type=int, default=4)
    ap.add_argument("--seed", type=int, default=20260703)
    ap.add_argument("--neuron-backend", default=None, help="set_backend(model, ...) on the converted network; 'fast' = this arm's kernel backend")
    ap.add_argument("--atol", type=float, default=None)
    ap.add_argument("--rtol", type=float, default=None)
    # rate-coding model
    ap.add_argument("--image-size", type=int, default=32)
    ap.add_argument("--in-channels", type=int, default=3)
    ap.add_argument("--channels", type=int, default=64)
    ap.add_argument("--conv-depth", type=int, default=3)
    ap.add_argument("--hidden-dim", type=int, default=512)
    # transformer model
    ap.add_argument("--seq-len", type=int, default=64)
    ap.add_argument("--input-dim", type=int, default=128)
    ap.add_argument("--embed-dim", type=int, default=256)
    ap.add_argument("--mlp-dim", type=int, default=1024)
    ap.add_argument("--depth", type=int, default=4)
    ap.add_argument("--num-heads", type=int, default=8)
    ap.add_argument("--num-classes", type=int, default=1000)
    a = ap.parse_args()
    rate = a.recipe == "rate"
    bs = a.batch_size or (64 if rate else 32)
    nb = a.batches_per_epoch or (64 if rate else 32)
    tol = dict(atol=a.atol if a.atol is not None else (1e-5 if rate else 1e-4), rtol=a.rtol if a.rtol is not None else (1e-5 if rate else 1e-4))
    try:
        arm = _arms.load(a.impl)
        functional, ann2snn = arm.get("functional"), arm.get("ann2snn")
    except Exception as exc:
        return _arms.unavailable(a.impl, exc)
    dev = torch.device(a.device)
    torch.manual_seed(a.seed)
    shape = (bs, a.in_channels, a.image_size, a.image_size) if rate else (bs, a.seq_len, a.input_dim)
    batches = [torch.rand(shape, device=dev) if rate else torch.randn(shape, device=dev) for _ in range(nb)]
    calib = [(torch.rand(shape, device=dev) if rate else torch.randn(shape, device=dev), torch.zeros(bs, dtype=torch.long))
             for _ in range(a.calibration_batches)]
    if rate:
        ann = ConvClassifier(a.in_channels, a.channels, a.image_size, a.conv_depth, a.hidden_dim, a.num_classes).to(dev).eval()
        recipe = ann2snn.RateCodingRecipe(dataloader=calib, mode="Max", fuse_flag=True)
    else:
        ann = TransformerClassifier(a.input_dim, a.embed_dim, a.depth, a.num_heads, a.mlp_dim, a.num_classes).to(dev).eval()
        recipe = ann2snn.STATransformerRecipe(dataloader=calib if a.sta_mode == "spiking_encoder" else None,
                                              time_steps=a.time_steps, mode=a.sta_mode)
    base = ann2snn.Converter(recipe=recipe, device=dev).convert(ann)
    if a.neuron_backend:
        functional.set_backend(base, arm.fast_backend if a.neuron_backend == "fast" else a.neuron_backend)
    T = a.time_steps

    def sequence(x):                 # rate coding repeats the frame; STA feeds it once and zeros afterwards
        if rate:
            return x.unsqueeze(0).expand(T, *x.shape).contiguous()
        seq = torch.zeros((T, *x.shape), dtype=x.dtype, device=x.device)
        seq[0] = x
        return seq

    def single_epoch(model, bl):
        functional.set_step_mode(model, "s")
        out = None
        for x in bl:
            functional.reset_net(model)
            seq, out = sequence(x), None
            for t in range(T):
                y = model(seq[t])
                out = y if out is None else out + y
        return out

    def multi_epoch(model, bl):
        functional.set_step_mode(model, "m")
        out = None
        for x in bl:
            functional.reset_net(model)
            out = model(sequence(x)).sum(dim=0)
        return out

    sync = (lambda: torch.cuda.synchronize(dev)) if dev.type == "cuda" else (lambda: None)
    single, multi = copy.deepcopy(base).eval(), copy.deepcopy(base).eval()
    worst = 0.0
    with torch.inference_mode():
        for x in batches[:2]:
            s, m = single_epoch(single, [x]), multi_epoch(multi, [x])
            worst = max(worst, (s - m).abs().max().item())
            if not torch.allclose(s, m, **tol):
                raise AssertionError(f"single-step loop and multi-step outputs differ: max_abs_diff={worst:.6g}")
    rows = {}
    with torch.inference_mode():
        for name, fn, model in (("single_step_loop", single_epoch, single), ("multi_step", multi_epoch, multi)):
            for _ in range(a.warmup_epochs):
                fn(model, batches)
            sync()
            t0 = time.perf_counter()
            for _ in range(a.epochs):
                fn(model, batches)
            sync()
            dt = time.perf_counter() - t0
            rows[name] = {"seconds_per_epoch": round(dt / a.epochs, 5), "samples_per_second": round(a.epochs * nb * bs / dt, 1)}
    print(json.dumps({"impl": a.impl, "recipe": a.recipe, "device": str(dev), "time_steps": T, "batch_size": bs,
                      "batches_per_epoch": nb, "neuron_backend": a.neuron_backend or "as converted", "parity_max_abs_diff": worst, "results": rows,
                      "multi_step_speedup": round(rows["single_step_loop"]["seconds_per_epoch"] / rows["multi_step"]["seconds_per_epoch"], 3)}))


if __name__ == "__main__":
    main()
