"""Shared pieces of the example scripts: device choice, synthetic stand-ins for datasets (the scripts run without any
download when ``--synthetic`` is given) and a small train / evaluate loop."""
from __future__ import annotations

import argparse
import time
from typing import Callable, Iterable, Tuple

import torch
import torch.nn as nn
from torch.utils.data import DataLoader, TensorDataset

from .. import functional


def pick_device(name: str = "auto") -> torch.device:
    if name == "auto":
        name = "cuda" if torch.cuda.is_available() else "cpu"
    return torch.device(name)


def pick_backend(device: torch.device, requested: str = "auto") -> str:
    return ("cuda" if device.type == "cuda" else "torch") if requested == "auto" else requested


def synthetic_images(n: int, shape: Tuple[int, ...], classes: int, seed: int = 0) -> TensorDataset:
    """Class-dependent blobs: learnable in a few steps, so the scripts' loss curves mean something."""
    g = torch.Generator().manual_seed(seed)
    y = torch.randint(0, classes, (n,), generator=g)
    proto = torch.rand(classes, *shape, generator=g)
    x = (proto[y] * 0.8 + torch.rand(n, *shape, generator=g) * 0.2).clamp(0, 1)
    return TensorDataset(x, y)


def add_common_args(p: argparse.ArgumentParser) -> argparse.ArgumentParser:
    p.add_argument("--device", default="auto")
    p.add_argument("--backend", default="auto", help="neuron backend: auto | torch | cuda")
    p.add_argument("--synthetic", action="store_true", help="use generated data instead of the real dataset")
    p.add_argument("--data-dir", default="./data")
    p.add_argument("-b", "--batch-size", type=int, default=64)
    p.add_argument("--epochs", type=int, default=1)
    p.add_argument("--max-steps", type=int, default=0, help="stop each epoch after this many batches (0 = all)")
    p.add_argument("--lr", type=float, default=1e-3)
    p.add_argument("--amp", action="store_true", help="bf16 autocast")
    return p


def run_epochs(net: nn.Module, train: Iterable, test: Iterable, forward: Callable, loss_fn: Callable, args, device) -> dict:
    """``forward(net, x) -> [N, classes]`` firing rates; resets the network after every batch."""
    opt = torch.optim.Adam(net.parameters(), lr=args.lr)
    stats = {}
    for epoch in range(args.epochs):
        for phase, loader in (("train", train), ("test", test)):
            net.train(phase == "train")
            seen = correct = 0
            total_loss, t0 = 0.0, time.time()
            for step, (x, y) in enumerate(loader):
                if args.max_steps and step >= args.max_steps:
                    break
                x, y = x.to(device, non_blocking=True), y.to(device, non_blocking=True)
                with torch.set_grad_enabled(phase == "train"), torch.autocast(device.type, dtype=torch.bfloat16, enabled=args.amp):
                    out = forward(net, x)
                    loss = loss_fn(out.float(), y)
                if phase == "train":
                    opt.zero_grad(set_to_none=True)
                    loss.backward()
                    opt.step()
                functional.reset_net(net)
                seen += y.numel()
                correct += (out.argmax(1) == y).sum().item()
                total_loss += loss.item() * y.numel()
            stats[f"{phase}_loss"], stats[f"{phase}_acc"] = total_loss / max(seen, 1), correct / max(seen, 1)
            print(f"epoch {epoch} {phase}: loss {stats[f'{phase}_loss']:.4f} acc {stats[f'{phase}_acc']:.4f} "
                  f"{seen / max(time.time() - t0, 1e-9):.0f} samples/s")
    return stats


def loaders(train_set, test_set, args) -> Tuple[DataLoader, DataLoader]:
    kw = dict(batch_size=args.batch_size, num_workers=0, pin_memory=torch.cuda.is_available())
    return DataLoader(train_set, shuffle=True, drop_last=True, **kw), DataLoader(test_set, shuffle=False, **kw)
