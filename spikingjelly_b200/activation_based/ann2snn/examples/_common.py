"""Shared pieces of the conversion examples: generated stand-ins for the datasets (``--synthetic``: no download, no
checkpoint), a short supervised fit of the source network, and accuracy of the source network and of the converted
network as a function of the number of simulation steps."""
import argparse
import json
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
from torch.utils.data import DataLoader, TensorDataset

from ... import functional


def add_common_args(p: argparse.ArgumentParser) -> argparse.ArgumentParser:
    p.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    p.add_argument("--synthetic", action="store_true", help="generated data and a briefly fitted / random network instead of dataset and checkpoint")
    p.add_argument("--output", default=None, help="optional JSON output path")
    p.add_argument("--seed", type=int, default=0)
    return p


def class_blobs(n: int, shape: Tuple[int, ...], classes: int, seed: int = 0, prototypes_seed: int = 1234) -> TensorDataset:
    """Images in [0, 1]: one fixed coarse random pattern per class (4 x 4 cells, so pooling keeps it) plus pixel noise; a small
    network separates them in a few steps."""
    g = torch.Generator().manual_seed(prototypes_seed)
    coarse = (torch.rand((classes, shape[0], 4, 4), generator=g) > 0.5).float()
    prototypes = nn.functional.interpolate(coarse, size=tuple(shape[1:]), mode="nearest")
    g = torch.Generator().manual_seed(seed)
    labels = torch.randint(0, classes, (n,), generator=g)
    images = (0.6 * prototypes[labels] + 0.4 * torch.rand((n,) + tuple(shape), generator=g)).clamp_(0, 1)
    return TensorDataset(images, labels)


def loaders(train_set, test_set, batch_size: int, test_batch_size: Optional[int] = None) -> Tuple[DataLoader, DataLoader]:
    return (DataLoader(train_set, batch_size=batch_size, shuffle=True, drop_last=True),
            DataLoader(test_set, batch_size=test_batch_size or batch_size, shuffle=False))


def fit(net: nn.Module, loader: Iterable, device, epochs: int = 1, lr: float = 1e-3, max_steps: Optional[int] = None) -> float:
    """Plain cross-entropy training of the source ANN; returns the last loss."""
    net.train()
    opt, step, loss = torch.optim.Adam(net.parameters(), lr=lr), 0, torch.tensor(0.0)
    for _ in range(epochs):
        for img, label in loader:
            loss = nn.functional.cross_entropy(net(img.to(device)), label.to(device))
            opt.zero_grad(set_to_none=True)
            loss.backward()
            opt.step()
            step += 1
            if max_steps is not None and step >= max_steps:
                return float(loss.detach())
    return float(loss.detach())


@torch.no_grad()
def ann_accuracy(net: nn.Module, loader: Iterable, device, max_batches: Optional[int] = None) -> float:
    net.eval()
    hit = total = 0
    for i, (img, label) in enumerate(loader):
        hit += int((net(img.to(device)).argmax(1).cpu() == label).sum())
        total += label.numel()
        if max_batches is not None and i + 1 >= max_batches:
            break
    return hit / max(total, 1)


@torch.no_grad()
def snn_accuracy_curve(snn: nn.Module, loader: Iterable, device, time_steps: int, max_batches: Optional[int] = None,
                       delay_start: int = 0) -> List[float]:
    """Accuracy of the accumulated output after each of ``time_steps`` steps (constant input current at every step).  Steps
    before ``delay_start`` run but are not accumulated (the deep layers have not received spikes yet)."""
    snn.eval()
    hits, total = torch.zeros(time_steps), 0
    for i, (img, label) in enumerate(loader):
        functional.reset_net(snn)
        img, acc = img.to(device), 0.0
        for t in range(time_steps):
            out = snn(img)
            if t >= delay_start:
                acc = acc + out
            if torch.is_tensor(acc):
                hits[t] += float((acc.argmax(1).cpu() == label).sum())
        total += label.numel()
        if max_batches is not None and i + 1 >= max_batches:
            break
    functional.reset_net(snn)
    return (hits / max(total, 1)).tolist()


def firing_rates(snn: nn.Module, loader: Iterable, device, time_steps: int) -> Dict[str, float]:
    """Mean firing rate of every spiking neuron layer of the converted network on the first batch."""
    from ... import neuron
    sums: Dict[str, List[float]] = {}
    hooks = [m.register_forward_hook(lambda mod, i, o, n=n: sums.setdefault(n, []).append(float(o.float().mean())))
             for n, m in snn.named_modules() if isinstance(m, neuron.BaseNode)]
    img, _ = next(iter(loader))
    functional.reset_net(snn)
    with torch.no_grad():
        for _ in range(time_steps):
            snn(img.to(device))
    for h in hooks:
        h.remove()
    functional.reset_net(snn)
    return {n: sum(v) / len(v) for n, v in sums.items()}


def report(results: dict, output: Optional[str]) -> dict:
    text = json.dumps(results, indent=1)
    print(text)
    if output:
        Path(output).parent.mkdir(parents=True, exist_ok=True)
        Path(output).write_text(text)
    return results


def curve_summary(curve: Sequence[float], marks: Sequence[int] = (1, 2, 4, 8, 16, 32, 64, 128)) -> Dict[str, float]:
    return {f"T={t}": round(curve[t - 1], 4) for t in marks if t <= len(curve)}
