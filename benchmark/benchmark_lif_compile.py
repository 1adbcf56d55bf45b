#!/usr/bin/env python
"""A LIF written as plain PyTorch, stepped T times per sequence, gradient-free: eager, under ``torch.compile``, and the same
sequence through this framework's scan kernel in one launch.  Counterpart of the reference's
``benchmark/flexsn/benchmark_lif_compile.py`` (eager against ``torch.compile``), with the kernel as a third row.

    python benchmark/benchmark_lif_compile.py [--T 32 --batch 64 --neurons 50176] [--no-compile]
"""
import argparse
import json
import sys
from pathlib import Path

import torch
import torch.nn as nn

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))
import _arms  # noqa: E402


class PlainLIF(nn.Module):
    """Charge ``v += (x - v) / tau``, fire at ``v >= threshold``, hard reset to 0: the defaults of ``LIFNode``."""

    def __init__(self, tau: float = 2.0, threshold: float = 1.0):
        super().__init__()
        self.tau, self.threshold = tau, threshold

    def forward(self, x, v):
        v = v + (x - v) / self.tau
        s = (v >= self.threshold).to(x.dtype)
        return s, v * (1.0 - s)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--T", type=int, default=32)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--neurons", type=int, default=224 * 224)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--no-compile", action="store_true")
    a = ap.parse_args()
    dev = torch.device("cuda")
    torch.manual_seed(0)
    x = torch.rand(a.T, a.batch, a.neurons, device=dev)

    def stepped(model):
        def run():
            v = torch.zeros_like(x[0])
            for t in range(a.T):
                s, v = model(x[t], v)
            return s
        return run
    rows = {}
    with torch.no_grad():
        eager = PlainLIF().to(dev)
        rows["eager"] = _arms.summary(_arms.time_cuda(stepped(eager), 3, a.iters))["median_ms"]
        if not a.no_compile:
            try:
                rows["torch.compile"] = _arms.summary(_arms.time_cuda(stepped(torch.compile(PlainLIF().to(dev))), 5, a.iters))["median_ms"]
            except Exception as exc:
                rows["torch.compile"] = f"{type(exc).__name__}: {exc}"[:120]
        from spikingjelly_b200.activation_based import functional, neuron
        node = neuron.LIFNode(tau=2.0, step_mode="m", backend="cuda").to(dev)
        want = torch.stack([eager(x[t], v)[0] for v in [torch.zeros_like(x[0])] for t in range(1)])      # first step only: same rule

        def kernel():
            functional.reset_net(node)
            return node(x)
        assert torch.equal(kernel()[0], want[0])
        rows["scan kernel (one launch)"] = _arms.summary(_arms.time_cuda(kernel, 3, a.iters))["median_ms"]
    out = {"T": a.T, "batch": a.batch, "neurons": a.neurons, "ms": {k: (round(v, 3) if isinstance(v, float) else v) for k, v in rows.items()}}
    if isinstance(rows.get("eager"), float):
        out["kernel_over_eager_speedup"] = round(rows["eager"] / rows["scan kernel (one launch)"], 1)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
