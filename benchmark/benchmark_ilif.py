#!/usr/bin/env python
"""ILIF neuron (integer-valued multi-level spikes, soft reset), multi-step, forward or forward + backward: time per call and
peak memory for each backend (counterpart of the reference's ``benchmark/benchmark_ilif.py``).  ``--impl ours`` compares the
eager backend with the generated CUDA kernel (the neuron's own step rule compiled by the FlexSN generator);
``--impl reference`` the reference's eager and Triton backends.

    python benchmark/benchmark_ilif.py [--T 32 --numel 262144 --mode train] [--impl ours|reference]
"""
import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))
import _arms  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--T", type=int, default=32)
    ap.add_argument("--numel", type=int, default=1 << 18)
    ap.add_argument("--mode", choices=("eval", "train"), default="train")
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--repeat", type=int, default=50)
    a = ap.parse_args()
    try:
        arm = _arms.load(a.impl)
        neuron = arm.get("neuron")
    except Exception as exc:
        return _arms.unavailable(a.impl, exc)
    train = a.mode == "train"
    for backend in ("torch", arm.fast_backend):
        try:
            node = neuron.ILIFNode(step_mode="m", backend=backend).cuda()
            x = torch.randn(a.T, a.numel, device="cuda", requires_grad=train)

            def step():
                node.reset()
                x.grad = None
                y = node(x)
                if train:
                    y.sum().backward()
            samples = _arms.time_cuda(step, a.warmup, a.repeat)
            torch.cuda.synchronize()
            torch.cuda.reset_peak_memory_stats()
            step()
            torch.cuda.synchronize()
            row = {"impl": a.impl, "backend": backend, "T": a.T, "numel": a.numel, "mode": a.mode, "peak_mb": round(torch.cuda.max_memory_allocated() / 2 ** 20, 1)}
            row.update({k: round(v, 4) for k, v in _arms.summary(samples).items()})
        except Exception as exc:
            row = {"impl": a.impl, "backend": backend, "failed": f"{type(exc).__name__}: {exc}"[:200]}
        print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
