#!/usr/bin/env python
"""Training step of a small convolutional SNN (Conv-BN-LIF-Pool x 2, Linear-LIF-Linear; T 16, batch 64, 3 x 64 x 64
input) under each neuron backend, eager and through ``torch.compile``.  Counterpart of the reference's
``benchmark/benchmark_train_backends.py`` (same network, same sizes, Adam, cross entropy, shared initial weights).
``--impl ours``: backends ``torch`` and ``cuda``; ``--impl reference``: ``torch`` and ``triton``.

    python benchmark/benchmark_train_backends.py [--impl ours|reference] [--iters 100] [--no-compile] [--out file.jsonl]

Timing: CUDA events around ``--iters`` steps after ``--warmup`` steps; one JSON line per mode.
"""
import argparse
import json
import sys
from pathlib import Path

import torch
import torch.nn as nn

sys.path.insert(0, str(Path(__file__).resolve().parent))
import _arms  # noqa: E402

T, BATCH, C_IN, IMG, C1, C2, HIDDEN, CLASSES = 16, 64, 3, 64, 64, 128, 1024, 10
SEED = 20260420


def build(arm, backend: str) -> nn.Module:
    layer, neuron, surrogate = arm.get("layer"), arm.get("neuron"), arm.get("surrogate")

    def lif():
        return neuron.LIFNode(tau=2.0, decay_input=True, v_threshold=1.0, v_reset=0.0, surrogate_function=surrogate.Sigmoid(alpha=4.0),
                              detach_reset=False, step_mode="m", backend=backend)

    class SmallSNN(nn.Module):
        def __init__(self):
            super().__init__()
            self.conv1, self.bn1, self.sn1 = layer.Conv2d(C_IN, C1, 3, padding=1, step_mode="m"), layer.BatchNorm2d(C1, step_mode="m"), lif()
            self.pool1 = layer.MaxPool2d(2, 2, step_mode="m")
            self.conv2, self.bn2, self.sn2 = layer.Conv2d(C1, C2, 3, padding=1, step_mode="m"), layer.BatchNorm2d(C2, step_mode="m"), lif()
            self.pool2 = layer.MaxPool2d(2, 2, step_mode="m")
            self.flat = layer.Flatten(step_mode="m")
            self.fc1, self.sn3 = layer.Linear(C2 * (IMG // 4) ** 2, HIDDEN, step_mode="m"), lif()
            self.fc2 = layer.Linear(HIDDEN, CLASSES, step_mode="m")

        def forward(self, x):
            x = self.pool1(self.sn1(self.bn1(self.conv1(x))))
            x = self.pool2(self.sn2(self.bn2(self.conv2(x))))
            return self.fc2(self.sn3(self.fc1(self.flat(x)))).mean(0)
    return SmallSNN()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--no-compile", action="store_true")
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    try:
        arm = _arms.load(a.impl)
        functional = arm.get("functional")
    except Exception as exc:
        return _arms.unavailable(a.impl, exc)
    dev = torch.device("cuda")
    torch.manual_seed(SEED)
    x = torch.randn(T, BATCH, C_IN, IMG, IMG, device=dev)
    y = torch.randint(CLASSES, (BATCH,), device=dev)
    state = build(arm, "torch").to(dev).state_dict()
    modes = [("torch", False), (arm.fast_backend, False)]
    if not a.no_compile:
        modes += [("torch", True), (arm.fast_backend, True)]
    for backend, compiled in modes:
        name = f"{backend} backend" + (" + torch.compile" if compiled else "")
        try:
            model = build(arm, backend).to(dev)
            model.load_state_dict(state, strict=True)
            model.train()
            run = torch.compile(model) if compiled else model
            opt = torch.optim.Adam(model.parameters(), lr=1e-3)
            loss_fn = nn.CrossEntropyLoss()

            def step():
                functional.reset_net(model)
                opt.zero_grad(set_to_none=True)
                loss_fn(run(x), y).backward()
                opt.step()
            for _ in range(a.warmup):
                step()
            torch.cuda.synchronize()
            torch.cuda.empty_cache()
            torch.cuda.reset_peak_memory_stats()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(a.iters):
                step()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / a.iters
            row = {"impl": a.impl, "mode": name, "avg_step_ms": round(ms, 3), "samples_per_s": round(BATCH / ms * 1e3, 1),
                   "max_mem_mb": round(torch.cuda.max_memory_allocated() / 2 ** 20, 1)}
        except Exception as exc:
            row = {"impl": a.impl, "mode": name, "failed": f"{type(exc).__name__}: {exc}"[:200]}
        print(json.dumps(row), flush=True)
        if a.out:
            with open(a.out, "a") as f:
                f.write(json.dumps(row) + "\n")


if __name__ == "__main__":
    main()
