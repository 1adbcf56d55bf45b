#!/usr/bin/env python
"""Training and inference of a deep fully connected SNN (``--depth`` x [Linear(4096) + LIF], T 16, batch 256) under each
precision policy, through the public precision API (counterpart of the reference's
``benchmark/benchmark_train_precision_snn_fc.py``).  ``--impl reference`` runs the reference's policies and Triton neurons.

    python benchmark/benchmark_train_precision_snn_fc.py [--precisions fp32 bf16 fp8] [--depth 20] [--impl ours|reference]
"""
import argparse
import json
import sys
from pathlib import Path

import torch
import torch.nn as nn

sys.path.insert(0, str(Path(__file__).resolve().parent))
import _arms  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--precisions", nargs="+", default=None)
    ap.add_argument("--time-steps", type=int, default=16)
    ap.add_argument("--batch-size", type=int, default=256)
    ap.add_argument("--input-dim", type=int, default=4096)
    ap.add_argument("--hidden-dim", type=int, default=4096)
    ap.add_argument("--num-classes", type=int, default=1024)
    ap.add_argument("--depth", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--inference-steps", type=int, default=40)
    ap.add_argument("--seed", type=int, default=20260531)
    a = ap.parse_args()
    try:
        arm = _arms.load(a.impl)
        layer, neuron, surrogate, functional, precision = (arm.get(n) for n in ("layer", "neuron", "surrogate", "functional", "precision"))
    except Exception as exc:
        return _arms.unavailable(a.impl, exc)
    modes = a.precisions or (["fp32", "bf16", "fp8"] if a.impl == "ours" else ["fp32", "bf16", "fp8-torchao", "fp8-te"])
    dev = torch.device("cuda", 0)

    def build():
        torch.manual_seed(a.seed)
        sg, mods, width = surrogate.Sigmoid(alpha=4.0), [], a.input_dim
        for _ in range(a.depth - 1):
            mods += [layer.Linear(width, a.hidden_dim, step_mode="m"), neuron.LIFNode(tau=2.0, surrogate_function=sg, step_mode="m", backend=arm.fast_backend)]
            width = a.hidden_dim
        return nn.Sequential(*mods, layer.Linear(width, a.num_classes, step_mode="m")).to(dev)
    x = torch.rand(a.time_steps, a.batch_size, a.input_dim, device=dev)
    y = torch.randint(a.num_classes, (a.batch_size,), device=dev)
    for mode in modes:
        try:
            net = build()
            art = precision.prepare_model_for_precision(net, dev, precision.PrecisionConfig(mode=mode, strictness="strict", device=str(dev)))
            net = art.model
            opt = torch.optim.SGD(net.parameters(), lr=5e-2, momentum=0.9)
            last = {}

            def train():
                opt.zero_grad(set_to_none=True)
                with art.autocast_context():
                    loss = nn.functional.cross_entropy(net(x).mean(0).float(), y)
                art.backward(loss, opt, parameters=net.parameters())
                functional.reset_net(net)
                last["loss"] = loss.detach()

            def infer():
                with torch.inference_mode(), art.autocast_context():
                    net(x)
                functional.reset_net(net)
            net.train()
            t_train = _arms.summary(_arms.time_cuda(train, a.warmup, a.steps))["median_ms"]
            torch.cuda.reset_peak_memory_stats()
            train()
            peak = torch.cuda.max_memory_allocated() / 2 ** 20
            net.eval()
            t_inf = _arms.summary(_arms.time_cuda(infer, a.warmup, a.inference_steps))["median_ms"]
            row = {"impl": a.impl, "precision": mode, "depth": a.depth, "train_ms": round(t_train, 3), "train_samples_per_s": round(a.batch_size / t_train * 1e3, 1),
                   "inference_ms": round(t_inf, 3), "train_peak_mb": round(peak, 1), "loss": round(float(last["loss"]), 4)}
        except Exception as exc:
            row = {"impl": a.impl, "precision": mode, "unavailable": f"{type(exc).__name__}: {exc}"[:200]}
        print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
