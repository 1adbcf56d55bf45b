#!/usr/bin/env python
"""Training step time and peak memory of a spiking MLP after ``memopt.memory_optimization`` at levels 0 - 4 (0 = no
rewrite).  Counterpart of the reference's ``benchmark/benchmark_memopt.py``: the same two toy models (a chain of
Linear + IF, and the same chain grouped into blocks that declare a spatial split), the same defaults (T 16, N 32, C 512).
``--impl reference`` runs the reference's pipeline on the same models.

    python benchmark/benchmark_memopt.py [--model-kind neuron|block] [--levels 0 1 2 3 4] [--impl ours|reference]
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


def build(arm, kind: str, C: int):
    neuron = arm.get("neuron")
    IF = lambda: neuron.IFNode(step_mode="m")
    if kind == "neuron":
        return nn.Sequential(nn.Linear(C, C), IF(), nn.Linear(C, C), IF(), nn.Linear(C, C), IF()), neuron.IFNode

    class Block(nn.Sequential):
        def __init__(self):
            super().__init__(nn.Linear(C, C), IF(), nn.Linear(C, C), IF())
            self.n_seq_inputs = self.n_outputs = 1

        def __spatial_split__(self):
            return [nn.Sequential(self[0], self[1]), nn.Sequential(self[2], self[3])]
    return nn.Sequential(*[Block() for _ in range(3)]), Block


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--model-kind", choices=("neuron", "block"), default="neuron")
    ap.add_argument("--T", type=int, default=16)
    ap.add_argument("--N", type=int, default=32)
    ap.add_argument("--C", type=int, default=512)
    ap.add_argument("--levels", type=int, nargs="+", default=[0, 1, 2, 3, 4])
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    try:
        arm = _arms.load(a.impl)
        functional, memopt = arm.get("functional"), arm.get("memopt")
    except Exception as exc:
        return _arms.unavailable(a.impl, exc)
    dev = torch.device("cuda")
    torch.manual_seed(0)
    base, instance = build(arm, a.model_kind, a.C)
    x = torch.rand(a.T, a.N, a.C, device=dev)

    def step(net):
        net.train()
        net.zero_grad(set_to_none=True)
        net(x).sum().backward()
        net.zero_grad(set_to_none=True)
        functional.reset_net(net)

    rows = []
    for level in a.levels:
        t0 = time.perf_counter()
        net = copy.deepcopy(base).cpu()
        if level > 0:
            net = memopt.memory_optimization(net, instance, dummy_input=(x.detach().cpu(),), compress_x=True, level=level)
        optimize_ms = (time.perf_counter() - t0) * 1e3
        net = net.to(dev)
        samples = _arms.time_cuda(lambda: step(net), a.warmup, a.iters)
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        step(net)
        torch.cuda.synchronize()
        row = {"impl": a.impl, "model_kind": a.model_kind, "T": a.T, "N": a.N, "C": a.C, "level": level, "optimize_ms": round(optimize_ms, 1),
               "peak_allocated_mb": round(torch.cuda.max_memory_allocated() / 2 ** 20, 2)}
        row.update({k: round(v, 4) for k, v in _arms.summary(samples).items()})
        rows.append(row)
        print(json.dumps(row), flush=True)
        del net
        torch.cuda.empty_cache()
    if a.out:
        Path(a.out).parent.mkdir(parents=True, exist_ok=True)
        with open(a.out, "a") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")


if __name__ == "__main__":
    main()
