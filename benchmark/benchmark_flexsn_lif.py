#!/usr/bin/env python
"""A LIF neuron written as a FlexSN step function against the built-in LIF kernel, forward + backward (counterpart of the
reference's ``benchmark/flexsn/benchmark_flexsn_lif.py``): how close the generated kernel comes to the hand-written one.
``--impl reference`` runs the reference's FlexSN (Triton template) against its built-in Triton LIF.

    python benchmark/benchmark_flexsn_lif.py [--T 16 --numel 1048576] [--impl ours|reference]
"""
import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))
import _arms  # noqa: E402


def lif_core(x: torch.Tensor, v: torch.Tensor):
    h = v + (x - v) * 0.5
    s = (h >= 1.0).to(h.dtype)
    return s, h * (1.0 - s)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--T", type=int, default=16)
    ap.add_argument("--numel", type=int, default=1 << 20)
    ap.add_argument("--iters", type=int, default=30)
    a = ap.parse_args()
    try:
        arm = _arms.load(a.impl)
        neuron, surrogate = arm.get("neuron"), arm.get("surrogate")
    except Exception as exc:
        return _arms.unavailable(a.impl, exc)
    sg = surrogate.Sigmoid()

    def core(x, v):                              # the spike goes through the surrogate so that backward exists
        h = v + (x - v) * 0.5
        s = sg(h - 1.0)
        return s, h * (1.0 - s)
    x = torch.randn(a.T, a.numel, device="cuda", requires_grad=True)
    g = torch.randn(a.T, a.numel, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    rows = {}
    for name, make in (("builtin_lif", lambda: neuron.LIFNode(tau=2.0, surrogate_function=sg, step_mode="m", backend=arm.fast_backend)),
                       ("flexsn_lif", lambda: neuron.FlexSN(core=core, num_inputs=1, num_states=1, num_outputs=1, step_mode="m", backend=arm.fast_backend))):
        try:
            node = make().cuda()

            def step():
                node.reset()
                x.grad = None
                out = node(x)
                (out[0] if isinstance(out, (tuple, list)) else out).backward(g)
            rows[name] = round(_arms.summary(_arms.time_cuda(step, 5, a.iters, flush=flush))["median_ms"] * 1e3, 1)
        except Exception as exc:
            rows[name] = f"{type(exc).__name__}: {exc}"[:160]
    out = {"impl": a.impl, "backend": arm.fast_backend, "T": a.T, "numel": a.numel, "forward_backward_us": rows}
    if all(isinstance(v, float) for v in rows.values()):
        out["generated_over_builtin"] = round(rows["flexsn_lif"] / rows["builtin_lif"], 2)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
