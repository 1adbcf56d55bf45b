#!/usr/bin/env python
"""Parallel spiking neuron (PSN) forward + backward: the fused operator (``ops/psn.py``: one kernel per direction, the
pre-activation is never written) against the eager formulation (``addmm`` + surrogate), which is also what the reference
runs (``--impl reference`` times the reference's module).

    python benchmark/benchmark_psn.py [--impl ours|reference] [--out gpurun_out/psn.jsonl]

CUDA events, median of ``--iters`` after warm-up, a 256 MB write between samples; algorithmic traffic = read X + write S
(forward), read X, dS + write dX, dH (backward)."""
import argparse
import json
import statistics
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))
import _arms  # noqa: E402

SHAPES = [(4, 1 << 22), (8, 1 << 22), (16, 1 << 21), (32, 1 << 20)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    try:
        arm = _arms.load(a.impl)
        neuron = arm.get("neuron")
    except Exception as exc:
        return _arms.unavailable(a.impl, exc)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for dtype in (torch.bfloat16, torch.float32):
        for T, N in SHAPES:
            net = neuron.PSN(T).cuda()
            x = torch.randn(T, N, device="cuda", dtype=dtype, requires_grad=True)
            g = torch.randn(T, N, device="cuda", dtype=dtype)
            ctx = torch.autocast("cuda", dtype=torch.bfloat16, enabled=dtype == torch.bfloat16)

            def fwd():
                with ctx:
                    return net(x)

            def both():
                x.grad = None
                net.zero_grad(set_to_none=True)
                fwd().backward(g)
            f = statistics.median(_arms.time_cuda(fwd, 3, a.iters, flush=flush))
            fb = statistics.median(_arms.time_cuda(both, 3, a.iters, flush=flush))
            es = x.element_size()
            row = {"impl": a.impl, "T": T, "N": N, "dtype": str(dtype).removeprefix("torch."), "forward_us": round(f * 1e3, 1),
                   "forward_backward_us": round(fb * 1e3, 1), "forward_gbs": round(2 * T * N * es / f / 1e6, 1),
                   "forward_backward_gbs": round(6 * T * N * es / fb / 1e6, 1)}
            print(json.dumps(row), flush=True)
            if a.out:
                with open(a.out, "a") as fh:
                    fh.write(json.dumps(row) + "\n")


if __name__ == "__main__":
    main()
