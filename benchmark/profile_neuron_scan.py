#!/usr/bin/env python
"""A few forward+backward launches of the multi-step LIF kernels on one tensor, for use
under a profiler: ``ncu --set full --clock-control none -k regex:scan_ -c 2 python benchmark/profile_neuron_scan.py --logN 22``
(a small case: one kernel, two launches, well under 1 GB on the device).
Prints CUDA-event times of the isolated forward and backward kernels (median of `--iters`)."""
import argparse
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from spikingjelly_b200.ops.neuron_scan import KIND, NeuronSpec  # noqa: E402
from spikingjelly_b200 import ops  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--T", type=int, default=4)
    ap.add_argument("--logN", type=int, default=24)
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args()
    ops.require()
    dt = {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}[a.dtype]
    N = 1 << a.logN
    x = (torch.randn(a.T, N, device="cuda") + 0.5).to(dt)
    g = torch.randn(a.T, N, device="cuda").to(dt)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    fwd, bwd = [], []
    for _ in range(a.iters):
        flush.zero_()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        e[0].record()
        outs = torch.ops.sjb200.scan_forward(x, None, 0.0, None, KIND["lif_di"], 2.0, 0.0, 0.0, 0.0, 1.0, 0.0, False,
                                             False, False, True)
        e[1].record()
        flush.zero_()
        e[2].record()
        torch.ops.sjb200.scan_backward(g, None, None, x, None, 0.0, None, outs[4] if outs[4].numel() else None,
                                       KIND["lif_di"], 2.0, 0.0, 0.0, 0.0, 1.0, 0.0, False, 1, 2.0, 0.0, False, False)
        e[3].record()
        torch.cuda.synchronize()
        fwd.append(e[0].elapsed_time(e[1]))
        bwd.append(e[2].elapsed_time(e[3]))
    fwd.sort(); bwd.sort()
    es = x.element_size()
    f, b = fwd[len(fwd) // 2] * 1e3, bwd[len(bwd) // 2] * 1e3
    print(f"T={a.T} N=2^{a.logN} {a.dtype}: forward {f:.1f} us ({2 * a.T * N * es / f / 1e3:.0f} GB/s), "
          f"backward {b:.1f} us ({3 * a.T * N * es / b / 1e3:.0f} GB/s)")


if __name__ == "__main__":
    main()
