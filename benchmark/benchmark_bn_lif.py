#!/usr/bin/env python
"""Device time of the fused BatchNorm+LIF kernels (forward, backward) on Spikformer-sized
activations [T, B*L, C], against the algorithmic HBM traffic.

    python benchmark/benchmark_bn_lif.py [--batch 32] [--out file.json]

Timed with CUDA events after warm-up; a 256 MB buffer is rewritten between iterations so that
every iteration starts with a cold L2.
"""
import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from spikingjelly_b200.ops import bn_lif as B  # noqa: E402
from spikingjelly_b200.ops.neuron_scan import KIND, NeuronSpec  # noqa: E402


def timed(fn, flush, iters=20, warmup=5):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters * 1e3      # us


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--T", type=int, default=4)
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    dev = torch.device("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    peaks = json.loads(Path(__file__).resolve().parents[1].joinpath("MEASURED_PEAKS.json").read_text()) \
        if Path(__file__).resolve().parents[1].joinpath("MEASURED_PEAKS.json").exists() else {}
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    rows = a.batch * 196
    results = []
    for C in (512, 1536, 2048):
        y = torch.randn(a.T, rows, C, device=dev, dtype=torch.bfloat16, requires_grad=True)
        bn = torch.nn.BatchNorm1d(C).to(dev).train()
        spec = NeuronSpec(kind=KIND["lif_di"], v_threshold=1.0, v_reset=0.0, tau=2.0, sg=(0, 4.0, 0.0), detach_reset=True)
        call = lambda: B.bn_lif(y, bn, spec)
        out = call()
        g = torch.randn_like(out)
        n_bytes = y.numel() * 2
        t_f = timed(call, flush)
        def bwd():
            y.grad = None
            o = call()
            o.backward(g)
        t_fb = timed(bwd, flush)
        t_b = t_fb - t_f
        rec = {"C": C, "rows": rows, "T": a.T, "fwd_us": round(t_f, 1), "bwd_us": round(t_b, 1),
               # forward: stats read + apply read + spike write = 3 passes; backward: (y, g) -> gx, (gx, y) -> dy = 6 passes
               "fwd_frac_of_measured_hbm": round(3 * n_bytes / (t_f * 1e-6) / 1e9 / hbm, 3),
               "bwd_frac_of_measured_hbm": round(6 * n_bytes / (t_b * 1e-6) / 1e9 / hbm, 3)}
        print(json.dumps(rec))
        results.append(rec)
    if a.out:
        Path(a.out).write_text(json.dumps(results, indent=1))


if __name__ == "__main__":
    main()
