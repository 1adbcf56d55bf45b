#!/usr/bin/env python
"""Per-layer timing of the implicit-GEMM convolution (``ops/conv.py``) against cuDNN on the 3 x 3 / 1 x 1 convolutions of
SEW-ResNet-18 (T = 16, batch 32, 128 x 128 input) and of the Spikformer-8-512 stem (T = 4, batch 32, 224 x 224):

    python benchmark/benchmark_conv.py [--out gpurun_out/conv_layers.json] [--scale 1.0]

Each row: forward / data-gradient / weight-gradient time (CUDA events, median of --iters, a 256 MB write between launches
flushes L2), TFLOP/s of this framework's kernel and the ratio library time / own time (> 1: faster than cuDNN).  Both
sides get channels-last bf16 operands; the library side is ``F.conv2d`` and ``aten.convolution_backward`` with one output
mask at a time.
"""
import argparse
import json
import statistics
import sys
from pathlib import Path

import torch
import torch.nn.functional as F

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from spikingjelly_b200 import ops  # noqa: E402
from spikingjelly_b200.ops import gemm as G  # noqa: E402

# (name, images, C_in, H, W, C_out, k, stride, pad)
LAYERS = [
    ("sew.layer1 3x3 64->64 @32", 512, 64, 32, 32, 64, 3, 1, 1),
    ("sew.layer2.0 3x3s2 64->128 @32", 512, 64, 32, 32, 128, 3, 2, 1),
    ("sew.layer2 3x3 128->128 @16", 512, 128, 16, 16, 128, 3, 1, 1),
    ("sew.layer2.ds 1x1s2 64->128 @32", 512, 64, 32, 32, 128, 1, 2, 0),
    ("sew.layer3.0 3x3s2 128->256 @16", 512, 128, 16, 16, 256, 3, 2, 1),
    ("sew.layer3 3x3 256->256 @8", 512, 256, 8, 8, 256, 3, 1, 1),
    ("sew.layer4.0 3x3s2 256->512 @8", 512, 256, 8, 8, 512, 3, 2, 1),
    ("sew.layer4 3x3 512->512 @4", 512, 512, 4, 4, 512, 3, 1, 1),
    ("spikformer.stem2 3x3 64->128 @112", 128, 64, 112, 112, 128, 3, 1, 1),
    ("spikformer.stem3 3x3 128->256 @56", 128, 128, 56, 56, 256, 3, 1, 1),
    ("spikformer.stem4 3x3 256->512 @28", 128, 256, 28, 28, 512, 3, 1, 1),
    ("spikformer.pos 3x3 512->512 @14", 128, 512, 14, 14, 512, 3, 1, 1),
]


def timed(fn, flush, iters):
    ts = []
    for i in range(iters + 3):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        if i >= 3:
            ts.append(e0.elapsed_time(e1) * 1e3)
    return statistics.median(ts)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--scale", type=float, default=1.0, help="scales the number of images (small captures)")
    ap.add_argument("--only", default=None, help="substring of the layer name")
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    ops.require()
    dev = torch.device("cuda")
    torch.backends.cudnn.benchmark = True
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []
    for name, n, ci, h, w, co, k, s, p in LAYERS:
        if a.only and a.only not in name:
            continue
        n = max(1, int(n * a.scale))
        torch.manual_seed(0)
        x = (torch.rand(n, h, w, ci, device=dev) < 0.2).to(torch.bfloat16)
        wt = (torch.randn(co, ci, k, k, device=dev) * 0.05).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        w_krsc = wt.permute(0, 2, 3, 1).contiguous()
        x_nchw = x.permute(0, 3, 1, 2)
        oh, ow = (h + 2 * p - k) // s + 1, (w + 2 * p - k) // s + 1
        gy = torch.randn(n * oh * ow, co, device=dev, dtype=torch.bfloat16)
        gy_nchw = gy.view(n, oh, ow, co).permute(0, 3, 1, 2)
        flops = 2.0 * n * oh * ow * co * ci * k * k
        st, pd, dl = [s, s], [p, p], [1, 1]
        ours = {
            "fwd": lambda: torch.ops.sjb200.conv2d_nhwc_forward(x, w_krsc, st, pd, dl, True),
            "dgrad": lambda: torch.ops.sjb200.conv2d_nhwc_dgrad(gy, w_krsc, h, w, st, pd),
            "wgrad": lambda: torch.ops.sjb200.conv2d_nhwc_wgrad(x, gy, k, k, st, pd, dl),
        }
        lib = {
            "fwd": lambda: F.conv2d(x_nchw, wt, None, s, p),
            "dgrad": lambda: torch.ops.aten.convolution_backward(gy_nchw, x_nchw, wt, None, st, pd, dl, False, [0, 0], 1, [True, False, False]),
            "wgrad": lambda: torch.ops.aten.convolution_backward(gy_nchw, x_nchw, wt, None, st, pd, dl, False, [0, 0], 1, [False, True, False]),
        }
        rec = {"layer": name, "images": n, "gflop": round(flops / 1e9, 1)}
        for key in ("fwd", "dgrad", "wgrad"):
            t_own = timed(ours[key], flush, a.iters)
            G.check_status(x)
            t_lib = timed(lib[key], flush, a.iters)
            rec[key] = {"own_us": round(t_own, 1), "lib_us": round(t_lib, 1), "own_tflops": round(flops / t_own / 1e6, 1),
                        "lib_over_own": round(t_lib / t_own, 2)}
        rows.append(rec)
        print(json.dumps(rec), flush=True)
    if a.out:
        Path(a.out).parent.mkdir(parents=True, exist_ok=True)
        Path(a.out).write_text(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
