#!/usr/bin/env python
"""One forward, one data-gradient and one weight-gradient launch of the implicit-GEMM convolution on a small case, for use
under a profiler (after a plain run of the same command):

    python benchmark/profile_conv.py --layer stem2 &&
    ncu --set full --clock-control none -k regex:gemm_kernel -s 3 -c 3 -o gpurun_out/prof_conv -f python benchmark/profile_conv.py --layer stem2

The case holds 8 images (tens of MB on the device); the first three ``gemm_kernel`` launches are a warm-up round.
Prints the CUDA-event time of each pass of the second round."""
import argparse
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from spikingjelly_b200 import ops  # noqa: E402

LAYERS = {"stem2": (64, 112, 128, 3, 1, 1), "stem3": (128, 56, 256, 3, 1, 1), "stem4": (256, 28, 512, 3, 1, 1),
          "layer1": (64, 32, 64, 3, 1, 1), "layer2s2": (64, 32, 128, 3, 2, 1)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layer", default="stem2", choices=sorted(LAYERS))
    ap.add_argument("--images", type=int, default=8)
    a = ap.parse_args()
    ops.require()
    ci, hw, co, k, s, p = LAYERS[a.layer]
    dev = torch.device("cuda")
    torch.manual_seed(0)
    x = (torch.rand(a.images, hw, hw, ci, device=dev) < 0.2).to(torch.bfloat16)
    w = (torch.randn(co, k, k, ci, device=dev) * 0.05).to(torch.bfloat16)
    o = (hw + 2 * p - k) // s + 1
    gy = torch.randn(a.images * o * o, co, device=dev, dtype=torch.bfloat16)
    st, pd, dl = [s, s], [p, p], [1, 1]
    for rnd in range(2):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        ev[0].record()
        torch.ops.sjb200.conv2d_nhwc_forward(x, w, st, pd, dl, True)
        ev[1].record()
        torch.ops.sjb200.conv2d_nhwc_dgrad(gy, w, hw, hw, st, pd)
        ev[2].record()
        torch.ops.sjb200.conv2d_nhwc_wgrad(x, gy, k, k, st, pd, dl)
        ev[3].record()
        torch.cuda.synchronize()
    print({"layer": a.layer, "images": a.images, "fwd_us": round(ev[0].elapsed_time(ev[1]) * 1e3, 1),
           "dgrad_us": round(ev[1].elapsed_time(ev[2]) * 1e3, 1), "wgrad_us": round(ev[2].elapsed_time(ev[3]) * 1e3, 1)})


if __name__ == "__main__":
    main()
