#!/usr/bin/env python
"""A few SEW-ResNet-18 training steps (config: T = 16, 2 x 128 x 128 event frames, bf16) for use under a profiler:
``ncu --metrics gpu__time_duration.sum --clock-control none --profile-from-start off --csv python benchmark/profile_sew_step.py``
(one pass per launch; run the same command without ``ncu`` first).
Only the last step lies between cudaProfilerStart/Stop."""
import argparse
import sys
from pathlib import Path

import torch
import torch.nn.functional as F

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from benchmark.benchmark_sew_resnet import build  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("-T", type=int, default=16)
    ap.add_argument("--impl", default="ours")
    a = ap.parse_args()
    device = torch.device("cuda")
    torch.backends.cudnn.benchmark = True
    net, functional = build(a.impl, device)
    opt = torch.optim.AdamW(net.parameters(), lr=1e-4, fused=True)
    x = (torch.rand(a.T, a.batch, 2, 128, 128, device=device) < 0.05).float()
    y = torch.randint(0, 11, (a.batch,), device=device)

    def step():
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out = net(x)
        loss = F.cross_entropy(out.float().mean(0), y)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        functional.reset_net(net)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStart()
    step()
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    print("done")


if __name__ == "__main__":
    main()
