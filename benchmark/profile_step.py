#!/usr/bin/env python
"""One Spikformer-8-512 training step inside a cudaProfilerStart/Stop range, for a kernel
launch list:

    ncu --metrics gpu__time_duration.sum --clock-control none --profile-from-start off \
        --csv --log-file launches.csv python benchmark/profile_step.py

(compare SHARES of device time between kernels; absolute times under a profiler are not
benchmark numbers)."""
import argparse
import sys
from pathlib import Path

import torch
import torch.nn.functional as F

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from spikingjelly_b200.activation_based import functional  # noqa: E402
from spikingjelly_b200.models import spikformer  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--modular", action="store_true", help="module-by-module path instead of the fused schedule")
    a = ap.parse_args()
    dev = torch.device("cuda")
    torch.manual_seed(0)
    torch.backends.cudnn.benchmark = True
    net = spikformer.spikformer_8_512(backend="cuda").to(dev)
    net.fused = not a.modular
    opt = torch.optim.AdamW(net.parameters(), lr=1e-4, fused=True)
    x = torch.randn(a.batch, 3, 224, 224, device=dev)
    y = torch.randint(0, 1000, (a.batch,), device=dev)

    def step():
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out = net(x)
        loss = F.cross_entropy(out.float().mean(0), y)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        functional.reset_net(net)

    for _ in range(a.warmup):
        step()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print("done")


if __name__ == "__main__":
    main()
