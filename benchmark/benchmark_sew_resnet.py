#!/usr/bin/env python
"""SEW-ResNet-18 (ADD, multi-step LIF tau 2, ATan) training throughput on synthetic event frames
[T = 16, B = 32 per GPU, 2 polarity channels, 128 x 128], 11 classes, bf16 autocast, AdamW, data parallel.

    python benchmark/benchmark_sew_resnet.py [--impl reference] [--steps 10 --warmup 3]
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmark/benchmark_sew_resnet.py

CUDA-event timing, 256 MB L2 flush inside every step, max over ranks; one JSON line on rank 0.  The reference's
``sew_resnet18`` hard-codes 3 input channels, so for that arm the first convolution is replaced by a 2-channel one.
"""
import argparse
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.nn.functional as F

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def build(impl: str, device):
    if impl == "reference":
        sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
        from spikingjelly.activation_based import functional, layer, neuron, surrogate
        from spikingjelly.activation_based.model import sew_resnet
        net = sew_resnet.sew_resnet18(num_classes=11, cnf="ADD", spiking_neuron=neuron.LIFNode, tau=2.0, detach_reset=True,
                                      surrogate_function=surrogate.ATan())
        net.conv1 = layer.Conv2d(2, 64, kernel_size=7, stride=2, padding=3, bias=False)
        functional.set_step_mode(net, "m")
        functional.set_backend(net, "triton", instance=neuron.LIFNode)
        return net.to(device), functional
    from spikingjelly_b200 import ops
    from spikingjelly_b200.activation_based import functional, neuron, surrogate
    from spikingjelly_b200.models import sew_resnet
    ops.require()
    net = sew_resnet.sew_resnet18(num_classes=11, cnf="ADD", spiking_neuron=neuron.LIFNode, tau=2.0, detach_reset=True,
                                  surrogate_function=surrogate.ATan(), in_channels=2)
    functional.set_step_mode(net, "m")
    functional.set_backend(net, "cuda", instance=neuron.LIFNode)
    return net.to(device), functional


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("-T", type=int, default=16)
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    torch.manual_seed(1 + rank)
    torch.backends.cudnn.benchmark = True
    net, functional = build(a.impl, device)
    model = net
    if world > 1:
        if a.impl == "reference":
            model = torch.nn.parallel.DistributedDataParallel(net, device_ids=[local])
        else:
            from spikingjelly_b200.parallel import data_parallel
            model = data_parallel.prepare_snn_data_parallel(net, device_ids=[local])
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, fused=True)
    x = (torch.poisson(torch.full((a.T, a.batch, 2, 128, 128), 0.05, device=device)) > 0).float()
    y = torch.randint(0, 11, (a.batch,), device=device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def step():
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out = model(x)
        loss = F.cross_entropy(out.float().mean(0), y)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        functional.reset_net(net)
        flush.zero_()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(a.warmup):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    barrier()
    if hasattr(model, "check_communication"):
        model.check_communication()          # a timed-out gradient exchange must not be reported as throughput
    t = torch.tensor([e0.elapsed_time(e1)], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms = t.item() / a.steps
        rec = {"config": "SEW-ResNet-18 ADD, T=16, 2x128x128, bf16, dp%d" % world, "impl": a.impl, "n_gpus": world,
               "per_gpu_batch": a.batch, "ms_per_step": round(ms, 3), "samples_per_s": round(world * a.batch / ms * 1e3, 1),
               "last_loss": round(float(loss), 4), "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 2)}
        line = json.dumps(rec)
        print(line)
        if a.out:
            with open(a.out, "a") as f:
                f.write(line + "\n")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
