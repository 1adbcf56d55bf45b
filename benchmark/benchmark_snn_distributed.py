#!/usr/bin/env python
"""Weak-scaling training throughput of the two networks whose numbers the reference publishes for its own
``benchmark/benchmark_snn_distributed.py`` (CIFAR10-DVS VGG at per-rank batch 16, T = 10, 2 x 48 x 48 frames; Spikformer-Ti
at per-rank batch 16, T = 8, 224 x 224 images), in the modes ``none`` / ``dp`` / ``tp`` / ``fsdp2`` / ``fsdp2_tp``.

    python benchmark/benchmark_snn_distributed.py --model cifar10dvs_vgg --mode none
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmark/benchmark_snn_distributed.py --model spikformer_ti --mode dp
    ... --impl reference      # the unmodified reference (baseline/_ref) on the same step, modes none and dp

fp32 parameters and activations unless ``--amp`` (the published numbers are fp32).  CUDA events around ``--steps`` steps after
``--warmup``, 256 MB L2 flush inside every step, max over ranks; one JSON line on rank 0 with step time, global samples/s and
peak allocated memory, next to the published RTX 4090 figure for the same row where there is one.
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

# published by the reference for 7 x RTX 4090 (step ms, global samples/s): docs/source/tutorials/en/distributed_training.rst:365-565
PUBLISHED = {("cifar10dvs_vgg", "none", 1): (38.34, 417.36), ("cifar10dvs_vgg", "dp", 2): (39.34, 813.40),
             ("cifar10dvs_vgg", "tp", 2): (85.71, 186.69), ("cifar10dvs_vgg", "fsdp2", 2): (47.88, 668.31),
             ("spikformer_ti", "none", 1): (85.54, 187.04), ("spikformer_ti", "dp", 2): (87.62, 365.22),
             ("spikformer_ti", "tp", 2): (197.99, 80.81), ("spikformer_ti", "fsdp2", 2): (91.82, 348.51)}


def build(args, device, world, local_rank):
    if args.impl == "reference":
        sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
        from spikingjelly.activation_based import functional
        from spikingjelly.activation_based.model import spikformer
        if args.model == "cifar10dvs_vgg":
            from spikingjelly.activation_based.examples.memopt.models import CIFAR10DVSVGG
            net = CIFAR10DVSVGG(dropout=0.0, backend=args.backend or "triton").to(device)
        else:
            net = spikformer.__dict__[args.model](T=args.T, img_size_h=args.image_size, img_size_w=args.image_size,
                                                  num_classes=args.num_classes, backend=args.backend or "triton").to(device)
        if args.mode == "dp":
            from spikingjelly.activation_based.distributed.data_parallel import prepare_snn_data_parallel
            net = prepare_snn_data_parallel(net, device_ids=[local_rank])
        elif args.mode != "none":
            raise SystemExit("the reference arm of this script covers modes none and dp")
        return net, functional, torch.optim.AdamW(net.parameters(), lr=1e-3), (lambda o: o)
    from spikingjelly_b200 import ops
    from spikingjelly_b200.activation_based import distributed as D
    from spikingjelly_b200.activation_based import functional
    from spikingjelly_b200.models import spikformer
    ops.require()
    backend = args.backend or "cuda"
    if args.model == "cifar10dvs_vgg":
        from spikingjelly_b200.activation_based.examples.memopt.models import CIFAR10DVSVGG
        net = CIFAR10DVSVGG(dropout=0.0, backend=backend).to(device)
        roots = dict(tensor_parallel_roots=("classifier",), conv_tensor_parallel_roots=("features",))
    else:
        net = spikformer.__dict__[args.model](T=args.T, img_size_h=args.image_size, img_size_w=args.image_size,
                                              num_classes=args.num_classes, backend=backend).to(device)
        roots = dict(tensor_parallel_roots=("head",))
    if args.mode == "none":
        return net, functional, torch.optim.AdamW(net.parameters(), lr=1e-3), (lambda o: o)
    cfg = D.SNNDistributedConfig(mode=args.mode, device_type="cuda", mesh_shape=tuple(args.mesh_shape) if args.mesh_shape else None, **roots)
    net, _, _ = D.configure_snn_distributed(net, cfg)
    opt = D.build_snn_optimizer(net, args.mode, lr=1e-3, weight_decay=0.0, optimizer_sharding=args.optimizer_sharding)
    return net, functional, opt, getattr(D, "materialize_dtensor_output", lambda o: o)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="cifar10dvs_vgg", choices=["cifar10dvs_vgg", "spikformer_ti", "spikformer_s"])
    ap.add_argument("--mode", default="none", choices=["none", "dp", "tp", "fsdp2", "fsdp2_tp"])
    ap.add_argument("--batch-size", type=int, default=16, help="per rank")
    ap.add_argument("--T", type=int, default=0, help="0: 10 for the VGG, 8 for the Spikformers (the published settings)")
    ap.add_argument("--image-size", type=int, default=224)
    ap.add_argument("--num-classes", type=int, default=1000)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--backend", default="")
    ap.add_argument("--amp", action="store_true")
    ap.add_argument("--mesh-shape", type=int, nargs="*", default=None)
    ap.add_argument("--optimizer-sharding", default="none", choices=["none", "zero"])
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    a.T = a.T or (10 if a.model == "cifar10dvs_vgg" else 8)
    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    if a.mode == "none" and world > 1:
        raise SystemExit("mode none is a single-process measurement")
    torch.manual_seed(1234 + rank)
    torch.backends.cudnn.benchmark = True
    net, functional, opt, materialize = build(a, device, world, local)
    B = a.batch_size
    if a.model == "cifar10dvs_vgg":
        x, y = torch.randn(B, a.T, 2, 48, 48, device=device), torch.randint(0, 10, (B,), device=device)
    else:
        x, y = torch.randn(B, 3, a.image_size, a.image_size, device=device), torch.randint(0, a.num_classes, (B,), device=device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def step():
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=a.amp):
            out = materialize(net(x))
        out = out.float()
        loss = F.cross_entropy(out.mean(0) if out.dim() == 3 else out, y)
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
    torch.cuda.reset_peak_memory_stats()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    barrier()
    if hasattr(net, "check_communication"):
        net.check_communication()          # a timed-out gradient exchange must not be reported as throughput
    t = torch.tensor([e0.elapsed_time(e1) / a.steps, torch.cuda.max_memory_allocated() / 2 ** 20], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms, mb = t.tolist()
        # ranks of one tensor-parallel group work on the SAME samples: only the data-parallel replicas multiply the batch
        if a.mode == "tp":
            replicas = 1
        elif a.mode == "fsdp2_tp":
            replicas = (a.mesh_shape[0] if a.mesh_shape else max(1, world // 2))
        else:
            replicas = world
        rec = {"impl": a.impl, "model": a.model, "mode": a.mode, "n_gpus": world, "per_rank_batch": B, "T": a.T,
               "dtype": "bf16 autocast" if a.amp else "fp32", "step_ms": round(ms, 2), "samples_per_s": round(replicas * B / ms * 1e3, 1),
               "peak_allocated_mb": round(mb, 1), "last_loss": round(float(loss), 4)}
        pub = PUBLISHED.get((a.model, a.mode, world))
        if pub and B == 16:
            rec["published_rtx4090"] = {"step_ms": pub[0], "samples_per_s": pub[1]}
            rec["vs_published"] = round(rec["samples_per_s"] / pub[1], 2)
        line = json.dumps(rec)
        print(line)
        if a.out:
            Path(a.out).parent.mkdir(parents=True, exist_ok=True)
            with open(a.out, "a") as f:
                f.write(line + "\n")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
