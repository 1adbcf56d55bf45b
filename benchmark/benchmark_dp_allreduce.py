#!/usr/bin/env python
"""The fused gradient all-reduce (``ops/csrc/comm_allreduce.cu``) in isolation and inside the Spikformer-8-512
data-parallel step, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29533 \
        benchmark/benchmark_dp_allreduce.py --out gpurun_out/dp_allreduce_n8.json

Part 1 — kernel alone: for each bucket size and each variant (wire fp32 / bf16, peer ld/st / multimem, block count) the
CUDA-event time of one launch (median of ``--iters``, max over ranks), the bytes one rank must send over NVLink
(``2 (world-1)/world x bucket``: reduce phase + broadcast phase) and that rate as a fraction of the link roofline
(``--link-gbs``, the measured peer-copy rate per direction).  These kernels wait on their peers, so they are timed
with events and algorithmic bytes, never replayed under a profiler.

Part 2 — exposed communication: the full training step with the exchange switched on against the same step inside
``no_sync()`` (no exchange at all), for each variant.  The difference is what the all-reduce costs after overlap.
"""
import argparse
import json
import os
import statistics
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.nn.functional as F

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from spikingjelly_b200.parallel.comm import SymmetricBucket  # noqa: E402
from spikingjelly_b200.parallel.data_parallel import SNNDataParallel  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--steps", type=int, default=15)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    ap.add_argument("--sizes-mb", type=float, nargs="+", default=[1.0, 8.0, 25.0])
    ap.add_argument("--skip-step", action="store_true")
    ap.add_argument("--out", default=None)
    a = ap.parse_args()

    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        raise SystemExit("run with torchrun on 2 or more GPUs")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    records = {"world": world, "link_gbs": a.link_gbs, "kernel": [], "step": []}

    def maxr(v):
        t = torch.tensor([v], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ------------------------------------------------------------------ part 1: the kernel alone
    probe = SymmetricBucket(1024, device)
    has_mc = probe.uses_multimem
    variants = [(w, m) for w in ("fp32", "bf16") for m in ((False, True) if has_mc else (False,))]
    for mb in a.sizes_mb:
        numel = int(mb * (1 << 20) / 4)
        for wire, mm in variants:
            for blocks in (4, 8, 16, 32):
                bucket = SymmetricBucket(numel, device, use_multimem=mm, wire=wire, blocks=blocks, timeout_s=20.0)
                bucket.buffer.normal_()
                times = []
                for it in range(a.iters + 3):
                    flush.zero_()
                    dist.barrier()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    bucket.all_reduce_(1.0 / world)
                    e1.record()
                    torch.cuda.synchronize()
                    if it >= 3:
                        times.append(e0.elapsed_time(e1) * 1e3)
                bucket.check()
                us = maxr(statistics.median(times))
                gbs = bucket.wire_bytes() / 2 / (us * 1e-6) / 1e9      # per direction: half of it is sent, half received per phase
                rec = {"mb": mb, "wire": wire, "multimem": mm, "blocks": blocks, "us": round(us, 1),
                       "wire_bytes_per_rank": bucket.wire_bytes(), "gbs_per_direction": round(gbs * 2, 1),
                       "fraction_of_link": round(gbs * 2 / a.link_gbs, 3)}
                records["kernel"].append(rec)
                if rank == 0:
                    print(json.dumps(rec), flush=True)
                del bucket

    # ------------------------------------------------------------------ part 2: inside the training step
    if not a.skip_step:
        from spikingjelly_b200.activation_based import functional
        from spikingjelly_b200.models import spikformer
        torch.manual_seed(1234 + rank)
        torch.backends.cudnn.benchmark = True
        net = spikformer.Spikformer(backend="cuda", T=4, in_channels=3, img_size_h=224, img_size_w=224, num_classes=1000,
                                    embed_dims=512, num_heads=8, mlp_ratio=4.0, depths=8).to(device)
        x = torch.randn(a.batch, 3, 224, 224, device=device)
        y = torch.randint(0, 1000, (a.batch,), device=device)

        def run(dp, opt, sync):
            def step():
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    out = dp(x)
                loss = F.cross_entropy(out.float().mean(0), y)
                opt.zero_grad(set_to_none=True)
                loss.backward()
                opt.step()
                functional.reset_net(net)
                flush.zero_()
            def loop(n):
                for _ in range(n):
                    if sync:
                        step()
                    else:
                        with dp.no_sync():
                            step()
            loop(a.warmup)
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            loop(a.steps)
            e1.record()
            dist.barrier()
            torch.cuda.synchronize()
            dp.check_communication()
            return maxr(e0.elapsed_time(e1) / a.steps)

        configs = [dict(wire="fp32", use_multimem=False)]
        if has_mc:
            configs += [dict(wire="fp32", use_multimem=True), dict(wire="bf16", use_multimem=True)]
        configs += [dict(wire="bf16", use_multimem=False)]
        for cfg in configs:
            dp = SNNDataParallel(net, timeout_s=60.0, **cfg)
            opt = torch.optim.AdamW(dp.parameters(), lr=1e-4, weight_decay=0.01, fused=True)
            ms_sync = run(dp, opt, True)
            ms_local = run(dp, opt, False)
            rec = dict(cfg, ms_per_step=round(ms_sync, 3), ms_per_step_no_sync=round(ms_local, 3),
                       exposed_ms=round(ms_sync - ms_local, 3), layout=dp.describe())
            records["step"].append(rec)
            if rank == 0:
                print(json.dumps({k: v for k, v in rec.items() if k != "layout"}), flush=True)
            dp.release()
            del dp, opt
    if rank == 0 and a.out:
        Path(a.out).parent.mkdir(parents=True, exist_ok=True)
        Path(a.out).write_text(json.dumps(records, indent=1))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
