#!/usr/bin/env python
"""Fused tensor-parallel FFN sub-layer of the SNN-LLM shape (d 2048, FFN 5504, T 4) against the same sub-layer
built from library pieces: NCCL all-gather of bf16 spikes -> cuBLAS -> LIF -> cuBLAS -> NCCL reduce-scatter.

One process per GPU (torchrun); with one process the collectives vanish and the comparison is bit-operand
GEMM vs cuBLAS.  CUDA-event timing on the launching stream, L2 flushed between iterations, median per rank,
maximum over ranks.  The roofline line gives, per rank, max(FLOPs / measured bf16 peak, NVLink bytes / 770 GB/s).

    python benchmark/benchmark_tp_fused.py --tokens-per-rank 2048 [--out out/tp_fused.json]
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmark/benchmark_tp_fused.py ...
"""
import argparse
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from spikingjelly_b200 import ops  # noqa: E402
from spikingjelly_b200.parallel.fused_tp import FusedSpikingSubLayer, FusedTPWorkspace, pack_pitch  # noqa: E402


def timeit(fn, flush, iters, barrier):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2] * 1e3          # us


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens-per-rank", type=int, default=2048)
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--d-ffn", type=int, default=5504)
    ap.add_argument("--T", type=int, default=4)
    ap.add_argument("--iters", type=int, default=11)
    ap.add_argument("--out", default="")
    a = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ops.require()
    barrier = (lambda: dist.barrier()) if world > 1 else (lambda: None)

    T, tpr, d, F = a.T, a.tokens_per_rank, a.d_model, a.d_ffn
    tokens = tpr * world
    g = torch.Generator().manual_seed(0)
    h0 = (torch.randn(T, tokens, d, generator=g) * 2)[:, rank * tpr:(rank + 1) * tpr].contiguous().to(dev, torch.bfloat16)
    norm_w = (torch.rand(d, generator=g) + 1.5).to(dev)
    w1 = (torch.randn(F, d, generator=g) * 0.05)
    w2 = (torch.randn(d, F, generator=g) * 0.02)
    ws = FusedTPWorkspace(T=T, tokens_per_rank=tpr, d_model=d, device=dev)
    layer = FusedSpikingSubLayer(ws, norm_w, w1, w2)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    h = h0.clone()
    fused_us = timeit(lambda: layer(h), flush, a.iters, barrier)
    ws.check()

    # ---- the same sub-layer from library parts (same LIF/norm kernels, bf16 payloads, NCCL, cuBLAS)
    fpad = layer.f_pad
    w1p, w2p = layer.w1, layer.w2
    pu = pack_pitch(fpad)
    from spikingjelly_b200.activation_based import neuron
    lif_a = neuron.LIFNode(tau=2.0, step_mode="m", backend="cuda")
    lif_b = neuron.LIFNode(tau=2.0, step_mode="m", backend="cuda")
    nw16 = norm_w.to(torch.bfloat16)

    @torch.no_grad()
    def baseline():
        lif_a.reset()
        lif_b.reset()
        s_local = lif_a(torch.nn.functional.rms_norm(hb, (d,), nw16, 1e-6))
        if world > 1:
            s_all = torch.empty(world, T, tpr, d, dtype=torch.bfloat16, device=dev)
            dist.all_gather_into_tensor(s_all, s_local)
            s_all = s_all.permute(1, 0, 2, 3).reshape(T * tokens, d)
        else:
            s_all = s_local.reshape(T * tokens, d)
        u = s_all @ w1p.t()
        su = lif_b(u.view(T, tokens, fpad)).view(T * tokens, fpad)
        y = su @ w2p.t()                                             # [T*tokens, d] partial sums
        if world > 1:
            y = y.view(T, world, tpr, d).permute(1, 0, 2, 3).contiguous()
            mine = torch.empty(T, tpr, d, dtype=torch.bfloat16, device=dev)
            dist.reduce_scatter_tensor(mine, y)
        else:
            mine = y.view(T, tpr, d)
        hb.add_(mine)

    hb = h0.clone()
    base_us = timeit(baseline, flush, a.iters, barrier)

    # ---- kernels alone
    M = T * tokens
    up_us = timeit(lambda: torch.ops.sjb200.spike_gemm(ws.bits_ptrs, ws.x_pitch, M, d, w1p, tokens, tpr, rank, [], 0), flush, a.iters, barrier)
    lb = ws.local_bits(fpad)
    down_us = timeit(lambda: torch.ops.sjb200.spike_gemm([lb.data_ptr()], pu, M, fpad, w2p, tokens, tpr, rank, ws.stage_ptrs, ws.slot_elems),
                     flush, a.iters, barrier)
    xs = torch.randn(M, d, device=dev).to(torch.bfloat16)
    xu = torch.randn(M, fpad, device=dev).to(torch.bfloat16)
    cub_up = timeit(lambda: xs @ w1p.t(), flush, a.iters, barrier)
    cub_down = timeit(lambda: xu @ w2p.t(), flush, a.iters, barrier)
    ws.check()

    vals = torch.tensor([fused_us, base_us, up_us, down_us, cub_up, cub_down], device=dev)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    fused_us, base_us, up_us, down_us, cub_up, cub_down = vals.tolist()
    if rank == 0:
        peaks = {}
        pk = Path(__file__).resolve().parents[1] / "MEASURED_PEAKS.json"
        if pk.exists():
            peaks = json.loads(pk.read_text())
        tflops_peak = float(peaks.get("bf16_tflops", 1590.0))
        flops = 2.0 * M * d * fpad * 2
        nv_bytes = (world - 1) / world * (M * d / 8 + M * d * 2) if world > 1 else 0.0     # bits in, bf16 partials out
        t_flops = flops / (tflops_peak * 1e12) * 1e6
        t_link = nv_bytes / 770e9 * 1e6
        rec = {
            "world": world, "T": T, "tokens_per_rank": tpr, "d_model": d, "d_ffn": F, "f_local_padded": fpad,
            "fused_sublayer_us": round(fused_us, 1), "library_sublayer_us": round(base_us, 1),
            "speedup": round(base_us / fused_us, 2),
            "spike_gemm_up_us": round(up_us, 1), "cublas_up_us": round(cub_up, 1),
            "spike_gemm_down_push_us": round(down_us, 1), "cublas_down_us": round(cub_down, 1),
            "up_tflops": round(2.0 * M * d * fpad / up_us / 1e6, 1), "down_tflops": round(2.0 * M * d * fpad / down_us / 1e6, 1),
            "roofline_us": round(max(t_flops, t_link), 1), "roofline_bound": "nvlink" if t_link > t_flops else "tensor",
            "frac_of_roofline_gemms_only": round(max(t_flops, t_link) / (up_us + down_us), 3),
            "peak_source": "measured" if peaks else "fallback",
        }
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
