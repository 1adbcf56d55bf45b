#!/usr/bin/env python
"""Three launches of one tensor-core kernel on a case that exceeds L2 but holds well under 1 GB, for use under
``ncu --set full --clock-control none -k regex:<gemm_kernel|spike_gemm_kernel> -c 1``.  Prints the CUDA-event time of the last launch.

    python benchmark/profile_gemm.py --kind bf16|fp8|spike [--M 16384 --N 4096 --K 2048]
"""
import argparse
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from spikingjelly_b200 import ops  # noqa: E402
from spikingjelly_b200.ops import gemm as G  # noqa: E402
from spikingjelly_b200.parallel.fused_tp import pack_pitch  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kind", default="bf16")
    ap.add_argument("--M", type=int, default=16384)
    ap.add_argument("--N", type=int, default=4096)
    ap.add_argument("--K", type=int, default=2048)
    a = ap.parse_args()
    ops.require()
    dev = "cuda"
    M, N, K = a.M, a.N, a.K
    w = (torch.randn(N, K, device=dev) * 0.1).to(torch.bfloat16)
    if a.kind == "bf16":
        x = torch.randn(M, K, device=dev).to(torch.bfloat16)
        fn = lambda: G.gemm(x, w)
    elif a.kind == "fp8":
        from spikingjelly_b200.ops import fp8
        xq, xs = fp8.quantize(torch.randn(M, K, device=dev).to(torch.bfloat16))
        wq, wsc = fp8.quantize(w)
        alpha = (xs * wsc).reshape(1)
        fn = lambda: torch.ops.sjb200.gemm_fp8(xq, wq, alpha, False, 1)
    else:
        pitch = pack_pitch(K)
        bits = torch.randint(0, 256, (M, pitch), dtype=torch.uint8, device=dev)
        fn = lambda: torch.ops.sjb200.spike_gemm([bits.data_ptr()], pitch, M, K, w, M, M, 0, [], 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(3):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3
    print(f"{a.kind} M={M} N={N} K={K}: {us:.1f} us, {2.0 * M * N * K / us / 1e6:.0f} TFLOP/s")


if __name__ == "__main__":
    main()
