#!/usr/bin/env python
"""tcgen05 GEMM against torch.matmul (cuBLAS) on the linear-layer shapes of Spikformer-8-512
(forward, dgrad, wgrad) and on a large square problem.  CUDA-event timing, L2 flushed between
iterations, median of `--iters`.

    python benchmark/benchmark_gemm.py [--out out/gemm.json] [--only NAME]
"""
import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from spikingjelly_b200.ops import gemm as G  # noqa: E402


def timeit(fn, flush, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2] * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--iters", type=int, default=11)
    ap.add_argument("--only", default="")
    ap.add_argument("--pair", type=int, default=-1, help="1 / 0: force the two-CTA (cta_group::2) kernel on / off; -1: library default")
    a = ap.parse_args()
    dev = "cuda"
    G.require()
    if a.pair >= 0:
        torch.ops.sjb200.gemm_set_pair_mode(a.pair)
    M = 4 * 32 * 196
    shapes = [("qkv_fwd", M, 1536, 512), ("proj_fwd", M, 512, 512), ("fc1_fwd", M, 2048, 512), ("fc2_fwd", M, 512, 2048),
              ("n128", M, 128, 2048), ("square8k", 8192, 8192, 8192)]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []
    for name, m, n, k in shapes:
        if a.only and a.only != name:
            continue
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        w = torch.randn(n, k, device=dev).to(torch.bfloat16)
        gy = torch.randn(m, n, device=dev).to(torch.bfloat16)
        flops = 2.0 * m * n * k
        cases = {
            "fwd": (lambda: G.gemm(x, w), lambda: x @ w.t()),
            "dgrad": (lambda: G.gemm(gy, w, False, True), lambda: gy @ w),
            "wgrad": (lambda: G.gemm(gy, x, True, True), lambda: gy.t() @ x),
        }
        for cname, (ours, ref) in cases.items():
            t_o = timeit(ours, flush, a.iters)
            t_r = timeit(ref, flush, a.iters)
            row = {"pair": a.pair, "shape": name, "op": cname, "M": m, "N": n, "K": k, "ours_us": round(t_o, 1), "cublas_us": round(t_r, 1),
                   "ours_tflops": round(flops / t_o / 1e6, 1), "cublas_tflops": round(flops / t_r / 1e6, 1)}
            print(json.dumps(row), flush=True)
            rows.append(row)
        # fp8 forward (e4m3 x e4m3 -> bf16) against torch._scaled_mm (cuBLASLt fp8)
        from spikingjelly_b200.ops import fp8
        xq, wq = x.to(torch.float8_e4m3fn), w.to(torch.float8_e4m3fn)
        one = torch.ones(1, device=dev)
        t_o = timeit(lambda: fp8.matmul_nt(xq, wq, one), flush, a.iters)
        try:
            t_r = timeit(lambda: torch._scaled_mm(xq, wq.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16), flush, a.iters)
        except Exception:
            t_r = float("nan")
        row = {"shape": name, "op": "fwd_fp8", "M": m, "N": n, "K": k, "ours_us": round(t_o, 1), "cublas_us": round(t_r, 1),
               "ours_tflops": round(flops / t_o / 1e6, 1), "cublas_tflops": round(flops / t_r / 1e6, 1)}
        print(json.dumps(row), flush=True)
        rows.append(row)
        G.check_status(x)
    if a.out:
        Path(a.out).parent.mkdir(parents=True, exist_ok=True)
        Path(a.out).write_text(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
