#!/usr/bin/env python
"""SpikeZIP ternary IF neuron (``STBIFNeuron``): a Python loop of single steps against the multi-step call, outputs and
final states compared.  Counterpart of the reference's ``benchmark/benchmark_ann2snn_spikezip_stbif.py`` (its columns:
old loop, ``torch`` multi-step, ``triton`` multi-step; here: loop, eager multi-step on CPU, compiled kernel on CUDA).

    python benchmark/benchmark_ann2snn_spikezip_stbif.py [--impl ours|reference] [--time-steps 64 --numel 1048576]
"""
import argparse
import json
import sys
import time
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))
import _arms  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--time-steps", type=int, default=64)
    ap.add_argument("--numel", type=int, default=1 << 20)
    ap.add_argument("--dtype", choices=("float32", "float16"), default="float32")
    ap.add_argument("--level", type=int, default=32)
    ap.add_argument("--scale", type=float, default=0.25)
    ap.add_argument("--sym", action="store_true")
    ap.add_argument("--repeat", type=int, default=10)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()
    try:
        arm = _arms.load(a.impl)
        functional, STBIFNeuron = arm.get("functional"), arm.get("neuron").STBIFNeuron
    except Exception as exc:
        return _arms.unavailable(a.impl, exc)
    dev = torch.device(a.device)
    dtype = getattr(torch, a.dtype)
    g = torch.Generator().manual_seed(a.seed)
    x = (torch.randn(a.numel, generator=g) * a.scale * 2).to(dev, dtype)
    x_seq = torch.zeros(a.time_steps, a.numel, device=dev, dtype=dtype)
    x_seq[0] = x                                          # the value arrives once; the neuron spends T steps emitting it
    sync = (lambda: torch.cuda.synchronize(dev)) if dev.type == "cuda" else (lambda: None)

    def best(fn):
        times, res = [], None
        for _ in range(a.repeat):
            sync()
            t0 = time.perf_counter()
            res = fn()
            sync()
            times.append(time.perf_counter() - t0)
        return min(times), res

    def state(n):
        return {k: getattr(n, k).detach().clone() for k in ("q", "acc_q", "cur_output")}

    def loop(n):
        functional.reset_net(n)
        return torch.stack([n.single_step_forward(xt) for xt in x_seq])

    def multi(n):
        functional.reset_net(n)
        return n(x_seq)

    out = {"impl": a.impl, "device": str(dev), "dtype": a.dtype, "time_steps": a.time_steps, "numel": a.numel, "level": a.level,
           "scale": a.scale, "sym": a.sym}
    with torch.inference_mode():
        ref = STBIFNeuron(a.scale, level=a.level, sym=a.sym).to(dev)
        t_loop, y_loop = best(lambda: loop(ref))
        s_loop = state(ref)
        out["loop_ms"] = round(t_loop * 1e3, 3)
        backends = ["torch"] + (["triton"] if a.impl == "reference" and dev.type == "cuda" and arm.fast_backend == "triton" else [])
        if a.impl == "ours":
            backends = ["cuda" if dev.type == "cuda" else "torch"]
        for backend in backends:
            n = STBIFNeuron(a.scale, level=a.level, sym=a.sym).to(dev)
            functional.set_step_mode(n, "m")
            n.backend = backend
            multi(n)                                      # builds / compiles outside the timed region
            t, y = best(lambda: multi(n))
            s = state(n)
            out[f"{backend}_ms"] = round(t * 1e3, 3)
            out[f"{backend}_speedup_vs_loop"] = round(t_loop / t, 2)
            out[f"{backend}_max_abs_diff"] = float((y.float() - y_loop.float()).abs().max())
            out[f"{backend}_state_max_abs_diff"] = max(float((s[k].float() - s_loop[k].float()).abs().max()) for k in s)
    # the time-summed output is the quantised input
    want = torch.clamp(torch.floor(x.float() / a.scale + 0.5), float(ref.neg_min), float(ref.pos_max)) * a.scale
    out["sum_equals_quantiser"] = bool(torch.allclose(y_loop.float().sum(0), want, atol=1e-3)) if a.time_steps >= a.level else None
    print(json.dumps(out))


if __name__ == "__main__":
    main()
