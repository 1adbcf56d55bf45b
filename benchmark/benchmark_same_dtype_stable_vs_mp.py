#!/usr/bin/env python
"""The plain functional neurons (``multistep_if`` / ``multistep_lif`` / ``multistep_plif``) against their mixed-precision
forms called with a prepared plan whose storage, compute and spike dtype all equal the input dtype: inference forward and
training forward + backward, per size and dtype.  Counterpart of the reference's
``benchmark/benchmark_same_dtype_stable_vs_mp.py`` (there the two forms are different Triton kernels; here both names reach
the same CUDA scan kernel, so the table is a check that the plan form costs nothing extra).

    python benchmark/benchmark_same_dtype_stable_vs_mp.py [--sizes 32x4096,64x65536,256x65536,1024x65536] [--impl ours|reference]
"""
import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))
import _arms  # noqa: E402

R_TAU = 0.5


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--sizes", default="32x4096,64x65536,256x65536,1024x65536")
    ap.add_argument("--neurons", nargs="+", default=["if", "lif", "plif"])
    ap.add_argument("--dtypes", nargs="+", default=["fp32", "fp16", "bf16"])
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--repeats", type=int, default=10)
    ap.add_argument("--out", default=None, help="also write all rows to this JSON file")
    a = ap.parse_args()
    try:
        arm = _arms.load(a.impl)
        sg = arm.get("surrogate").Sigmoid()
        K = arm.get("triton_kernel.neuron_kernel")
        KI, KL, KP, KU = (arm.get(f"triton_kernel.neuron_kernel.{m}") for m in ("integrate_and_fire", "lif", "plif", "utils"))
        del K
    except Exception as exc:
        return _arms.unavailable(a.impl, exc)
    dev = torch.device("cuda", 0)
    table = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}

    def stable(kind, x, v, r):
        if kind == "if":
            return KI.multistep_if(x, v, 1.0, 0.0, False, sg)
        if kind == "lif":
            return KL.multistep_lif(x, v, True, 2.0, 1.0, 0.0, False, sg)
        return KP.multistep_plif(x, v, r, True, 1.0, 0.0, False, sg)

    def mixed(kind, x, v, r, plan):
        if kind == "if":
            return KI.multistep_if_mp_with_plan(x, v, plan, v_threshold=1.0, v_reset=0.0)
        if kind == "lif":
            return KL.multistep_lif_mp_with_plan(x, v, plan, decay_input=True, tau=2.0, v_threshold=1.0, v_reset=0.0)
        return KP.multistep_plif_mp_with_plan(x, v, r, plan, decay_input=True, v_threshold=1.0, v_reset=0.0)
    rows = []
    for size in a.sizes.split(","):
        T, N = (int(p) for p in size.lower().split("x"))
        for kind in a.neurons:
            for name in a.dtypes:
                dt = table[name]
                torch.manual_seed(0)
                x = torch.randn(T, N, device=dev).to(dt)
                for process in ("inference_forward", "training_forward_backward"):
                    train = process.startswith("training")
                    row = {"impl": a.impl, "T": T, "N": N, "neuron": kind, "dtype": name, "process": process}
                    try:
                        plan = KU.prepare_triton_neuron_execution_plan(neuron_type=kind, device=dev, storage_dtype=dt, forward_compute_dtype=name,
                                                                       backward_compute_dtype=name, spike_dtype=dt, save_intermediates=train)
                        xr = x.detach().clone().requires_grad_(train)
                        v = torch.zeros(N, device=dev, dtype=dt, requires_grad=train)
                        r = torch.tensor(R_TAU, device=dev, dtype=dt, requires_grad=train and kind == "plif")
                        for variant in ("stable", "mp"):
                            def fn():
                                xr.grad = v.grad = r.grad = None
                                with torch.set_grad_enabled(train):
                                    out = stable(kind, xr, v, r) if variant == "stable" else mixed(kind, xr, v, r, plan)
                                    if train:
                                        (out[0].float().sum() + out[1].float().sum() * 0.125).backward()
                            row[f"{variant}_ms"] = round(_arms.summary(_arms.time_cuda(fn, a.warmup, a.repeats))["median_ms"], 4)
                        row["mp_over_stable"] = round(row["mp_ms"] / row["stable_ms"], 3)
                    except Exception as exc:
                        row["error"] = f"{type(exc).__name__}: {exc}"[:160]
                    rows.append(row)
                    print(json.dumps(row), flush=True)
    if a.out:
        Path(a.out).parent.mkdir(parents=True, exist_ok=True)
        Path(a.out).write_text(json.dumps({"gpu": torch.cuda.get_device_name(dev), "rows": rows}, indent=1))


if __name__ == "__main__":
    main()
