#!/usr/bin/env python
"""bf16 against fp8 on a stack of wide linear layers (``--depth`` x Linear(width) + GELU, batch 4096), training and
inference, through the public precision API (``precision.prepare_model_for_precision``).  Counterpart of the reference's
``benchmark/benchmark_fp8_training_inference.py`` and ``fp8_efficiency.py``: same workload and defaults, several trials per
precision, medians, and the same verdict (fp8 "pays" when its median speed-up over the baseline reaches
``--min-training-speedup`` / ``--min-inference-speedup``).

    python benchmark/benchmark_fp8_training_inference.py [--precisions bf16 fp8] [--fp8-recipe delayed|current] [--impl ours|reference]

With ``--impl reference`` the fp8 modes are the reference's (``fp8-torchao``, ``fp8-te``); they need vendor libraries and
report why they cannot run when those are absent.  Times are CUDA events over all steps of a phase.
"""
import argparse
import json
import statistics
import sys
import time
from pathlib import Path

import torch
import torch.nn as nn

sys.path.insert(0, str(Path(__file__).resolve().parent))
import _arms  # noqa: E402


def workload(width: int, depth: int, classes: int) -> nn.Module:
    mods = []
    for _ in range(depth - 1):
        mods += [nn.Linear(width, width), nn.GELU()]
    return nn.Sequential(*mods, nn.Linear(width, classes))


def timed(steps: int, fn) -> float:
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def run(a, precision_api, mode: str, state, x, target, device):
    model = workload(a.width, a.depth, a.num_classes).to(device)
    model.load_state_dict(state)
    model.train()
    t0 = time.perf_counter()
    conf = {"mode": mode, "strictness": "strict", "device": str(device)}
    if mode.startswith("fp8") and a.impl == "ours":
        conf["fp8_recipe"] = a.fp8_recipe
    art = precision_api.prepare_model_for_precision(model, device, precision_api.PrecisionConfig(**conf))
    torch.cuda.synchronize()
    prep_ms = (time.perf_counter() - t0) * 1e3
    model = art.model
    report = art.policy.conversion_report()
    if mode.startswith("fp8") and not report["converted_modules"]:
        raise RuntimeError(f"{mode} did not convert any benchmark modules.")
    opt = torch.optim.SGD(model.parameters(), lr=a.lr)
    last = {}

    def train_step():
        opt.zero_grad(set_to_none=True)
        with art.autocast_context():
            loss = nn.functional.cross_entropy(model(x), target)
        art.backward(loss, opt, parameters=model.parameters())
        last["loss"] = loss.detach()
    for _ in range(a.warmup):
        train_step()
    if not bool(torch.isfinite(last["loss"])):
        raise RuntimeError(f"{mode} training produced a non-finite loss.")
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    train_ms = timed(a.training_steps, train_step)
    train_peak = torch.cuda.max_memory_allocated() / 2 ** 20
    opt.zero_grad(set_to_none=True)
    model.eval()

    def infer_step():
        with torch.inference_mode(), art.autocast_context():
            last["out"] = model(x)
    for _ in range(a.warmup):
        infer_step()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    infer_ms = timed(a.inference_steps, infer_step)
    return {"precision": mode, "preparation_ms": round(prep_ms, 2), "training_ms": round(train_ms, 4),
            "training_samples_per_sec": round(a.batch_size / train_ms * 1e3, 1), "training_peak_allocated_mb": round(train_peak, 1),
            "inference_ms": round(infer_ms, 4), "inference_samples_per_sec": round(a.batch_size / infer_ms * 1e3, 1),
            "inference_peak_allocated_mb": round(torch.cuda.max_memory_allocated() / 2 ** 20, 1), "final_loss": round(float(last["loss"]), 5),
            "output_checksum": float(last["out"].float().mean()), "converted_modules": len(report["converted_modules"])}


def assess(rows, baseline: str, min_train: float, min_infer: float):
    """Median speed-up of every fp8 precision over ``baseline`` and whether it reaches the two thresholds."""
    med = {}
    for r in rows:
        med.setdefault(r["precision"], []).append(r)
    pick = lambda p, k: statistics.median(x[k] for x in med[p])
    if baseline not in med:
        return {"baseline": baseline, "verdicts": {}}
    out = {}
    for p in med:
        if p == baseline:
            continue
        ts, is_ = pick(baseline, "training_ms") / pick(p, "training_ms"), pick(baseline, "inference_ms") / pick(p, "inference_ms")
        out[p] = {"training_speedup": round(ts, 3), "inference_speedup": round(is_, 3), "training_pays": ts >= min_train,
                  "inference_pays": is_ >= min_infer}
    return {"baseline": baseline, "min_training_speedup": min_train, "min_inference_speedup": min_infer, "verdicts": out}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--precisions", nargs="+", default=None)
    ap.add_argument("--fp8-recipe", default="delayed")
    ap.add_argument("--batch-size", type=int, default=4096)
    ap.add_argument("--width", type=int, default=2048)
    ap.add_argument("--depth", type=int, default=8)
    ap.add_argument("--num-classes", type=int, default=2048)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--training-steps", type=int, default=30)
    ap.add_argument("--inference-steps", type=int, default=100)
    ap.add_argument("--trials", type=int, default=5)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--seed", type=int, default=20260718)
    ap.add_argument("--baseline-precision", default="bf16")
    ap.add_argument("--min-training-speedup", type=float, default=1.05)
    ap.add_argument("--min-inference-speedup", type=float, default=1.05)
    ap.add_argument("--output", type=Path)
    a = ap.parse_args()
    try:
        arm = _arms.load(a.impl)
        precision_api = arm.get("precision")
    except Exception as exc:
        return _arms.unavailable(a.impl, exc)
    modes = a.precisions or (["bf16", "fp8"] if a.impl == "ours" else ["bf16", "fp8-torchao", "fp8-te"])
    device = torch.device("cuda", 0)
    torch.manual_seed(a.seed)
    state = workload(a.width, a.depth, a.num_classes).state_dict()
    x = torch.randn(a.batch_size, a.width, device=device)
    target = torch.randint(a.num_classes, (a.batch_size,), device=device)
    rows = []
    for mode in modes:
        for trial in range(a.trials):
            try:
                row = run(a, precision_api, mode, state, x, target, device)
                row.update(impl=a.impl, trial=trial)
                rows.append(row)
            except Exception as exc:
                row = {"impl": a.impl, "precision": mode, "trial": trial, "unavailable": f"{type(exc).__name__}: {exc}"[:240]}
            print(json.dumps(row), flush=True)
            if "unavailable" in row:
                break
    verdict = assess(rows, a.baseline_precision, a.min_training_speedup, a.min_inference_speedup)
    print(json.dumps(verdict))
    if a.output:
        a.output.parent.mkdir(parents=True, exist_ok=True)
        a.output.write_text(json.dumps({"gpu": torch.cuda.get_device_name(0), "torch": torch.__version__, "rows": rows, "efficiency": verdict}, indent=2))


if __name__ == "__main__":
    main()
