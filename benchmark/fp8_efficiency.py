"""Pass / fail gates over benchmark rows: does fp8 pay?  Pure functions (no torch), shared by the fp8 model benchmark and the
neuron-kernel benchmark; the role of the reference's ``benchmark/fp8_efficiency.py``.

``assess_model_efficiency(rows, baseline_precision=..., min_training_speedup=..., min_inference_speedup=...)``
    rows carry ``precision``, ``training_samples_per_sec``, ``inference_samples_per_sec`` and the two ``*_peak_allocated_mb``;
    every precision whose name starts with ``fp8`` is compared with the single baseline row.
``assess_neuron_efficiency(rows, min_speedup=...)``
    rows carry ``T``, ``N``, ``neuron_type``, ``process``, ``variant``, ``success``, ``median_ms``, ``peak_allocated_mb``; per group the
    fastest successful fp8 variant (name starting with ``fp8_variant_prefix``) is compared with the ``baseline_variant`` row.
``require_efficiency(report)`` raises ``RuntimeError`` listing the failures of a report that did not pass.
"""
from __future__ import annotations

import math
from typing import Any, Iterable, Mapping

__all__ = ["percentile", "assess_model_efficiency", "assess_neuron_efficiency", "assess_triton_efficiency", "require_efficiency"]


def _positive(row: Mapping[str, Any], key: str) -> float:
    try:
        v = float(row[key])
    except KeyError:
        raise ValueError(f"{key} is required.") from None
    except (TypeError, ValueError):
        v = float("nan")
    if not math.isfinite(v) or v <= 0:
        raise ValueError(f"{key} must be a finite positive number, but got {row[key]!r}.")
    return v


def _threshold(name: str, value: float) -> float:
    if not math.isfinite(value) or value <= 0:
        raise ValueError(f"{name} must be finite and positive.")
    return value


def percentile(values, quantile: float) -> float:
    if not values:
        raise ValueError("Cannot compute a percentile from an empty sequence.")
    if not 0.0 <= quantile <= 1.0:
        raise ValueError("quantile must be in [0, 1].")
    v = sorted(values)
    pos = (len(v) - 1) * quantile
    lo = int(pos)
    hi = min(lo + 1, len(v) - 1)
    return v[lo] + (v[hi] - v[lo]) * (pos - lo)


def assess_model_efficiency(results: Iterable[Mapping[str, Any]], *, baseline_precision: str, min_training_speedup: float,
                            min_inference_speedup: float) -> dict:
    rows = list(results)
    _threshold("Minimum speedups", min_training_speedup)
    _threshold("Minimum speedups", min_inference_speedup)
    if baseline_precision.startswith("fp8"):
        raise ValueError(f"baseline_precision must not be an FP8 variant, but got {baseline_precision!r}.")
    for r in rows:
        if "precision" not in r:
            raise ValueError("precision is required.")
    base = [r for r in rows if str(r["precision"]) == baseline_precision]
    if len(base) != 1:
        raise ValueError(f"Expected exactly one {baseline_precision!r} baseline, but found {len(base)}.")
    fp8 = [r for r in rows if str(r["precision"]).startswith("fp8")]
    if not fp8:
        raise ValueError("At least one FP8 precision result is required.")
    keys = ("training_samples_per_sec", "inference_samples_per_sec", "training_peak_allocated_mb", "inference_peak_allocated_mb")
    b = {k: _positive(base[0], k) for k in keys}
    comparisons, failures = [], []
    for r in fp8:
        c = {k: _positive(r, k) / b[k] for k in keys}
        ok_t, ok_i = c[keys[0]] >= min_training_speedup, c[keys[1]] >= min_inference_speedup
        if not ok_t:
            failures.append(f"{r['precision']} training speedup {c[keys[0]]:.4f}x < {min_training_speedup:.4f}x")
        if not ok_i:
            failures.append(f"{r['precision']} inference speedup {c[keys[1]]:.4f}x < {min_inference_speedup:.4f}x")
        comparisons.append({"precision": str(r["precision"]), "training_speedup": c[keys[0]], "inference_speedup": c[keys[1]],
                            "training_memory_ratio": c[keys[2]], "inference_memory_ratio": c[keys[3]], "training_passed": ok_t,
                            "inference_passed": ok_i, "passed": ok_t and ok_i})
    return {"baseline_precision": baseline_precision, "min_training_speedup": min_training_speedup,
            "min_inference_speedup": min_inference_speedup, "comparisons": comparisons, "failures": failures, "passed": not failures}


_GROUP = ("T", "N", "neuron_type", "process")


def _label(group) -> str:
    return f"T={group[0]} N={group[1]} neuron={group[2]} process={group[3]}"


def assess_neuron_efficiency(rows: Iterable[Mapping[str, Any]], *, min_speedup: float, baseline_variant: str = "stable_fp32",
                             fp8_variant_prefix: str = "mp_plan_float8_") -> dict:
    _threshold("min_speedup", min_speedup)
    rows = list(rows)
    key = lambda r: tuple(r.get(f) for f in _GROUP)                                   # noqa: E731
    is_fp8 = lambda r: r.get("success") is True and str(r.get("variant", "")).startswith(fp8_variant_prefix)   # noqa: E731
    baselines = [r for r in rows if r.get("variant") == baseline_variant]
    comparisons, failures, seen = [], [], set()
    if not baselines:
        failures.append(f"no usable {baseline_variant} baseline results")
    for b in baselines:
        g = key(b)
        if b.get("success") is not True:
            failures.append(f"{_label(g)} {baseline_variant} baseline failed: {b.get('failure_reason') or 'unknown failure'}")
            continue
        missing = [f for f, v in zip(_GROUP, g) if v is None]
        if missing:
            failures.append(f"{_label(g)} {baseline_variant} baseline is missing required group fields: " + ", ".join(missing))
            continue
        if g in seen:
            failures.append(f"{_label(g)} has duplicate successful {baseline_variant} baselines")
            continue
        seen.add(g)
        cands = [r for r in rows if is_fp8(r) and key(r) == g]
        if not cands:
            failures.append(f"{_label(g)} has no successful FP8 prepared-plan result")
            continue
        best = min(cands, key=lambda r: _positive(r, "median_ms"))
        speedup = _positive(b, "median_ms") / _positive(best, "median_ms")
        if speedup < min_speedup:
            failures.append(f"{_label(g)} best FP8 speedup {speedup:.4f}x < {min_speedup:.4f}x")
        comparisons.append({**dict(zip(_GROUP, g)), "baseline_variant": baseline_variant, "best_fp8_variant": best["variant"],
                            "best_compute_dtype": best.get("compute_dtype"), "speedup": speedup,
                            "memory_ratio": _positive(best, "peak_allocated_mb") / _positive(b, "peak_allocated_mb"),
                            "passed": speedup >= min_speedup})
    with_baseline = {key(b) for b in baselines}
    for g in sorted({key(r) for r in rows if is_fp8(r)} - with_baseline, key=repr):
        failures.append(f"{_label(g)} has no successful {baseline_variant} baseline")
    return {"baseline_variant": baseline_variant, "min_speedup": min_speedup, "comparisons": comparisons, "failures": failures,
            "passed": not failures}


assess_triton_efficiency = assess_neuron_efficiency      # the reference's name for the same gate


def require_efficiency(report: Mapping[str, Any]) -> None:
    if report.get("passed") is True:
        return
    raise RuntimeError("FP8 efficiency validation failed: " + "; ".join(report.get("failures") or ["efficiency requirements were not met"]))
