#!/usr/bin/env python
"""``benchmark_train_precision_snn_fc.py`` over a range of widths (input = hidden = each of ``--hidden-dims``), one child process per
width, collected into one table with the fp8 / bf16 and bf16 / fp32 ratios per width.  Counterpart of the reference's
``benchmark/benchmark_train_precision_snn_fc_sweep.py`` (which also draws the curves; this one writes the numbers).

    python benchmark/benchmark_train_precision_snn_fc_sweep.py [--hidden-dims 512 1024 2048 4096] [--impl ours|reference] [--out file.json]
"""
import argparse
import json
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent


def collect(lines):
    """``{precision: row}`` from the child's JSON lines; other output is ignored."""
    rows = {}
    for line in lines:
        line = line.strip()
        if line.startswith("{"):
            try:
                r = json.loads(line)
            except json.JSONDecodeError:
                continue
            if "precision" in r:
                rows[r["precision"]] = r
    return rows


def ratios(rows):
    ms = {p: r["train_ms"] for p, r in rows.items() if "train_ms" in r}
    out = {}
    fp8 = [p for p in ms if p.startswith("fp8")]
    if "bf16" in ms and "fp32" in ms:
        out["bf16_over_fp32_speedup"] = round(ms["fp32"] / ms["bf16"], 3)
    for p in fp8:
        if "bf16" in ms:
            out[f"{p}_over_bf16_speedup"] = round(ms["bf16"] / ms[p], 3)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--hidden-dims", type=int, nargs="+", default=[512, 1024, 2048, 4096])
    ap.add_argument("--precisions", nargs="+", default=None)
    ap.add_argument("--time-steps", type=int, default=16)
    ap.add_argument("--batch-size", type=int, default=256)
    ap.add_argument("--num-classes", type=int, default=1024)
    ap.add_argument("--depth", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--out", type=Path, default=None)
    a = ap.parse_args(argv)
    bad = [v for v in (*a.hidden_dims, a.num_classes) if v % 16]
    if bad:
        raise ValueError(f"All sweep dimensions must be divisible by 16; got {', '.join(map(str, bad))}.")
    table = []
    for h in a.hidden_dims:
        cmd = [sys.executable, str(HERE / "benchmark_train_precision_snn_fc.py"), "--impl", a.impl, "--time-steps", str(a.time_steps),
               "--batch-size", str(a.batch_size), "--input-dim", str(h), "--hidden-dim", str(h), "--num-classes", str(a.num_classes),
               "--depth", str(a.depth), "--warmup", str(a.warmup), "--steps", str(a.steps)]
        if a.precisions:
            cmd += ["--precisions", *a.precisions]
        proc = subprocess.run(cmd, text=True, capture_output=True)
        rows = collect(proc.stdout.splitlines())
        entry = {"impl": a.impl, "hidden_dim": h, "compute_proxy": a.time_steps * a.batch_size * h * h * a.depth,
                 "results_by_precision": rows, **ratios(rows)}
        if proc.returncode != 0 and not rows:
            entry["error"] = proc.stderr.strip().splitlines()[-1][:200] if proc.stderr.strip() else f"exit {proc.returncode}"
        table.append(entry)
        print(json.dumps({k: v for k, v in entry.items() if k != "results_by_precision"}
                         | {"train_ms": {p: r.get("train_ms") for p, r in rows.items()}}), flush=True)
    if a.out:
        a.out.parent.mkdir(parents=True, exist_ok=True)
        a.out.write_text(json.dumps(table, indent=1))
    return table


if __name__ == "__main__":
    main()
