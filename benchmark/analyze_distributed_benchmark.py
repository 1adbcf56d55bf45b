#!/usr/bin/env python
"""Group, aggregate and compare the JSON-lines records written by the benchmarks of this folder
(``benchmark_snn_distributed.py``, ``benchmark_snn_llm.py``, ``benchmark_train_backends.py``, ``bench.py`` lines saved to a
file ...).  Counterpart of the reference's ``benchmark/analyze_distributed_benchmark.py``.

    python benchmark/analyze_distributed_benchmark.py results.jsonl --group-by impl,model,n_gpus
    python benchmark/analyze_distributed_benchmark.py results.jsonl --filter model=spikformer_ti --group-by impl --format csv
    python benchmark/analyze_distributed_benchmark.py results.jsonl --group-by model,n_gpus --compare impl=ours:reference --metric samples_per_s
    python benchmark/analyze_distributed_benchmark.py results.jsonl --filter impl=ours --group-by model --scaling n_gpus --metric samples_per_s

``--compare key=a:b`` adds, per group, the ratio of the metric's median between the records with ``key == a`` and those with
``key == b``; ``--scaling key`` adds the weak-scaling efficiency ``metric(n) / (n * metric(min n))`` along an integer key.
Every numeric field of the records is a metric; without ``--metric`` all of them are aggregated (median, min, max, count).
"""
import argparse
import csv
import io
import json
import statistics
import sys
from collections import OrderedDict
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple


def load_records(path: str) -> List[Dict[str, Any]]:
    rows = []
    with open(path, encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if line.startswith("{"):
                rows.append(json.loads(line))
    return rows


def parse_pairs(text: Optional[str]) -> Dict[str, str]:
    out = {}
    for item in (text or "").split(","):
        if item:
            key, sep, value = item.partition("=")
            if not sep:
                raise ValueError(f"expected key=value, got {item!r}")
            out[key] = value
    return out


def filter_records(rows: Iterable[Dict[str, Any]], wanted: Dict[str, str]) -> List[Dict[str, Any]]:
    return [r for r in rows if all(k in r and str(r[k]) == v for k, v in wanted.items())]


def _number(value) -> Optional[float]:
    if isinstance(value, bool) or value is None:
        return None
    try:
        return float(value)
    except (TypeError, ValueError):
        return None


def group_and_aggregate(rows: Sequence[Dict[str, Any]], keys: Sequence[str], metrics: Optional[Sequence[str]] = None) -> List[Dict[str, Any]]:
    groups: "OrderedDict[Tuple, List[Dict[str, Any]]]" = OrderedDict()
    for r in rows:
        groups.setdefault(tuple(str(r.get(k)) for k in keys), []).append(r)
    out = []
    for gk, members in groups.items():
        names = metrics or sorted({k for m in members for k, v in m.items() if k not in keys and _number(v) is not None})
        row: Dict[str, Any] = dict(zip(keys, gk))
        row["count"] = len(members)
        for name in names:
            values = [v for v in (_number(m.get(name)) for m in members) if v is not None]
            if values:
                row[f"{name}.median"] = statistics.median(values)
                if len(values) > 1:
                    row[f"{name}.min"], row[f"{name}.max"] = min(values), max(values)
        out.append(row)
    return out


def compare(rows, keys, key: str, a: str, b: str, metric: str) -> List[Dict[str, Any]]:
    """Per group: median(metric | key == a) / median(metric | key == b)."""
    left = {tuple(r[k] for k in keys): r for r in group_and_aggregate(filter_records(rows, {key: a}), keys, [metric])}
    right = {tuple(r[k] for k in keys): r for r in group_and_aggregate(filter_records(rows, {key: b}), keys, [metric])}
    out = []
    for gk in left:
        if gk in right and f"{metric}.median" in left[gk] and f"{metric}.median" in right[gk] and right[gk][f"{metric}.median"]:
            row = dict(zip(keys, gk))
            row[f"{metric}[{key}={a}]"] = left[gk][f"{metric}.median"]
            row[f"{metric}[{key}={b}]"] = right[gk][f"{metric}.median"]
            row["ratio"] = left[gk][f"{metric}.median"] / right[gk][f"{metric}.median"]
            out.append(row)
    return out


def scaling(rows, keys, along: str, metric: str) -> List[Dict[str, Any]]:
    """Per group: metric at every value n of ``along`` and ``metric(n) / (n / n0 * metric(n0))`` for the smallest n0."""
    table = group_and_aggregate(rows, list(keys) + [along], [metric])
    by_group: Dict[Tuple, List[Tuple[int, float]]] = {}
    for r in table:
        if f"{metric}.median" in r and str(r[along]).lstrip("-").isdigit():
            by_group.setdefault(tuple(r[k] for k in keys), []).append((int(r[along]), r[f"{metric}.median"]))
    out = []
    for gk, points in by_group.items():
        points.sort()
        n0, v0 = points[0]
        for n, v in points:
            row = dict(zip(keys, gk))
            row.update({along: n, metric: v, "efficiency": v / (n / n0 * v0) if v0 else float("nan")})
            out.append(row)
    return out


def render(rows: List[Dict[str, Any]], fmt: str) -> str:
    if fmt == "json":
        return json.dumps(rows, indent=2)
    cols: List[str] = []
    for r in rows:
        cols += [c for c in r if c not in cols]
    cell = lambda v: f"{v:.4g}" if isinstance(v, float) else ("" if v is None else str(v))
    if fmt == "csv":
        buf = io.StringIO()
        w = csv.writer(buf)
        w.writerow(cols)
        for r in rows:
            w.writerow([cell(r.get(c)) for c in cols])
        return buf.getvalue()
    body = [[cell(r.get(c)) for c in cols] for r in rows]
    width = [max(len(c), *(len(b[i]) for b in body)) if body else len(c) for i, c in enumerate(cols)]
    line = lambda items: "| " + " | ".join(s.ljust(w) for s, w in zip(items, width)) + " |"
    return "\n".join([line(cols), "|" + "|".join("-" * (w + 2) for w in width) + "|"] + [line(b) for b in body])


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("path")
    ap.add_argument("--filter", default="")
    ap.add_argument("--group-by", default="impl,model,mode,n_gpus")
    ap.add_argument("--metric", default=None, help="comma-separated metric names (default: every numeric field)")
    ap.add_argument("--compare", default=None, help="key=a:b")
    ap.add_argument("--scaling", default=None, help="integer key to scale along, e.g. n_gpus")
    ap.add_argument("--format", choices=["table", "csv", "json"], default="table")
    a = ap.parse_args(argv)
    rows = filter_records(load_records(a.path), parse_pairs(a.filter))
    keys = [k for k in a.group_by.split(",") if k]
    metrics = [m for m in a.metric.split(",") if m] if a.metric else None
    if a.compare:
        key, _, pair = a.compare.partition("=")
        left, _, right = pair.partition(":")
        if not (key and left and right and metrics and len(metrics) == 1):
            ap.error("--compare needs key=a:b and exactly one --metric")
        table = compare(rows, [k for k in keys if k != key], key, left, right, metrics[0])
    elif a.scaling:
        if not (metrics and len(metrics) == 1):
            ap.error("--scaling needs exactly one --metric")
        table = scaling(rows, [k for k in keys if k != a.scaling], a.scaling, metrics[0])
    else:
        table = group_and_aggregate(rows, keys, metrics)
    print(render(table, a.format))
    return 0


if __name__ == "__main__":
    sys.exit(main())
