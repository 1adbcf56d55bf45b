#!/usr/bin/env python
"""IF / LIF neurons in last-state mode (``store_v_seq=False``: only the final membrane potential is kept), inference and
training: latency (median, quartiles) and the peak allocation one step adds.  Counterpart of the reference's
``benchmark/benchmark_triton_last_state.py`` (same six shapes, same protocol); ``--impl reference`` runs the reference's
Triton neurons through the same loop.

    python benchmark/benchmark_last_state.py --output gpurun_out/last_state.json [--impl ours|reference]
"""
import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))
import _arms  # noqa: E402

CASES = tuple((kind, mode, T, N, dtype) for kind in ("if", "lif") for mode in ("inference", "training")
              for T, N, dtype in ((16, 4096, torch.float32), (32, 16381, torch.float16), (65, 16381, torch.float32)))


def run_case(arm, kind, mode, T, N, dtype, warmup, repetitions, inner):
    torch.manual_seed(20260717)
    neuron = arm.get("neuron")
    x = torch.randn(T, N, device="cuda", dtype=dtype, requires_grad=mode == "training")
    node = (neuron.IFNode if kind == "if" else neuron.LIFNode)(step_mode="m", backend=arm.fast_backend, store_v_seq=False).cuda()

    def train():
        node.reset()
        x.grad = None
        node(x).sum().backward()

    def infer():
        node.reset()
        with torch.inference_mode():
            node(x)
    step = train if mode == "training" else infer
    samples = _arms.time_cuda(step, warmup, repetitions, inner)
    node.reset()
    x.grad = None
    torch.cuda.empty_cache()
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    torch.cuda.reset_peak_memory_stats()
    step()
    torch.cuda.synchronize()
    row = {"impl": arm.name, "backend": arm.fast_backend, "neuron": kind, "mode": mode, "T": T, "N": N, "dtype": str(dtype).removeprefix("torch."),
           "peak_delta_bytes": torch.cuda.max_memory_allocated() - before}
    row.update(_arms.summary(samples))
    return row


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repetitions", type=int, default=25)
    ap.add_argument("--iterations-per-repetition", type=int, default=10)
    ap.add_argument("--output", type=Path, default=None)
    a = ap.parse_args()
    try:
        arm = _arms.load(a.impl)
    except Exception as exc:
        return _arms.unavailable(a.impl, exc)
    rows = []
    for case in CASES:
        rows.append(run_case(arm, *case, a.warmup, a.repetitions, a.iterations_per_repetition))
        print(json.dumps(rows[-1]), flush=True)
    if a.output:
        a.output.parent.mkdir(parents=True, exist_ok=True)
        a.output.write_text(json.dumps({"torch": torch.__version__, "gpu": torch.cuda.get_device_name(0), "results": rows}, indent=2))


if __name__ == "__main__":
    main()
