"""Both arms of a benchmark behind one handle: ``load("ours")`` gives this framework's ``activation_based`` package,
``load("reference")`` the unmodified reference's (installed under ``baseline/_ref``).  A script built on the handle runs
the same workload through either package, so the two columns of a table come from one code path."""
import importlib
import json
import statistics
import sys
from pathlib import Path
from types import SimpleNamespace

import torch

ROOT = Path(__file__).resolve().parents[1]
REF_DIR = ROOT / "baseline" / "_ref"


def load(impl: str) -> SimpleNamespace:
    """``SimpleNamespace(name, package, fast_backend, get(submodule))``."""
    if impl == "ours":
        sys.path.insert(0, str(ROOT))
        from spikingjelly_b200 import ops
        if torch.cuda.is_available():
            ops.require()
        pkg, fast = "spikingjelly_b200.activation_based", "cuda"
    elif impl == "reference":
        if not (REF_DIR / "spikingjelly").is_dir():
            raise FileNotFoundError("baseline/_ref is empty: the reference is not installed")
        sys.path.insert(0, str(REF_DIR))
        pkg = "spikingjelly.activation_based"
        try:
            import triton  # noqa: F401
            fast = "triton"
        except Exception:
            fast = "torch"
    else:
        raise ValueError(impl)
    return SimpleNamespace(name=impl, package=pkg, fast_backend=fast, get=lambda sub: importlib.import_module(f"{pkg}.{sub}"))


def unavailable(impl: str, exc: BaseException) -> None:
    print(json.dumps({"impl": impl, "unavailable": f"{type(exc).__name__}: {exc}"[:300]}))


def percentile(values, q: float) -> float:
    v = sorted(values)
    pos = (len(v) - 1) * q
    lo = int(pos)
    hi = min(lo + 1, len(v) - 1)
    return v[lo] * (1 - (pos - lo)) + v[hi] * (pos - lo)


def time_cuda(step, warmup: int, repetitions: int, inner: int = 1, flush=None):
    """CUDA-event samples (ms per call of ``step``): ``repetitions`` samples of ``inner`` calls each.  ``flush`` (a
    tensor larger than L2) is zeroed before every sample when given."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    out = []
    for _ in range(repetitions):
        if flush is not None:
            flush.zero_()
        e0.record()
        for _ in range(inner):
            step()
        e1.record()
        e1.synchronize()
        out.append(e0.elapsed_time(e1) / inner)
    return out


def summary(samples):
    return {"median_ms": statistics.median(samples), "p25_ms": percentile(samples, 0.25), "p75_ms": percentile(samples, 0.75)}
