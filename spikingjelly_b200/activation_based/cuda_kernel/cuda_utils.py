"""Timing and launch helpers (``cuda_kernel/cuda_utils.py:116-460`` of the reference)."""
from __future__ import annotations

import time
from typing import Callable, Union

import numpy as np
import torch

from ... import configure

__all__ = ["cpu_timer", "cuda_timer", "cal_fun_t", "cal_blocks", "get_contiguous", "DeviceEnvironment"]


def cpu_timer(f: Callable, *args, **kwargs) -> float:
    """Wall-clock milliseconds of one call."""
    t0 = time.perf_counter()
    f(*args, **kwargs)
    return (time.perf_counter() - t0) * 1e3


def cuda_timer(device: Union[torch.device, int], f: Callable, *args, **kwargs) -> float:
    """Milliseconds of one call measured with CUDA events on ``device``'s current stream."""
    with torch.cuda.device(device):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        f(*args, **kwargs)
        e1.record()
        torch.cuda.synchronize(device)
        return e0.elapsed_time(e1)


def cal_fun_t(n: int, device: Union[str, torch.device, int], f: Callable, *args, **kwargs) -> float:
    """Mean milliseconds over the second half of ``2 n`` calls (the first half warms up); ``n <= 2`` averages all."""
    on_cpu = device == "cpu" or (isinstance(device, torch.device) and device.type == "cpu")
    timer = (lambda: cpu_timer(f, *args, **kwargs)) if on_cpu else (lambda: cuda_timer(device, f, *args, **kwargs))
    if n <= 2:
        return float(np.mean([timer() for _ in range(max(n, 1))]))
    times = [timer() for _ in range(2 * n)]
    return float(np.mean(times[n:]))


def cal_blocks(numel: int, threads: int = -1) -> int:
    threads = configure.cuda_threads if threads == -1 else threads
    return (numel + threads - 1) // threads


def get_contiguous(*args):
    return tuple(a.contiguous() if torch.is_tensor(a) else a for a in args)


class DeviceEnvironment:
    """``with DeviceEnvironment(i):`` makes ``i`` the current CUDA device for the block (no-op on CPU-only hosts)."""

    def __init__(self, device: int):
        self.device, self._ctx = device, None

    def __enter__(self):
        if torch.cuda.is_available() and self.device is not None and int(self.device) >= 0:
            self._ctx = torch.cuda.device(int(self.device))
            self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        if self._ctx is not None:
            self._ctx.__exit__(*exc)
        return False
