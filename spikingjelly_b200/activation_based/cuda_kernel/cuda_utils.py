"""Timing and launch helpers, the custom-operator switch, integer handles for Python objects and raw-kernel argument
wrapping (``cuda_kernel/cuda_utils.py:25-460`` of the reference)."""
from __future__ import annotations

import time
from typing import Any, Callable, Union

import numpy as np
import torch

from ... import configure

__all__ = ["cpu_timer", "cuda_timer", "cal_fun_t", "cal_blocks", "get_contiguous", "DeviceEnvironment", "use_cupy_custom_op",
           "register_python_object", "resolve_python_object", "wrap_args_to_raw_kernel"]


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


# ---------------------------------------------------------------------------------------------------------------------
# switches, object handles and raw kernel arguments
# ---------------------------------------------------------------------------------------------------------------------
def use_cupy_custom_op() -> bool:
    """Whether the custom-operator path of the GPU neurons is on.  Here that path is the native library; the reference's
    switch ``SJ_USE_CUPY_OP`` (``0 / false / off / no`` to disable) is honoured so that scripts can force the eager path."""
    import os
    if os.getenv("SJ_USE_CUPY_OP", "1").strip().lower() in ("0", "false", "off", "no"):
        return False
    from ... import ops
    return ops.available()


class _Handles:
    """Integer handles for Python objects that must travel through operator schemas (which only take tensors and numbers).
    An object keeps its handle while it is alive; the entry disappears with the object (weak references)."""

    def __init__(self):
        import threading
        import weakref
        self._lock, self._next = threading.Lock(), 0
        self._by_handle: "weakref.WeakValueDictionary[int, Any]" = weakref.WeakValueDictionary()
        self._by_identity: dict = {}

    def register(self, obj) -> int:
        import weakref
        with self._lock:
            known = self._by_identity.get(id(obj))
            if known is not None and self._by_handle.get(known) is obj:
                return known
            handle, self._next = self._next, self._next + 1
            self._by_handle[handle] = obj
            self._by_identity[id(obj)] = handle
            weakref.finalize(obj, self._forget, id(obj), handle)
            return handle

    def _forget(self, identity: int, handle: int) -> None:
        with self._lock:
            if self._by_identity.get(identity) == handle:
                del self._by_identity[identity]

    def resolve(self, handle: int):
        obj = self._by_handle.get(int(handle))
        if obj is None:
            raise RuntimeError(f"Unknown python object id={handle}.")
        return obj


_HANDLES = _Handles()


def register_python_object(obj) -> int:
    """A stable integer for ``obj`` (the same one on every call while ``obj`` lives)."""
    return _HANDLES.register(obj)


def resolve_python_object(obj_id: int):
    """The object behind a handle of :func:`register_python_object`; ``RuntimeError`` once it has been collected."""
    return _HANDLES.resolve(obj_id)


def wrap_args_to_raw_kernel(device: int, *args):
    """Arguments for a raw kernel launch: tensors must be contiguous and on ``device`` and become their data pointers
    (``ctypes.c_void_p``); Python / NumPy scalars become ``c_int`` / ``c_float`` / ``c_bool``.  (The reference returns CuPy
    views; the launchers of ``auto_cuda/base.py`` take ctypes values.)"""
    import ctypes
    out = []
    for a in args:
        if isinstance(a, torch.Tensor):
            if a.get_device() != device:
                raise ValueError(f"tensor on device {a.get_device()}, expected {device}")
            if not a.is_contiguous():
                raise ValueError("raw kernels take contiguous tensors; call get_contiguous first")
            out.append(ctypes.c_void_p(a.data_ptr()))
        elif isinstance(a, (bool, np.bool_)):
            out.append(ctypes.c_bool(bool(a)))
        elif isinstance(a, (int, np.integer)):
            out.append(ctypes.c_int(int(a)))
        elif isinstance(a, (float, np.floating)):
            out.append(ctypes.c_float(float(a)))
        else:
            raise TypeError(f"unsupported raw kernel argument {type(a)}")
    return tuple(out)
