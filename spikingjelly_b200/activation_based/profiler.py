"""Memory and CUDA-time profilers built on module hooks.

Five profilers with the reference's names and result layouts
(``spikingjelly/activation_based/profiler.py:59-1247``): ``CategoryMemoryProfiler`` (weights /
buffers / gradients / optimizer state / everything else), ``LayerWiseMemoryProfiler`` (allocator
levels around every selected module's forward and backward), ``LayerWiseFPCUDATimeProfiler`` and
``LayerWiseBPCUDATimeProfiler`` (CUDA-event time of every selected module).

One thing is different by design: memory is read through a *meter*.  On a CUDA device the meter is
the caching allocator (current / peak allocated bytes).  On a machine without a GPU the meter is
``SavedActivationMeter``, which counts the bytes autograd keeps alive for backward (through
``torch.autograd.graph.saved_tensors_hooks``) — the quantity activation checkpointing changes —
so that layer-wise profiles and the automatic checkpoint placement also work, and are testable,
on the host.
"""
from __future__ import annotations

import abc
import gc
import inspect
import os
import time
from collections import defaultdict
from pathlib import Path
from typing import Iterable, Optional, Tuple

import torch
import torch.nn as nn
import torch.optim as optim

from ..logger import logger

KB = 1024.0
MB = 1024.0 * 1024.0

__all__ = ["BaseProfiler", "HookProfiler", "CategoryMemoryProfiler", "LayerWiseMemoryProfiler",
           "LayerWiseFPCUDATimeProfiler", "LayerWiseBPCUDATimeProfiler", "SavedActivationMeter", "CudaAllocatorMeter",
           "make_meter"]


def _caller(depth: int = 1) -> str:
    frame = inspect.currentframe().f_back
    for _ in range(depth - 1):
        if frame.f_back is None:
            break
        frame = frame.f_back
    return f"{frame.f_code.co_filename}:line{frame.f_lineno}, {frame.f_code.co_name}"


# ---------------------------------------------------------------------------------------------
# meters
# ---------------------------------------------------------------------------------------------
class CudaAllocatorMeter:
    """Current / peak bytes of the CUDA caching allocator on one device."""

    def __init__(self, device="cuda"):
        self.device = device

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False

    def settle(self):
        torch.cuda.synchronize(self.device)

    def reset_peak(self):
        torch.cuda.synchronize(self.device)
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats(self.device)

    def current(self) -> int:
        return torch.cuda.memory_allocated(self.device)

    def peak(self) -> int:
        return torch.cuda.max_memory_allocated(self.device)


class _Held:
    """What autograd stores instead of the tensor: the tensor plus a release notice."""
    __slots__ = ("tensor", "meter", "key")

    def __init__(self, tensor, meter, key):
        self.tensor, self.meter, self.key = tensor, meter, key

    def __del__(self):
        m = self.meter
        if self.key is not None and m is not None:
            left = m._refs.get(self.key, 0) - 1
            if left <= 0:
                m._refs.pop(self.key, None)
                m._live -= m._size.pop(self.key, 0)
            else:
                m._refs[self.key] = left


class SavedActivationMeter:
    """Bytes autograd currently keeps for backward (each storage counted once; parameters and
    buffers of ``exclude`` modules are not activations and are skipped).  Usable on any device."""

    def __init__(self, exclude: Iterable[nn.Module] = ()):
        self._skip = set()
        for m in exclude:
            for t in list(m.parameters()) + list(m.buffers()):
                self._skip.add(t.untyped_storage().data_ptr())
        self._refs, self._size = {}, {}
        self._live = 0
        self._peak = 0
        self._ctx = None

    def _pack(self, t: torch.Tensor):
        try:
            st = t.untyped_storage()
            key, n = st.data_ptr(), st.nbytes()
        except (RuntimeError, NotImplementedError):
            return _Held(t, None, None)
        if key in self._skip or key == 0:
            return _Held(t, None, None)
        if key not in self._refs:
            self._refs[key], self._size[key] = 0, n
            self._live += n
            self._peak = max(self._peak, self._live)
        self._refs[key] += 1
        return _Held(t, self, key)

    @staticmethod
    def _unpack(h: _Held):
        return h.tensor

    def __enter__(self):
        self._ctx = torch.autograd.graph.saved_tensors_hooks(self._pack, self._unpack)
        self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        ctx, self._ctx = self._ctx, None
        return ctx.__exit__(*exc) if ctx is not None else False

    def settle(self):
        pass

    def reset_peak(self):
        self._peak = self._live

    def current(self) -> int:
        return self._live

    def peak(self) -> int:
        return self._peak


def make_meter(device, models: Iterable[nn.Module] = ()):
    """The allocator meter for CUDA devices, the saved-activation meter otherwise."""
    if torch.device(device).type == "cuda" and torch.cuda.is_available():
        return CudaAllocatorMeter(device)
    return SavedActivationMeter(models)


# ---------------------------------------------------------------------------------------------
# profilers
# ---------------------------------------------------------------------------------------------
class BaseProfiler(abc.ABC):
    """Context manager; ``export()`` returns (and optionally logs) what was measured."""

    def __init__(self, models: Tuple[nn.Module]):
        self.models = (models,) if isinstance(models, nn.Module) else tuple(models)
        self._entered = False

    @abc.abstractmethod
    def export(self):
        ...

    @abc.abstractmethod
    def close(self):
        ...

    def __enter__(self):
        if self._entered:
            raise RuntimeError("Profiler already entered")
        self._entered = True
        return self

    def __exit__(self, *args):
        self.close()
        self._entered = False
        return False

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _replace_file(path) -> Path:
    path = Path(path)
    if path.is_file():      # never a device node such as os.devnull
        os.remove(path)
    return path


class CategoryMemoryProfiler(BaseProfiler):
    """Splits the live tensors of the process into weight / buffer / gradient / optimizer_state /
    input_or_state (everything else the garbage collector can see on the profiled device type)."""

    def __init__(self, models, optimizers, log_path="snn_memory.prof.txt", device_type: str = "cuda"):
        super().__init__(models)
        self.optimizers = (optimizers,) if isinstance(optimizers, optim.Optimizer) else tuple(optimizers)
        self.log_path = _replace_file(log_path)
        self.device_type = device_type
        self.device_count = torch.cuda.device_count() if device_type == "cuda" else 0

    def _on_device(self, t) -> bool:
        return t.device.type == self.device_type

    def _get_memory_stats(self):
        usage = defaultdict(float)
        seen = set()

        def account(t, category):
            if t is None or not torch.is_tensor(t) or not self._on_device(t):
                return
            try:
                ptr = t.data_ptr()
            except (RuntimeError, AttributeError, NotImplementedError):
                return
            if (category == "input_or_state" and ptr in seen):
                return
            usage[category] += t.element_size() * t.numel()
            seen.add(ptr)

        for model in self.models:
            for p in model.parameters():
                account(p, "weight")
            for b in model.buffers():
                account(b, "buffer")
        for model in self.models:
            for p in model.parameters():
                account(p.grad, "gradient")
        for opt in self.optimizers:
            for group in opt.param_groups:
                for p in group["params"]:
                    for value in opt.state.get(p, {}).values():
                        account(value, "optimizer_state")
        for obj in gc.get_objects():
            try:
                if torch.is_tensor(obj):
                    account(obj, "input_or_state")
            except Exception:
                pass
        return usage

    def export(self, depth=2, output: bool = True, *args, **kwargs):
        usage = self._get_memory_stats()
        total = {}
        for d in range(self.device_count):
            total[d] = {"allocated": torch.cuda.memory_allocated(d) / MB, "reserved": torch.cuda.memory_reserved(d) / MB}
        if output:
            head = f"=== Category-wise Memory ({time.ctime()}; {_caller(depth)}) ==="
            bar = "=" * len(head)
            lines = [bar, head, bar]
            lines += [f"cuda:{d} - Allocated: {v['allocated']:.2f} MB, Reserved: {v['reserved']:.2f} MB" for d, v in total.items()]
            lines.append("Memory Usage by Category:")
            lines += [f"  {k}: {v / MB:.2f} MB" for k, v in usage.items()]
            lines += [f"  Total: {sum(usage.values()) / MB:.2f} MB", bar, bar, "", "", ""]
            with open(self.log_path, "a") as f:
                f.write("\n".join(lines))
            logger.info("Category memory profile exported: devices=%s categories=%s", len(total), len(usage),
                        extra={"event": "profiler_export_summary", "profile_type": type(self).__name__,
                               "device_count": len(total), "category_count": len(usage)})
        return total, usage

    def close(self):
        pass


class HookProfiler(BaseProfiler):
    """Selects modules of ``models`` (``search_mode`` per model: ``"self"``, ``"direct_children"`` or
    ``"submodules"``; filtered by ``instances``) and lets subclasses hook them.  Module names are
    ``"<model_name>'s <path>"``."""

    def __init__(self, models, model_names=None, search_mode=("direct_children",), instances=(nn.Module,), log_path="prof.txt"):
        super().__init__(models)
        if model_names is None:
            model_names = tuple(f"net{i}" for i in range(len(self.models)))
        if not isinstance(model_names, (tuple, list)):
            raise ValueError("model_names should be a tuple of strings")
        if len(model_names) != len(self.models):
            raise ValueError("model_names should have the same length as models")
        self.model_names = tuple(model_names)
        self.search_mode = (search_mode,) if isinstance(search_mode, str) else tuple(search_mode)
        if len(self.search_mode) != len(self.models):
            raise ValueError("search_mode should have the same length as models")
        self.instances = (instances,) if isinstance(instances, type) else tuple(instances)
        self.log_path = _replace_file(log_path)
        self.hooks = []
        self.module_obj = {}

    def __enter__(self):
        super().__enter__()
        self._register_hooks()
        return self

    def _register_hooks(self):
        raise NotImplementedError

    def _remove_hooks(self):
        for h in getattr(self, "hooks", []):
            h.remove()
        if hasattr(self, "hooks"):
            self.hooks.clear()

    def close(self):
        self._remove_hooks()

    @staticmethod
    def _iterate(mode: str, model: nn.Module):
        if mode == "self":
            return (("self", model),)
        if mode == "submodules":
            return model.named_modules()
        if mode == "direct_children":
            return model.named_children()
        raise ValueError(f"Unknown search mode: {mode}")

    def _selected_modules(self):
        for model, mname, mode in zip(self.models, self.model_names, self.search_mode):
            for name, module in self._iterate(mode, model):
                if isinstance(module, self.instances):
                    full = f"{mname}'s {name}"
                    self.module_obj[full] = module
                    yield full, module


class LayerWiseMemoryProfiler(HookProfiler):
    """Records, per selected module, memory at forward start / end / peak and backward start / end /
    peak.  ``export`` returns rows ``(name, f_start, f_end, f_peak, f_delta, b_start, b_end, b_peak,
    b_delta)`` sorted by ``sort_by`` (default: the largest field of the row), largest first."""

    field_idx = {"name": 0, "forward_start_memory": 1, "forward_end_memory": 2, "forward_peak_memory": 3,
                 "forward_delta_memory": 4, "backward_start_memory": 5, "backward_end_memory": 6,
                 "backward_peak_memory": 7, "backward_delta_memory": 8}

    def __init__(self, models, model_names=None, search_mode=("direct_children",), instances=(nn.Module,),
                 log_path="layer_memory.prof.txt", data_path="layer_memory.prof.pt", device: str = "cuda"):
        super().__init__(models, model_names, search_mode, instances, log_path)
        self.device = device
        self.data_path = _replace_file(data_path)
        self.meter = make_meter(device, self.models)
        self.forward_start_memory = defaultdict(float)
        self.forward_end_memory = defaultdict(float)
        self.forward_peak_memory = defaultdict(float)
        self.backward_start_memory = defaultdict(float)
        self.backward_end_memory = defaultdict(float)
        self.backward_peak_memory = defaultdict(float)

    def __enter__(self):
        self.meter.__enter__()
        return super().__enter__()

    def close(self):
        super().close()
        meter = getattr(self, "meter", None)
        if meter is not None and getattr(meter, "_ctx", None) is not None:
            meter.__exit__(None, None, None)

    def _register_hooks(self):
        meter = self.meter

        def begin(start, peak, name):
            def hook(module, *_):
                meter.reset_peak()
                start[name] = meter.current()
                peak[name] = 0
            return hook

        def finish(end, peak, name):
            def hook(module, *_):
                meter.settle()
                peak[name] = max(meter.peak(), peak[name])
                end[name] = meter.current()
            return hook

        for name, module in self._selected_modules():
            self.hooks += [
                module.register_forward_pre_hook(begin(self.forward_start_memory, self.forward_peak_memory, name)),
                module.register_forward_hook(finish(self.forward_end_memory, self.forward_peak_memory, name)),
                module.register_full_backward_pre_hook(begin(self.backward_start_memory, self.backward_peak_memory, name)),
                module.register_full_backward_hook(finish(self.backward_end_memory, self.backward_peak_memory, name)),
            ]

    def export(self, depth=2, sort_by: Optional[str] = None, output: bool = True, *args, **kwargs):
        rows = []
        for name in self.forward_peak_memory:
            fs, fe, fp = self.forward_start_memory[name], self.forward_end_memory[name], self.forward_peak_memory[name]
            bs, be, bp = self.backward_start_memory[name], self.backward_end_memory[name], self.backward_peak_memory[name]
            rows.append((name, fs, fe, fp, fp - fs, bs, be, bp, bp - bs))
        key = (lambda r: r[self.field_idx[sort_by]]) if sort_by is not None else (lambda r: max(r[1:]))
        rows.sort(key=key, reverse=True)
        if output:
            head = f"=== Layer-wise Memory Stats ({time.ctime()}; {_caller(depth)}) ==="
            bar = "=" * len(head)
            lines = [bar, head, bar]
            for name, fs, fe, fp, fd, bs, be, bp, bd in rows:
                lines.append(f"{name}:{self.module_obj[name]}")
                lines.append(f" forward_start_memory: {fs / MB:.2f} MB, forward_end_memory: {fe / MB:.2f} MB, "
                             f"forward_peak_memory: {fp / MB:.2f} MB, forward_delta_memory: {fd / MB:.2f} MB, ")
                lines.append(f" backward_start_memory: {bs / MB:.2f} MB, backward_end_memory: {be / MB:.2f} MB, "
                             f"backward_peak_memory: {bp / MB:.2f} MB, backward_delta_memory: {bd / MB:.2f} MB")
            lines += [bar, bar, "", "", ""]
            with open(self.log_path, "a") as f:
                f.write("\n".join(lines))
            logger.info("Layer memory profile exported: modules=%s", len(rows),
                        extra={"event": "profiler_export_summary", "profile_type": type(self).__name__, "module_count": len(rows)})
            torch.save({k: dict(getattr(self, k)) for k in ("forward_start_memory", "forward_end_memory", "forward_peak_memory",
                                                            "backward_start_memory", "backward_end_memory", "backward_peak_memory")},
                       self.data_path)
        return rows


class _Stopwatch:
    """CUDA events when a GPU is present, the host clock otherwise."""

    def __init__(self):
        self.cuda = torch.cuda.is_available()

    def start(self):
        if self.cuda:
            torch.cuda.synchronize()
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            return ev
        return time.perf_counter()

    def stop(self, started) -> float:
        if self.cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            torch.cuda.synchronize()
            return started.elapsed_time(ev)
        return (time.perf_counter() - started) * 1e3


class _LayerWiseTimeProfiler(HookProfiler):
    _direction = "forward"

    def __init__(self, models, model_names=None, search_mode=("direct_children",), instances=(nn.Module,), warmup: int = 10,
                 log_path="layer_time.prof.txt"):
        super().__init__(models, model_names, search_mode, instances, log_path)
        self.warmup = warmup
        self.result = defaultdict(list)
        self.start_events = {}
        self._watch = _Stopwatch()

    def _hook_pair(self, module, begin, finish):
        raise NotImplementedError

    def _register_hooks(self):
        def begin(name):
            def hook(module, *_):
                self.start_events[name] = self._watch.start()
            return hook

        def finish(name):
            def hook(module, *_):
                started = self.start_events.get(name)
                if started is not None:
                    self.result[name].append(self._watch.stop(started))
                    self.start_events[name] = None
            return hook

        for name, module in self._selected_modules():
            self.start_events[name] = None
            self.hooks += list(self._hook_pair(module, begin(name), finish(name)))

    def export(self, output: bool = True, *args, **kwargs):
        table = []
        for name, samples in self.result.items():
            kept = samples[self.warmup:] or samples
            table.append((name, sum(kept) / len(kept)))
        table.sort(key=lambda r: r[1], reverse=True)
        if output:
            with open(self.log_path, "a") as f:
                for name, avg in table:
                    f.write(f"{name}:{self.module_obj[name]} {self._direction} => {avg:.2f} ms\n\n")
            logger.info("Layer %s CUDA time profile exported: modules=%s", self._direction, len(table),
                        extra={"event": "profiler_export_summary", "profile_type": type(self).__name__, "module_count": len(table)})
        return table


class LayerWiseFPCUDATimeProfiler(_LayerWiseTimeProfiler):
    """Average forward time (ms) of every selected module after ``warmup`` calls, slowest first."""
    _direction = "forward"

    def __init__(self, models, model_names=None, search_mode=("direct_children",), instances=(nn.Module,), warmup: int = 10,
                 log_path="layer_time_fp.prof.txt"):
        super().__init__(models, model_names, search_mode, instances, warmup, log_path)

    def _hook_pair(self, module, begin, finish):
        return module.register_forward_pre_hook(begin), module.register_forward_hook(finish)


class LayerWiseBPCUDATimeProfiler(_LayerWiseTimeProfiler):
    """Average backward time (ms) of every selected module after ``warmup`` calls, slowest first."""
    _direction = "backward"

    def __init__(self, models, model_names=None, search_mode=("direct_children",), instances=(nn.Module,), warmup: int = 10,
                 log_path="layer_time_bp.prof.txt"):
        super().__init__(models, model_names, search_mode, instances, warmup, log_path)

    def _hook_pair(self, module, begin, finish):
        return module.register_full_backward_pre_hook(begin), module.register_full_backward_hook(finish)
