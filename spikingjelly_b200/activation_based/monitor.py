"""Hook-based recorders of module inputs, outputs, attributes and gradients, plus a background GPU
utilisation sampler.

All recorders share one mechanism: they select the sub-modules of ``net`` that are instances of
``instance`` (default: the type of ``net`` itself), register one hook per module, push
``function(value)`` into ``records`` while enabled and keep, per module name, the indices of its
records: ``monitor[i]`` is the i-th record, ``monitor["layer.name"]`` the list of that layer's.

Parity: ``spikingjelly/activation_based/monitor.py:23-864``.
"""
from __future__ import annotations

import datetime
import logging
import os
import threading
import time
from typing import Callable, Optional, Union

import torch
from torch import nn

from ..logger import logger

__all__ = ["BaseMonitor", "OutputMonitor", "InputMonitor", "AttributeMonitor", "GradInputMonitor", "GradOutputMonitor",
           "GPUMonitor"]


def _unpack_len1_tuple(x):
    return x[0] if isinstance(x, tuple) and len(x) == 1 else x


def _identity(x):
    return x


class BaseMonitor:
    def __init__(self):
        self.hooks = []
        self.monitored_layers = []
        self.records = []
        self.name_records_index = {}
        self._enable = True

    def __getitem__(self, i):
        if isinstance(i, int):
            return self.records[i]
        if isinstance(i, str):
            return [self.records[k] for k in self.name_records_index[i]]
        raise ValueError(i)

    def _monitor_modules(self, net, instance):
        instance = type(net) if instance is None else instance
        selected = [(name, m) for name, m in net.named_modules() if isinstance(m, instance)]
        for name, _ in selected:
            self.monitored_layers.append(name)
            self.name_records_index[name] = []
        return selected

    def _record(self, name, value):
        self.name_records_index[name].append(len(self.records))
        self.records.append(value)

    def _attach(self, net, instance, register: str, pick: Callable, fn: Callable):
        """``register``: name of the nn.Module registration method; ``pick(module, *hook_args)``
        extracts the raw value; ``fn`` post-processes it."""
        self._pick, self._post = pick, fn
        for name, module in self._monitor_modules(net, instance):
            self.hooks.append(getattr(module, register)(self.create_hook(name)))

    def create_hook(self, name):
        """The hook registered on the module called ``name``; a subclass may override it to record something else."""
        def hook(m, *args):
            if self._enable:
                self._record(name, self._post(self._pick(m, *args)))
        return hook

    def clear_recorded_data(self):
        self.records.clear()
        for v in self.name_records_index.values():
            v.clear()

    def enable(self):
        self._enable = True

    def disable(self):
        self._enable = False

    def is_enable(self):
        return self._enable

    def remove_hooks(self):
        for h in self.hooks:
            h.remove()
        self.hooks.clear()

    def __del__(self):
        self.disable()
        self.clear_recorded_data()
        self.remove_hooks()


class OutputMonitor(BaseMonitor):
    """Records ``function_on_output(module output)`` after every forward of the selected modules."""

    def __init__(self, net: nn.Module, instance=None, function_on_output: Callable = _identity):
        super().__init__()
        self.function_on_output = function_on_output
        self._attach(net, instance, "register_forward_hook", lambda m, inputs, output: _unpack_len1_tuple(output),
                     function_on_output)


class InputMonitor(BaseMonitor):
    """Records ``function_on_input(module input)`` after every forward of the selected modules."""

    def __init__(self, net: nn.Module, instance=None, function_on_input: Callable = _identity):
        super().__init__()
        self.function_on_input = function_on_input
        self._attach(net, instance, "register_forward_hook", lambda m, inputs, output: _unpack_len1_tuple(inputs),
                     function_on_input)


class AttributeMonitor(BaseMonitor):
    """Records ``function_on_attribute(getattr(module, attribute_name))`` before (``pre_forward``) or
    after every forward, e.g. the membrane potential ``v`` of every neuron."""

    def __init__(self, attribute_name: str, pre_forward: bool, net: nn.Module, instance=None,
                 function_on_attribute: Callable = _identity):
        super().__init__()
        self.attribute_name = attribute_name
        self.function_on_attribute = function_on_attribute
        self._attach(net, instance, "register_forward_pre_hook" if pre_forward else "register_forward_hook",
                     lambda m, *args: getattr(m, attribute_name), function_on_attribute)


class GradInputMonitor(BaseMonitor):
    """Records the gradient w.r.t. the module *input* (full backward hook)."""

    def __init__(self, net: nn.Module, instance=None, function_on_grad_input: Callable = _identity):
        super().__init__()
        self.function_on_grad_input = function_on_grad_input
        self._attach(net, instance, "register_full_backward_hook", lambda m, gi, go: _unpack_len1_tuple(gi),
                     function_on_grad_input)


class GradOutputMonitor(BaseMonitor):
    """Records the gradient w.r.t. the module *output* (full backward hook)."""

    def __init__(self, net: nn.Module, instance=None, function_on_grad_output: Callable = _identity):
        super().__init__()
        self.function_on_grad_output = function_on_grad_output
        self._attach(net, instance, "register_full_backward_hook", lambda m, gi, go: _unpack_len1_tuple(go),
                     function_on_grad_output)


class GPUMonitor(threading.Thread):
    """Samples utilisation (%) and used memory (MiB) of ``gpu_ids`` every ``interval`` seconds in a
    daemon thread; writes to TensorBoard under ``log_dir/gpu_monitor`` or, without ``log_dir``, to
    the logger.  Reads through NVML (read-only queries); ``sampler`` can be replaced for tests."""

    def __init__(self, log_dir: Optional[str] = None, gpu_ids: tuple = (0,), interval: float = 600.0, start_now=True,
                 sampler: Optional[Callable] = None):
        super().__init__(daemon=True)
        self.gpu_ids, self.interval = tuple(gpu_ids), interval
        self.stopped = False
        self.step = 0
        self._wake = threading.Event()
        self._sampler = sampler or self._nvml_sample
        self.cmds = ("nvidia-smi --query-gpu=utilization.gpu,memory.used --format=csv -i "
                     + ",".join(str(g) for g in self.gpu_ids))
        self.writer = None
        if log_dir is not None:
            from torch.utils.tensorboard import SummaryWriter
            self.writer = SummaryWriter(os.path.join(log_dir, "gpu_monitor"))
        if start_now:
            self.start()

    def _nvml_sample(self):
        """[(utilisation %, memory used MiB)] per monitored GPU."""
        try:
            import pynvml
            pynvml.nvmlInit()
            out = []
            for g in self.gpu_ids:
                h = pynvml.nvmlDeviceGetHandleByIndex(g)
                out.append((int(pynvml.nvmlDeviceGetUtilizationRates(h).gpu), int(pynvml.nvmlDeviceGetMemoryInfo(h).used >> 20)))
            return out
        except Exception:
            import re
            with os.popen(self.cmds) as fp:
                rows = fp.read().split("\n")[1:-1]
            return [tuple(int(v) for v in re.findall(r"\d+", r)[:2]) for r in rows]

    def stop(self):
        self.stopped = True
        self._wake.set()

    def run(self):
        while not self.stopped:
            samples = self._sampler()
            if self.writer is not None:
                for gpu, (util, mem) in zip(self.gpu_ids, samples):
                    self.writer.add_scalar(f"utilization_{gpu}", util, self.step)
                    self.writer.add_scalar(f"memory_used_{gpu}", mem, self.step)
            elif logger.isEnabledFor(logging.INFO):
                logger.info("GPU monitor sample at %s: %s", datetime.datetime.now().strftime("%Y-%m-%d %H:%M:%S"),
                            ", ".join(f"gpu{g}: {u} %, {m} MiB" for g, (u, m) in zip(self.gpu_ids, samples)))
            self.step += 1
            self._wake.wait(self.interval)
