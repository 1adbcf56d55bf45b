"""Analytical energy estimate after Lemaire et al. ("An analytical estimation of spiking neural networks energy
efficiency", 2022): ``E = E_ops + E_addressing + E_memory`` with 45 nm unit costs (add 0.1 pJ, multiply 3.1 pJ) and a
memory cost per byte that grows piece-wise linearly with the size of the buffer being accessed (8 kB / 32 kB / 1 MB
break points).  Operations come from the SynOp / MAC / AC counters, state arithmetic and state traffic from
:class:`NeuronStateCounter`, addressing from :class:`LemaireAddressingCounter`, and input / output / parameter traffic
from forward hooks on the linear and convolution modules (sparse where the input is sparse).
Same report fields as ``op_counter/analytical_energy/core.py:49-567`` of the reference.
"""
from __future__ import annotations

import copy
import warnings
from dataclasses import dataclass, field
from numbers import Real
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ...neuron.base_node import BaseNode
from .._sparse_memory import active_element_count, dense_bytes, dense_bytes_tree, is_sparse_access_tensor, sparse_bytes
from ..base import DispatchCounterMode
from ..counters import ACCounter, MACCounter, SynOpCounter
from ..lemaire_addressing import LemaireAddressingCounter
from ..neuron_state import NeuronStateCounter

__all__ = ["LemaireEnergyConfig", "LemaireEnergyCostConfig", "LemaireEnergyProfiler", "LemaireEnergyReport", "estimate_lemaire_energy"]

_ACCESS_WIDTH_BYTES = 4.0
_MEMORY_MODULES = (nn.Linear, nn.Conv1d, nn.Conv2d, nn.Conv3d, nn.ConvTranspose1d, nn.ConvTranspose2d, nn.ConvTranspose3d)


@dataclass
class LemaireEnergyCostConfig:
    e_add_pj: float = 0.1
    e_mul_pj: float = 3.1
    #: (buffer size in bytes, pJ per byte): 10 / 20 / 100 pJ per 32-bit access at 8 kB / 32 kB / 1 MB
    memory_breakpoints: Tuple[Tuple[float, float], ...] = (
        (0.0, 0.0), (8.0 * 1024.0, 10.0 / _ACCESS_WIDTH_BYTES), (32.0 * 1024.0, 20.0 / _ACCESS_WIDTH_BYTES),
        (1024.0 * 1024.0, 100.0 / _ACCESS_WIDTH_BYTES))

    def __post_init__(self):
        pts = self.memory_breakpoints
        if len(pts) != 4 or any(not isinstance(p, tuple) or len(p) != 2 for p in pts):
            raise ValueError("memory_breakpoints must contain exactly 4 (x, y) pairs.")
        if any(not isinstance(v, Real) for p in pts for v in p):
            raise ValueError("memory_breakpoints entries must be numeric (x, y) pairs.")
        if any(b[0] <= a[0] for a, b in zip(pts, pts[1:])):
            raise ValueError("memory_breakpoints x values must be strictly increasing.")

    def memory_cost_pj(self, memory: float) -> float:
        """pJ per byte for a buffer of ``memory`` bytes (clamped to the first / last break point)."""
        pts = self.memory_breakpoints
        m = max(pts[0][0], min(memory, pts[-1][0]))
        for (x0, y0), (x1, y1) in zip(pts, pts[1:]):
            if m <= x1:
                return y0 + (y1 - y0) / (x1 - x0) * (m - x0)
        return pts[-1][1]


@dataclass
class LemaireEnergyConfig:
    strict: bool = False
    cost_config: LemaireEnergyCostConfig = field(default_factory=LemaireEnergyCostConfig)
    extra_state_rules: Dict[type, Callable] = field(default_factory=dict)
    sparse_zero_ratio_threshold: float = 0.5
    enable_sparse_memory_estimation: bool = True


@dataclass
class LemaireEnergyReport:
    total_pj: float
    breakdown_pj: Dict[str, float]
    counts: Dict[str, int]
    buffer_sizes_bytes: Dict[str, int]
    warnings: List[str]


class _TrafficTracker:
    """Input / output / parameter bytes of the weight layers, and the largest single transfer of each kind."""

    def __init__(self, zero_ratio_threshold: float, enable_sparse: bool):
        self.thr, self.enable_sparse = zero_ratio_threshold, enable_sparse
        self.handles: list = []
        self.warnings: List[str] = []
        self.reset()

    def reset(self):
        self.read_in = self.write_out = self.read_params = 0
        self.read_in_buffer_bytes = self.write_out_buffer_bytes = self.read_params_buffer_bytes = 0
        self.warnings.clear()
        self._warned: set = set()

    def _add(self, rin: int, wout: int, rpar: int):
        self.read_in += int(rin)
        self.write_out += int(wout)
        self.read_params += int(rpar)
        self.read_in_buffer_bytes = max(self.read_in_buffer_bytes, int(rin))
        self.write_out_buffer_bytes = max(self.write_out_buffer_bytes, int(wout))
        self.read_params_buffer_bytes = max(self.read_params_buffer_bytes, int(rpar))

    def _sparse(self, t: torch.Tensor) -> bool:
        return self.enable_sparse and is_sparse_access_tensor(t, zero_ratio_threshold=self.thr)

    def _hook(self, module: nn.Module, inputs, output):
        if not inputs:
            return
        x = inputs[0]
        out = output[0] if isinstance(output, (tuple, list)) and len(output) > 0 else output
        params = lambda: sum(dense_bytes(p) for p in module.parameters(recurse=False))
        if not torch.is_tensor(x) or not torch.is_tensor(out):
            return self._add(dense_bytes_tree(inputs), dense_bytes_tree(output), params())
        in_sparse, out_sparse = self._sparse(x), self._sparse(out)
        fan_out = None                       # weights read per active input
        if isinstance(module, nn.Linear):
            fan_out = module.out_features
        elif isinstance(module, (nn.Conv1d, nn.Conv2d, nn.Conv3d)):
            fan_out = (module.out_channels // module.groups)
            for k in module.kernel_size:
                fan_out *= int(k)
        if fan_out is None:
            if in_sparse or out_sparse:
                self._warn_dense(module)
            return self._add(dense_bytes_tree(inputs), dense_bytes_tree(output), params())
        if not in_sparse:
            return self._add(dense_bytes(x), dense_bytes(out), params())
        rpar = active_element_count(x) * fan_out * int(module.weight.element_size())
        if module.bias is not None:
            rpar += (active_element_count(out) if out_sparse else int(out.numel())) * int(module.bias.element_size())
        self._add(sparse_bytes(x), sparse_bytes(out) if out_sparse else dense_bytes(out), rpar)

    def _warn_dense(self, module):
        if type(module) in self._warned:
            return
        self._warned.add(type(module))
        msg = f"Lemaire forward tracker falls back to dense lower-bound memory for {type(module).__name__}."
        self.warnings.append(msg)
        warnings.warn(msg, RuntimeWarning, stacklevel=3)

    def attach(self, model: nn.Module):
        self.remove()
        self.handles = [m.register_forward_hook(self._hook) for m in model.modules() if isinstance(m, _MEMORY_MODULES)]

    def remove(self):
        for h in self.handles:
            h.remove()
        self.handles = []


class LemaireEnergyProfiler:
    """Context manager: run the model inside it, then ``get_report()``."""

    def __init__(self, *, config: Optional[LemaireEnergyConfig] = None):
        self.config = copy.deepcopy(config or LemaireEnergyConfig())
        self.model: Optional[nn.Module] = None
        self.synop_counter = SynOpCounter()
        self.mac_counter = MACCounter(extra_ignore_modules=[BaseNode])
        self.ac_counter = ACCounter(extra_ignore_modules=[BaseNode])
        self.neuron_state_counter = NeuronStateCounter(
            strict=self.config.strict, extra_state_rules=self.config.extra_state_rules,
            zero_ratio_threshold=self.config.sparse_zero_ratio_threshold,
            enable_sparse_memory_estimation=self.config.enable_sparse_memory_estimation)
        self.addressing_counter = LemaireAddressingCounter()
        self._counters = [self.synop_counter, self.mac_counter, self.ac_counter, self.neuron_state_counter, self.addressing_counter]
        self._mode = DispatchCounterMode(self._counters, strict=self.config.strict)
        self._warnings: List[str] = []
        self._traffic = _TrafficTracker(self.config.sparse_zero_ratio_threshold, self.config.enable_sparse_memory_estimation)

    def bind_model(self, model: nn.Module):
        self.model = model
        for m in model.modules():
            if isinstance(m, BaseNode) and m.backend != "torch":
                msg = (f"LemaireEnergyProfiler only supports torch backend for BaseNode modules, got {m.backend!r} "
                       f"from {m.__class__.__name__}.")
                if self.config.strict:
                    raise ValueError(msg)
                warnings.warn(msg, RuntimeWarning, stacklevel=2)
                self._warnings.append(msg)
                break

    def __enter__(self):
        for c in self._counters:
            c.reset()
        self._mode.__enter__()
        self._traffic.reset()
        if self.model is not None:
            self._traffic.attach(self.model)
        return self

    def __exit__(self, exc_type, exc, tb):
        self._traffic.remove()
        return self._mode.__exit__(exc_type, exc, tb)

    def _snapshot_counts(self):
        proj = self.neuron_state_counter.get_projection_counts().get("Global", {})
        addr = self.addressing_counter.get_metric_counts().get("Global", {})
        t = self._traffic
        counts = {
            "synop": int(self.synop_counter.get_total()), "mac": int(self.mac_counter.get_total()), "ac": int(self.ac_counter.get_total()),
            "state_mac_like": int(proj.get("state_mac_like", 0)), "state_acc_like": int(proj.get("state_acc_like", 0)),
            "read_in_bytes": int(t.read_in), "write_out_bytes": int(t.write_out), "read_params_bytes": int(t.read_params),
            "read_potential_bytes": int(proj.get("read_potential", 0)), "write_potential_bytes": int(proj.get("write_potential", 0)),
            "acc_addr": int(addr.get("acc_addr", 0)), "mac_addr": int(addr.get("mac_addr", 0)),
        }
        buffers = {"inout_buffer_bytes": max(int(t.read_in_buffer_bytes), int(t.write_out_buffer_bytes)),
                   "params_buffer_bytes": int(t.read_params_buffer_bytes),
                   "potential_buffer_bytes": int(proj.get("potential_buffer_bytes", 0))}
        return counts, buffers

    def get_report(self) -> LemaireEnergyReport:
        c, b = self._snapshot_counts()
        cost, t = self.config.cost_config, self._traffic
        mac_pj = cost.e_mul_pj + cost.e_add_pj
        ops = (c["synop"] + c["ac"] + c["state_acc_like"]) * cost.e_add_pj + (c["mac"] + c["state_mac_like"]) * mac_pj
        addressing = c["acc_addr"] * cost.e_add_pj + c["mac_addr"] * mac_pj
        inout = (c["read_in_bytes"] * cost.memory_cost_pj(max(0, t.read_in_buffer_bytes))
                 + c["write_out_bytes"] * cost.memory_cost_pj(max(0, t.write_out_buffer_bytes)))
        params = c["read_params_bytes"] * cost.memory_cost_pj(max(0, b["params_buffer_bytes"]))
        potential = (c["read_potential_bytes"] + c["write_potential_bytes"]) * cost.memory_cost_pj(max(0, b["potential_buffer_bytes"]))
        memory = inout + params + potential
        return LemaireEnergyReport(
            total_pj=ops + addressing + memory,
            breakdown_pj={"ops_pj": ops, "addressing_pj": addressing, "memory_pj": memory, "inout_pj": inout, "params_pj": params,
                          "potential_pj": potential},
            counts=c, buffer_sizes_bytes=b,
            warnings=list(self._warnings) + list(self.neuron_state_counter.warnings) + list(t.warnings))


def estimate_lemaire_energy(model: nn.Module, inputs, *, config: Optional[LemaireEnergyConfig] = None) -> LemaireEnergyReport:
    """One forward pass of ``model(inputs)`` (a tuple / list is unpacked) under the profiler."""
    prof = LemaireEnergyProfiler(config=config)
    prof.bind_model(model)
    with prof:
        model(*inputs) if isinstance(inputs, (tuple, list)) else model(inputs)
    return prof.get_report()
