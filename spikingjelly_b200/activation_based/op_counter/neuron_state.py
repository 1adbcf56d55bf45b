"""Cost of keeping neuron state: every ATen operator that runs inside a spiking neuron (torch backend) and touches one
of its state tensors is classified as a state read / write / add / multiply / compare / non-linearity / select, and
as spike-triggered (driven by a sparse tensor, e.g. a reset gated by the spike) or dense per time step.

A state tensor is a value of the module's registered memories, anything materialised by ``zeros_like`` / ``full_like``
at the start of a functional step, and every tensor later written from a state (tracked by storage identity through
weak references).  Per scope two tables are kept: the raw metrics and a projection on the vocabulary of analytical
energy models (``read_potential``, ``write_potential``, ``state_mac_like``, ``state_acc_like``,
``potential_buffer_bytes``).  Same contract as ``op_counter/neuron_state.py:138-610`` of the reference.
"""
from __future__ import annotations

import warnings
import weakref
from collections import defaultdict
from typing import Any, Callable, Dict, Optional

import torch
import torch.nn as nn
from torch.overrides import resolve_name

from ..neuron.base_node import BaseNode
from ._sparse_memory import active_element_count, dense_bytes, is_sparse_access_tensor
from .base import BaseCounter, _collect_tensors

__all__ = ["NeuronStateCounter"]

aten = torch.ops.aten

_VIEW_PREFIXES = ("aten.detach", "aten.view", "aten.alias", "aten._unsafe_view", "aten.as_strided", "aten.expand", "aten.slice",
                  "aten.select.int", "aten.select_copy", "aten.unsqueeze", "aten.squeeze", "aten.transpose", "aten.permute",
                  "aten.lift_fresh")


def _overloads(packets, names):
    found = set()
    for p in packets:
        for n in names:
            op = getattr(getattr(aten, p, None), n, None)
            if op is not None:
                found.add(op)
    return found


#: operator -> (metric it adds its output size to, does it write a state)
_KIND: Dict[Any, tuple] = {}
for _op in _overloads(("add", "add_", "sub", "sub_", "rsub"), ("Tensor", "Scalar")):
    _KIND[_op] = ("state_adds", True)
for _op in _overloads(("mul", "mul_", "div", "div_"), ("Tensor", "Scalar")):
    _KIND[_op] = ("state_muls", True)
for _op in _overloads(("eq", "ne", "lt", "le", "gt", "ge"), ("Tensor", "Scalar")):
    _KIND[_op] = ("state_comps", False)
for _op in _overloads(("sigmoid", "rsqrt", "sqrt", "exp", "tanh"), ("default",)):
    _KIND[_op] = ("state_nonlinear_ops", False)
for _op in _overloads(("sigmoid_", "sqrt_", "exp_", "tanh_"), ("default",)):
    _KIND[_op] = ("state_nonlinear_ops", True)
for _op in _overloads(("where",), ("self", "ScalarOther", "ScalarSelf")):
    _KIND[_op] = ("state_select_ops", True)
for _op in (aten.clone.default, aten.copy_.default, aten._to_copy.default):
    _KIND[_op] = (None, True)
_MATERIALISE = {aten.full_like.default, aten.zeros_like.default}
_METRICS = ("state_reads", "state_writes", "state_adds", "state_muls", "state_comps", "state_nonlinear_ops", "state_reset_ops",
            "state_select_ops", "spike_triggered_ops", "timestep_dense_ops")


def _storage_key(x: torch.Tensor):
    try:
        ptr = id(x) if x.is_meta else x.untyped_storage().data_ptr()
    except (RuntimeError, AttributeError):
        ptr = id(x)
    return (x.device.type, x.device.index, x.dtype, ptr)


class NeuronStateCounter(BaseCounter):
    def __init__(self, *, strict: bool = False, extra_state_rules: Optional[Dict[type, Callable]] = None,
                 zero_ratio_threshold: float = 0.5, enable_sparse_memory_estimation: bool = True):
        super().__init__()
        self.strict, self.zero_ratio_threshold = strict, zero_ratio_threshold
        self.enable_sparse_memory_estimation = enable_sparse_memory_estimation
        for t, rule in (extra_state_rules or {}).items():
            if not callable(rule):
                raise TypeError(f"extra_state_rules values must be callable, got {type(rule).__name__} for {t.__name__}.")
        self.extra_state_rules = dict(extra_state_rules or {})
        self.reset()

    def has_rule(self, func) -> bool:
        return True

    def _complain(self, module, message: str):
        if self.strict:
            raise ValueError(message)
        if id(module) not in self._warned_modules:
            self._warned_modules.add(id(module))
            self.warnings.append(message)
            warnings.warn(message, RuntimeWarning, stacklevel=3)

    def _nothing(self) -> int:
        self._pending_metrics = self._pending_projection = None
        return 0

    def _state_keys(self, nodes) -> set:
        keys = {_storage_key(v) for m in nodes for v in m._memories.values() if torch.is_tensor(v)}
        alive = [(r, r()) for r in self._functional_state_refs]
        self._functional_state_refs = [r for r, t in alive if t is not None]
        keys.update(_storage_key(t) for _, t in alive if t is not None)
        return keys

    def count(self, func, args, kwargs, out, active_modules=None, parent_names=None) -> int:
        nodes = [m for m in (active_modules or ()) if isinstance(m, BaseNode)]
        if not nodes:
            return self._nothing()
        for m in nodes:
            if m.backend is not None and m.backend != "torch":
                self._complain(m, f"NeuronStateCounter only supports torch backend, got {m.backend!r} from {m.__class__.__name__}.")
                return self._nothing()
        keys = self._state_keys(nodes)
        if not keys and func in _MATERIALISE:
            fresh = _collect_tensors(out)[0]
            self._functional_state_refs.append(weakref.ref(fresh))
            keys.add(_storage_key(fresh))
        if not keys:
            return self._nothing()
        for m in nodes:
            rule = self.extra_state_rules.get(type(m))
            if rule is not None:
                breakdown = rule(m, func, args, kwargs, out, keys)
                if breakdown is not None:
                    return self._store(breakdown)
        if resolve_name(func).startswith(_VIEW_PREFIXES):
            return self._nothing()

        inputs = _collect_tensors((args, kwargs))
        copy_into_state = func is aten.copy_.default and args and torch.is_tensor(args[0]) and _storage_key(args[0]) in keys
        if copy_into_state:
            sources = [x for x in _collect_tensors((args[1:], kwargs)) if _storage_key(x) in keys]
            targets = [args[0]]
        else:
            sources, targets = [x for x in inputs if _storage_key(x) in keys], []
        if not sources and not targets:
            return self._nothing()
        outputs = targets if copy_into_state else _collect_tensors(out)
        out_numel = sum(int(x.numel()) for x in _collect_tensors(out))
        drivers = [x for x in inputs if _storage_key(x) not in keys and self.enable_sparse_memory_estimation
                   and is_sparse_access_tensor(x, zero_ratio_threshold=self.zero_ratio_threshold)]
        active = max((active_element_count(x) for x in drivers), default=0)
        touched = lambda ts: sum(min(active, int(x.numel())) * int(x.element_size()) for x in ts)
        if copy_into_state:
            reads, out_bytes = sum(dense_bytes(x) for x in sources), sum(dense_bytes(x) for x in targets)
        elif drivers:
            reads, out_bytes = touched(sources), touched(outputs)
        else:
            reads, out_bytes = sum(dense_bytes(x) for x in sources), sum(dense_bytes(x) for x in _collect_tensors(out))
        metrics = dict.fromkeys(_METRICS, 0)
        metrics["state_reads"] = reads
        metric, writes = _KIND.get(func, (None, False))
        if metric is not None:
            metrics[metric] += out_numel
        if writes and outputs:
            metrics["state_writes"] += out_bytes
            self._functional_state_refs.extend(weakref.ref(t) for t in outputs)
            if drivers:                                   # gated by spikes: a reset-like, event-driven update
                metrics["state_reset_ops"] += out_numel
                metrics["spike_triggered_ops"] += out_numel
            else:
                metrics["timestep_dense_ops"] += out_numel
        if not any(metrics.values()):
            return self._nothing()
        return self._store(metrics, state_buffer_bytes=max((dense_bytes(x) for x in sources + targets), default=0))

    def _store(self, metrics: Dict[str, int], *, state_buffer_bytes: int = 0) -> int:
        self._pending_metrics = metrics
        self._pending_projection = {
            "read_potential": metrics.get("state_reads", 0), "write_potential": metrics.get("state_writes", 0),
            "state_mac_like": metrics.get("state_muls", 0), "potential_buffer_bytes": state_buffer_bytes,
            "state_acc_like": sum(metrics.get(k, 0) for k in ("state_adds", "state_comps", "state_nonlinear_ops", "state_select_ops")),
        }
        return sum(metrics.values())

    def record(self, scope, func, value):
        super().record(scope, func, value)
        for k, v in (self._pending_metrics or {}).items():
            self.metric_records[scope][k] += int(v)
        for k, v in (self._pending_projection or {}).items():
            if k == "potential_buffer_bytes":
                self.projection_records[scope][k] = max(self.projection_records[scope][k], int(v))
            else:
                self.projection_records[scope][k] += int(v)

    def finalize_record(self):
        self._pending_metrics = self._pending_projection = None

    def get_metric_counts(self) -> Dict[str, Dict[str, int]]:
        return {scope: dict(items) for scope, items in self.metric_records.items()}

    def get_projection_counts(self) -> Dict[str, Dict[str, int]]:
        return {scope: dict(items) for scope, items in self.projection_records.items()}

    def get_extra_counts(self) -> Dict[str, Dict[str, int]]:
        return self.get_projection_counts()

    def reset(self):
        super().reset()
        self.metric_records = defaultdict(lambda: defaultdict(int))
        self.projection_records = defaultdict(lambda: defaultdict(int))
        self.warnings, self._warned_modules = [], set()
        self._pending_metrics = self._pending_projection = None
        self._functional_state_refs = []
