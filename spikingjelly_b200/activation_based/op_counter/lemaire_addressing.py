"""Address-generation cost of Lemaire et al.'s analytical SNN/ANN energy model: index arithmetic needed to find the
weights and outputs touched by each input.  Event-driven (binary input) layers pay per spike; dense layers pay once per
input and output element (``op_counter/lemaire_addressing.py:14-259``).  Only matmuls issued by ``nn.Linear`` modules
and convolutions issued by ``nn.Conv*d`` modules are counted."""
from __future__ import annotations

from collections import defaultdict
from math import prod
from typing import Dict

import torch
import torch.nn as nn

from .base import BaseCounter, is_binary_tensor

aten = torch.ops.aten
__all__ = ["LemaireAddressingCounter"]

_ZERO = {"acc_addr": 0, "mac_addr": 0}
_MATMULS = {aten.mm.default: 0, aten.bmm.default: 0, aten.addmm.default: 1, aten.baddbmm.default: 1}    # op -> index of the input operand


def _linear(x: torch.Tensor, out: torch.Tensor) -> Dict[str, int]:
    if is_binary_tensor(x):
        return {"acc_addr": int(x.count_nonzero().item()) * int(out.shape[-1]), "mac_addr": 0}
    return {"acc_addr": int(x.numel()) + int(out.numel()), "mac_addr": 0}


def _conv(args, out) -> Dict[str, int]:
    x, w, transposed, groups = args[0], args[1], args[6], args[8]
    if transposed or not torch.is_tensor(x) or not torch.is_tensor(out):
        return dict(_ZERO)
    kvol, oc = prod(w.shape[2:]), int(w.shape[0])
    if is_binary_tensor(x):
        spikes = int(x.count_nonzero().item())
        return {"acc_addr": spikes * (oc // int(groups)) * kvol, "mac_addr": spikes * 2}
    return {"acc_addr": int(x.numel()) + int(out.numel()) + oc * kvol, "mac_addr": 0}


class LemaireAddressingCounter(BaseCounter):
    def __init__(self):
        super().__init__()
        self.rules = {op: None for op in (*_MATMULS, aten.convolution.default)}
        self.ignore_modules = []
        self.metric_records = defaultdict(lambda: defaultdict(int))
        self._pending = None

    def count(self, func, args, kwargs, out, active_modules=None, parent_names=None) -> int:
        active = active_modules or ()
        self._pending = None
        if func in _MATMULS:
            if not any(isinstance(m, nn.Linear) for m in active):
                return 0
            x = args[_MATMULS[func]]
            m = _linear(x, out) if torch.is_tensor(x) and torch.is_tensor(out) else dict(_ZERO)
        elif func == aten.convolution.default:
            if not any(isinstance(m, (nn.Conv1d, nn.Conv2d, nn.Conv3d)) for m in active):
                return 0
            m = _conv(args, out)
        else:
            return 0
        self._pending = {k: int(v) for k, v in m.items()}
        return self._pending["acc_addr"] + self._pending["mac_addr"]

    def record(self, scope, func, value):
        super().record(scope, func, value)
        for k, v in (self._pending or {}).items():
            self.metric_records[scope][k] += v

    def finalize_record(self):
        self._pending = None

    def get_metric_counts(self) -> Dict[str, Dict[str, int]]:
        return {scope: dict(items) for scope, items in self.metric_records.items()}

    def reset(self):
        super().reset()
        self.metric_records = defaultdict(lambda: defaultdict(int))
        self._pending = None
