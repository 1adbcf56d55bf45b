"""Containers that lift single-step modules to sequences.

Parity: ``spikingjelly/activation_based/layer/container.py:29-431``.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.nn as nn
from torch import Tensor

from .. import base, functional

__all__ = ["MultiStepContainer", "SeqToANNContainer", "TLastMultiStepContainer", "TLastSeqToANNContainer",
           "StepModeContainer", "ElementWiseRecurrentContainer", "LinearRecurrentContainer"]


def _require_single_step(block: nn.Sequential) -> None:
    for m in block:
        if getattr(m, "step_mode", "s") != "s":
            raise ValueError(f"{type(m).__name__}.step_mode must be 's' inside this container.")


class _SeqContainer(nn.Sequential, base.MultiStepModule):
    """``nn.Sequential`` of single-step modules driven by ``_lift`` (set by subclasses)."""
    _lift = None

    def __init__(self, *args):
        super().__init__(*args)
        _require_single_step(self)
        self._step_mode = "m"

    def _chain(self, x):
        return nn.Sequential.forward(self, x)

    def forward(self, x_seq: Tensor):
        return type(self)._lift(x_seq, self._chain)


class MultiStepContainer(_SeqContainer):
    """Call the wrapped chain once per time step (for stateful single-step modules)."""
    _lift = staticmethod(functional.multi_step_forward)


class SeqToANNContainer(_SeqContainer):
    """Fold ``T`` into the batch and call the wrapped (stateless) chain once."""
    _lift = staticmethod(functional.seq_to_ann_forward)


class TLastSeqToANNContainer(_SeqContainer):
    _lift = staticmethod(functional.t_last_seq_to_ann_forward)


class TLastMultiStepContainer(_SeqContainer):
    _lift = staticmethod(functional.t_last_multi_step_forward)


class StepModeContainer(nn.Sequential, base.StepModule):
    """Chain of single-step modules with a switchable step mode.  ``stateful`` selects the
    multi-step strategy (loop vs fold).  ``functional.set_step_mode`` sets the container but
    leaves its children in single-step mode."""

    def __init__(self, stateful: bool, step_mode: str = "s", *args):
        super().__init__(*args)
        self.stateful = stateful
        _require_single_step(self)
        self.step_mode = step_mode

    def forward(self, x: torch.Tensor):
        chain = lambda t: nn.Sequential.forward(self, t)  # noqa: E731
        if self.step_mode == "s":
            return chain(x)
        if self.stateful:
            return functional.multi_step_forward(x, chain)
        return functional.seq_to_ann_forward(x, chain)


class ElementWiseRecurrentContainer(base.MemoryModule):
    """Self-recurrence ``y_t = f(g(y_{t-1}, x_t))`` with an element-wise ``g`` and memory ``y``."""

    def __init__(self, sub_module: nn.Module, element_wise_function: Callable, step_mode="s"):
        super().__init__()
        self.step_mode = step_mode
        assert not hasattr(sub_module, "step_mode") or sub_module.step_mode == "s"
        self.sub_module = sub_module
        self.element_wise_function = element_wise_function
        self.register_memory("y", None)

    def materialize_states(self, inputs, states, step_mode):
        x = inputs[0] if step_mode == "s" else inputs[0][0]
        return (torch.zeros_like(x) if states[0] is None else states[0],)

    def single_step_functional_forward(self, inputs, states, **kwargs):
        y = self.sub_module(self.element_wise_function(states[0], inputs[0]))
        return (y,), (y,)

    def extra_repr(self) -> str:
        return f"element-wise function={self.element_wise_function}, step_mode={self.step_mode}"


class LinearRecurrentContainer(base.MemoryModule):
    """``y_t = f(W [x_t ; y_{t-1}])`` with ``W = rc: Linear(in + out, in)``."""

    def __init__(self, sub_module: nn.Module, in_features: int, out_features: int, bias: bool = True,
                 step_mode="s") -> None:
        super().__init__()
        self.step_mode = step_mode
        assert not hasattr(sub_module, "step_mode") or sub_module.step_mode == "s"
        self.sub_module_out_features = out_features
        self.rc = nn.Linear(in_features + out_features, in_features, bias)
        self.sub_module = sub_module
        self.register_memory("y", None)

    def materialize_states(self, inputs, states, step_mode):
        x = inputs[0] if step_mode == "s" else inputs[0][0]
        y = states[0]
        return (x.new_zeros(*x.shape[:-1], self.sub_module_out_features) if y is None else y,)

    def single_step_functional_forward(self, inputs, states, **kwargs):
        y = self.sub_module(self.rc(torch.cat((inputs[0], states[0]), dim=-1)))
        return (y,), (y,)

    def extra_repr(self) -> str:
        return f", step_mode={self.step_mode}"
