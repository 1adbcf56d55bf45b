"""Step-mode wrappers around converted linear modules that stay invisible in checkpoints
(``spikingjelly/activation_based/precision/float8_base.py:9-87``): a model whose ``nn.Linear`` became a wrapped low-precision
module saves and loads exactly the keys of the original model.

The transparency is done with state-dict hooks rather than by overriding ``state_dict`` itself: after saving, the
``wrapped.`` segment is cut out of this module's keys; before loading, it is put back in."""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import functional, layer

__all__ = ["Float8LinearStepModule", "wrap_float8_linear_module"]

_INNER = "wrapped."


def _hide_inner_segment(module, state_dict, prefix, local_metadata):
    inner = prefix + _INNER
    for key in [k for k in state_dict if k.startswith(inner)]:
        state_dict[prefix + key[len(inner):]] = state_dict.pop(key)


def _restore_inner_segment(module, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
    inner = prefix + _INNER
    expected = set(module.wrapped.state_dict().keys())
    for key in [k for k in state_dict if k.startswith(prefix) and not k.startswith(inner)]:
        tail = key[len(prefix):]
        if tail in expected:
            state_dict[inner + tail] = state_dict.pop(key)


class _Float8StepModule(nn.Module):
    """Holds the converted module as ``wrapped``; unknown attributes (``weight``, ``in_features`` ...) are looked up there."""

    def __init__(self, wrapped: nn.Module, step_mode: str):
        super().__init__()
        self.wrapped = wrapped
        self.step_mode = step_mode
        self._register_state_dict_hook(_hide_inner_segment)
        self.register_load_state_dict_pre_hook(_restore_inner_segment)

    def set_step_mode(self, step_mode: str):
        self.step_mode = step_mode

    def __getattr__(self, name: str):
        try:
            return super().__getattr__(name)
        except AttributeError:
            inner = self.__dict__.get("_modules", {}).get("wrapped")
            if inner is None or name == "wrapped":
                raise
            return getattr(inner, name)


class Float8LinearStepModule(_Float8StepModule):
    """Single-step: ``wrapped(x)``.  Multi-step: the time axis is folded into the batch around the call."""

    def __init__(self, wrapped: nn.Module, step_mode: str = "s"):
        super().__init__(wrapped, step_mode)

    def forward(self, x: torch.Tensor):
        if self.step_mode == "m":
            return functional.seq_to_ann_forward(x, self.wrapped)
        if self.step_mode == "s":
            return self.wrapped(x)
        raise ValueError(f"step_mode is 's' or 'm', not {self.step_mode!r}")


def wrap_float8_linear_module(original: nn.Module, converted: nn.Module) -> nn.Module:
    """Give ``converted`` the step-mode behaviour ``original`` had (``layer.Linear``: its mode; ``nn.Linear``: single step)."""
    if isinstance(original, nn.Linear):
        return Float8LinearStepModule(converted, step_mode=getattr(original, "step_mode", "s") if isinstance(original, layer.Linear) else "s")
    return converted
