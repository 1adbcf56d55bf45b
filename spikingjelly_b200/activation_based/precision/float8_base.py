"""Step-mode wrappers around converted linear modules.  A wrapper is transparent for checkpoints:
its state-dict keys are the wrapped module's (no ``wrapped.`` prefix), and attribute look-ups fall
through to the wrapped module.  Parity: ``spikingjelly/activation_based/precision/float8_base.py:9-90``."""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import functional, layer

__all__ = ["Float8LinearStepModule", "wrap_float8_linear_module"]


class _Float8StepModule(nn.Module):
    def __init__(self, wrapped: nn.Module, step_mode: str):
        super().__init__()
        self.wrapped = wrapped
        self.step_mode = step_mode

    def set_step_mode(self, step_mode: str):
        self.step_mode = step_mode

    def __getattr__(self, name: str):
        try:
            return super().__getattr__(name)
        except AttributeError:
            wrapped = self.__dict__.get("_modules", {}).get("wrapped")
            if wrapped is None:
                raise AttributeError(f"'{type(self).__name__}' object has no attribute '{name}'") from None
            return getattr(wrapped, name)

    def state_dict(self, *args, destination=None, prefix="", keep_vars=False):
        return self.wrapped.state_dict(destination=destination, prefix=prefix, keep_vars=keep_vars)

    def _save_to_state_dict(self, destination, prefix, keep_vars):
        self.wrapped._save_to_state_dict(destination, prefix, keep_vars)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        # route "<prefix>weight" to "<prefix>wrapped.weight" so that nn.Module's recursive loader finds it
        inner = prefix + "wrapped."
        own = set(self.wrapped.state_dict().keys())
        for k in [k for k in list(state_dict.keys()) if k.startswith(prefix) and not k.startswith(inner)]:
            if k[len(prefix):] in own:
                state_dict[inner + k[len(prefix):]] = state_dict.pop(k)


class Float8LinearStepModule(_Float8StepModule):
    """``step_mode='s'``: ``wrapped(x)``; ``'m'``: time folded into the batch around the call."""

    def __init__(self, wrapped: nn.Module, step_mode: str = "s"):
        super().__init__(wrapped, step_mode)

    def forward(self, x: torch.Tensor):
        if self.step_mode == "s":
            return self.wrapped(x)
        if self.step_mode == "m":
            return functional.seq_to_ann_forward(x, self.wrapped)
        raise ValueError(f"Unsupported step_mode {self.step_mode!r}.")


def wrap_float8_linear_module(original: nn.Module, converted: nn.Module) -> nn.Module:
    if isinstance(original, layer.Linear):
        return Float8LinearStepModule(converted, step_mode=original.step_mode)
    if isinstance(original, nn.Linear):
        return Float8LinearStepModule(converted, step_mode="s")
    return converted
