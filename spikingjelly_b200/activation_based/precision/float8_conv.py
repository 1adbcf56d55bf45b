"""1x1 ``Conv1d`` layers are linear maps over the channel axis: they convert to fp8 linear layers
behind a wrapper that keeps the Conv1d interface (``[N, C, L]`` / ``[T, N, C, L]`` tensors, 3-D
``weight`` in checkpoints).  Parity: ``spikingjelly/activation_based/precision/float8_conv.py:10-128``."""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import layer
from .float8_base import _Float8StepModule

__all__ = ["Float8PointwiseConv1dStepModule", "is_supported_pointwise_conv1d", "make_linear_from_pointwise_conv1d",
           "wrap_float8_pointwise_conv1d_module"]


def is_supported_pointwise_conv1d(module: nn.Module) -> bool:
    return (isinstance(module, (nn.Conv1d, layer.Conv1d)) and module.kernel_size == (1,) and module.stride == (1,)
            and module.padding == (0,) and module.dilation == (1,) and module.groups == 1 and module.padding_mode == "zeros")


def make_linear_from_pointwise_conv1d(conv: nn.Conv1d) -> nn.Linear:
    linear = nn.Linear(conv.in_channels, conv.out_channels, bias=conv.bias is not None, device=conv.weight.device,
                       dtype=conv.weight.dtype)
    with torch.no_grad():
        linear.weight.copy_(conv.weight.squeeze(-1))
        if conv.bias is not None:
            linear.bias.copy_(conv.bias)
    return linear


class Float8PointwiseConv1dStepModule(_Float8StepModule):
    def __init__(self, wrapped: nn.Module, original: nn.Conv1d, step_mode: str = "s"):
        super().__init__(wrapped, step_mode)
        for k in ("in_channels", "out_channels", "kernel_size", "stride", "padding", "dilation", "groups", "padding_mode"):
            setattr(self, k, getattr(original, k))

    @property
    def weight(self):
        return self.wrapped.weight.unsqueeze(-1)        # Conv1d-shaped view of the linear weight

    @property
    def bias(self):
        return getattr(self.wrapped, "bias", None)

    def forward(self, x: torch.Tensor):
        want = {"s": 3, "m": 4}.get(self.step_mode)
        if want is None:
            raise ValueError(f"Unsupported step_mode {self.step_mode!r}.")
        if x.dim() != want:
            shape = "[N, C, L]" if want == 3 else "[T, N, C, L]"
            raise ValueError(f"expected x with shape {shape}, but got x with shape {x.shape}!")
        return self.wrapped(x.transpose(-1, -2).contiguous()).transpose(-1, -2).contiguous()

    def _conv_shaped(self, destination, prefix):
        key = prefix + "weight"
        if key in destination and destination[key].dim() == 2:
            destination[key] = destination[key].unsqueeze(-1)
        return destination

    def state_dict(self, *args, destination=None, prefix="", keep_vars=False):
        return self._conv_shaped(super().state_dict(destination=destination, prefix=prefix, keep_vars=keep_vars), prefix)

    def _save_to_state_dict(self, destination, prefix, keep_vars):
        super()._save_to_state_dict(destination, prefix, keep_vars)
        self._conv_shaped(destination, prefix)

    def _load_from_state_dict(self, state_dict, prefix, *rest):
        key = prefix + "weight"
        if key in state_dict and state_dict[key].dim() == 3:
            state_dict[key] = state_dict[key].squeeze(-1)
        super()._load_from_state_dict(state_dict, prefix, *rest)


def wrap_float8_pointwise_conv1d_module(original: nn.Conv1d, converted: nn.Module) -> nn.Module:
    return Float8PointwiseConv1dStepModule(converted, original, step_mode=original.step_mode if isinstance(original, layer.Conv1d) else "s")
