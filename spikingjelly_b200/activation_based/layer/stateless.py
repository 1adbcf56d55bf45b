"""Step-mode aware versions of stateless ``torch.nn`` layers.

Each class subclasses the torch layer (so parameters, buffers and ``state_dict`` keys
are identical) and adds ``step_mode``.  In multi-step mode ``[T, N, *]`` is folded to
``[T*N, *]`` — a view — so the layer runs once over all time steps.

The wrappers are generated from one template; ``_WRAPPED`` lists (torch class,
tensor rank expected in multi-step mode, shape text for the error message).
Parity: ``spikingjelly/activation_based/layer/stateless_wrapper.py:52-1451``.
"""
from __future__ import annotations

import inspect
from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from .. import base, functional

__all__ = [
    "Conv1d", "Conv2d", "Conv3d", "Upsample", "ConvTranspose1d", "ConvTranspose2d", "ConvTranspose3d",
    "GroupNorm", "MaxPool1d", "MaxPool2d", "MaxPool3d", "MaxUnpool1d", "MaxUnpool2d", "MaxUnpool3d",
    "AvgPool1d", "AvgPool2d", "AvgPool3d", "AdaptiveAvgPool1d", "AdaptiveAvgPool2d", "AdaptiveAvgPool3d",
    "Linear", "Flatten", "WSConv2d", "WSLinear",
]


def _split_step_mode(torch_cls, args, kwargs):
    """``step_mode`` may be given by keyword or as one extra trailing positional."""
    step_mode = kwargs.pop("step_mode", "s")
    names = [n for n in inspect.signature(torch_cls.__init__).parameters if n not in ("self", "device", "dtype")]
    if len(args) == len(names) + 1:
        *args, step_mode = args
    return tuple(args), kwargs, step_mode


def _wrap(torch_cls, name: str, m_rank: Optional[int], shape_txt: str = ""):
    def __init__(self, *args, **kwargs):
        args, kwargs, step_mode = _split_step_mode(torch_cls, args, kwargs)
        torch_cls.__init__(self, *args, **kwargs)
        self.step_mode = step_mode

    def extra_repr(self):
        return torch_cls.extra_repr(self) + f", step_mode={self.step_mode}"

    def forward(self, x: Tensor):
        if self.step_mode == "s":
            return torch_cls.forward(self, x)
        if m_rank is not None and x.dim() != m_rank:
            raise ValueError(f"expected x with shape {shape_txt}, but got x with shape {x.shape}!")
        return functional.seq_to_ann_forward(x, lambda t: torch_cls.forward(self, t))

    doc = f"``torch.nn.{torch_cls.__name__}`` with ``step_mode`` ('s': ``[N, *]``, 'm': ``[T, N, *]``)."
    return type(name, (torch_cls, base.StepModule),
                {"__init__": __init__, "extra_repr": extra_repr, "forward": forward, "__doc__": doc,
                 "__module__": __name__})


def _wrap_unpool(torch_cls, name: str, m_rank: int, shape_txt: str):
    def __init__(self, kernel_size, stride=None, padding=0, step_mode="s"):
        torch_cls.__init__(self, kernel_size, stride, padding)
        self.step_mode = step_mode

    def extra_repr(self):
        return torch_cls.extra_repr(self) + f", step_mode={self.step_mode}"

    def forward(self, x: Tensor, indices: Tensor, output_size: Optional[Sequence[int]] = None):
        if self.step_mode == "s":
            return torch_cls.forward(self, x, indices, output_size)
        if x.dim() != m_rank:
            raise ValueError(f"expected x with shape {shape_txt}, but got x with shape {x.shape}!")
        if indices.shape != x.shape:
            raise ValueError(f"expected indices with the same shape as x ({x.shape}), "
                             f"but got indices with shape {indices.shape}!")
        return functional.seq_to_ann_forward(
            (x, indices), lambda v, i: torch_cls.forward(self, v, i, output_size))

    return type(name, (torch_cls, base.StepModule),
                {"__init__": __init__, "extra_repr": extra_repr, "forward": forward, "__module__": __name__,
                 "__doc__": f"``torch.nn.{torch_cls.__name__}`` with ``step_mode``."})


_L, _HW, _DHW = "[T, N, C, L]", "[T, N, C, H, W]", "[T, N, C, D, H, W]"
Conv1d = _wrap(nn.Conv1d, "Conv1d", 4, _L)
Conv2d = _wrap(nn.Conv2d, "Conv2d", 5, _HW)
Conv3d = _wrap(nn.Conv3d, "Conv3d", 6, _DHW)
Upsample = _wrap(nn.Upsample, "Upsample", None)
ConvTranspose1d = _wrap(nn.ConvTranspose1d, "ConvTranspose1d", 4, _L)
ConvTranspose2d = _wrap(nn.ConvTranspose2d, "ConvTranspose2d", 5, _HW)
ConvTranspose3d = _wrap(nn.ConvTranspose3d, "ConvTranspose3d", 6, _DHW)
GroupNorm = _wrap(nn.GroupNorm, "GroupNorm", None)
MaxPool1d = _wrap(nn.MaxPool1d, "MaxPool1d", 4, _L)
MaxPool2d = _wrap(nn.MaxPool2d, "MaxPool2d", 5, _HW)
MaxPool3d = _wrap(nn.MaxPool3d, "MaxPool3d", 6, _DHW)
MaxUnpool1d = _wrap_unpool(nn.MaxUnpool1d, "MaxUnpool1d", 4, _L)
MaxUnpool2d = _wrap_unpool(nn.MaxUnpool2d, "MaxUnpool2d", 5, _HW)
MaxUnpool3d = _wrap_unpool(nn.MaxUnpool3d, "MaxUnpool3d", 6, _DHW)
AvgPool1d = _wrap(nn.AvgPool1d, "AvgPool1d", 4, _L)
AvgPool2d = _wrap(nn.AvgPool2d, "AvgPool2d", 5, _HW)
AvgPool3d = _wrap(nn.AvgPool3d, "AvgPool3d", 6, _DHW)
AdaptiveAvgPool1d = _wrap(nn.AdaptiveAvgPool1d, "AdaptiveAvgPool1d", 4, _L)
AdaptiveAvgPool2d = _wrap(nn.AdaptiveAvgPool2d, "AdaptiveAvgPool2d", 5, _HW)
AdaptiveAvgPool3d = _wrap(nn.AdaptiveAvgPool3d, "AdaptiveAvgPool3d", 6, _DHW)
Flatten = _wrap(nn.Flatten, "Flatten", None)


class Linear(nn.Linear, base.StepModule):
    """``nn.Linear`` already broadcasts over leading axes, so both step modes share one
    forward; ``step_mode`` is kept for uniform tree walks."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, step_mode="s", **kw) -> None:
        super().__init__(in_features, out_features, bias, **kw)
        self.step_mode = step_mode

    def forward(self, x: Tensor) -> Tensor:
        dtype = _native_linear_dtype(x, self.weight)
        if dtype is None:
            return F.linear(x, self.weight, self.bias)
        from ...ops import gemm
        y = gemm.linear(x.to(dtype), self.weight.to(dtype))
        return y if self.bias is None else y + self.bias.to(dtype)


def _native_linear_dtype(x: Tensor, weight: Tensor) -> Optional[torch.dtype]:
    """The 16-bit dtype in which the tensor-core kernel should compute this product, or ``None`` for the library path."""
    from ... import configure
    if not (configure.native_linear and x.is_cuda and weight.is_cuda) or x.dim() < 2:
        return None
    if weight.shape[0] % 8 or weight.shape[1] % 8 or x.numel() == 0:
        return None
    if torch.is_autocast_enabled("cuda"):
        dtype = torch.get_autocast_dtype("cuda")
    elif x.dtype == weight.dtype:
        dtype = x.dtype
    else:
        return None
    if dtype not in (torch.bfloat16, torch.float16):
        return None
    from ... import ops
    return dtype if ops.available() else None


def _standardize(weight: Tensor, gain: Optional[Tensor], eps: float) -> Tensor:
    """Zero-mean, ``1/sqrt(fan_in)``-scaled weights per output unit, times ``gain``."""
    dims = tuple(range(1, weight.dim()))
    fan_in = weight[0].numel()
    mean = weight.mean(dim=dims, keepdim=True)
    var = weight.var(dim=dims, keepdim=True)
    w = (weight - mean) / ((var * fan_in + eps) ** 0.5)
    return w if gain is None else w * gain


class WSConv2d(Conv2d):
    """Conv2d with weight standardisation (learnable per-filter ``gain``)."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True,
                 padding_mode="zeros", step_mode="s", gain: bool = True, eps: float = 1e-4) -> None:
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias,
                         padding_mode, step_mode=step_mode)
        self.gain = nn.Parameter(torch.ones(self.out_channels, 1, 1, 1)) if gain else None
        self.eps = eps

    def get_weight(self):
        return _standardize(self.weight, self.gain, self.eps)

    def _forward(self, x: Tensor):
        return F.conv2d(x, self.get_weight(), self.bias, self.stride, self.padding, self.dilation, self.groups)

    def forward(self, x: Tensor):
        if self.step_mode == "s":
            return self._forward(x)
        if x.dim() != 5:
            raise ValueError(f"expected x with shape {_HW}, but got x with shape {x.shape}!")
        return functional.seq_to_ann_forward(x, self._forward)


class WSLinear(Linear):
    """Linear with weight standardisation."""

    def __init__(self, in_features, out_features, bias=True, step_mode="s", gain=True, eps=1e-4) -> None:
        super().__init__(in_features, out_features, bias, step_mode)
        self.gain = nn.Parameter(torch.ones(self.out_features, 1)) if gain else None
        self.eps = eps

    def get_weight(self):
        return _standardize(self.weight, self.gain, self.eps)

    def forward(self, x: Tensor):
        return F.linear(x, self.get_weight(), self.bias)
