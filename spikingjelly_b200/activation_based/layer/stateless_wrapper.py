"""Import path of the reference's ``spikingjelly/activation_based/layer/stateless_wrapper.py``: the names below live in the ``layer`` package here."""
from . import (  # noqa: F401
    Conv1d, Conv2d, Conv3d, Upsample, ConvTranspose1d, ConvTranspose2d, ConvTranspose3d, GroupNorm,
    MaxPool1d, MaxPool2d, MaxPool3d, MaxUnpool1d, MaxUnpool2d, MaxUnpool3d, AvgPool1d, AvgPool2d,
    AvgPool3d, AdaptiveAvgPool1d, AdaptiveAvgPool2d, AdaptiveAvgPool3d, Linear, Flatten, WSConv2d,
    WSLinear)

__all__ = ['Conv1d', 'Conv2d', 'Conv3d', 'Upsample', 'ConvTranspose1d', 'ConvTranspose2d', 'ConvTranspose3d',
           'GroupNorm', 'MaxPool1d', 'MaxPool2d', 'MaxPool3d', 'MaxUnpool1d', 'MaxUnpool2d', 'MaxUnpool3d',
           'AvgPool1d', 'AvgPool2d', 'AvgPool3d', 'AdaptiveAvgPool1d', 'AdaptiveAvgPool2d',
           'AdaptiveAvgPool3d', 'Linear', 'Flatten', 'WSConv2d', 'WSLinear']
