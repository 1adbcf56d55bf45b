"""The networks of "Incorporating Learnable Membrane Time Constant to Enhance Learning of Spiking
Neural Networks" (Fang et al., ICCV 2021): conv-BN-neuron-pool stacks, two dropout+linear+neuron
stages and a voting layer, all inside one ``conv_fc`` Sequential.

Parity: ``spikingjelly/activation_based/model/parametric_lif_net.py:11-300`` (identical
``conv_fc.N`` state_dict keys).
"""
from __future__ import annotations

from copy import deepcopy
from typing import Callable

import torch
import torch.nn as nn

from ..activation_based import layer

__all__ = ["MNISTNet", "FashionMNISTNet", "NMNISTNet", "CIFAR10Net", "CIFAR10DVSNet", "DVSGestureNet"]


def _conv_stack(in_channels, channels, groups, convs_per_group, make_neuron):
    mods = []
    for _ in range(groups):
        for _ in range(convs_per_group):
            mods += [layer.Conv2d(in_channels, channels, kernel_size=3, padding=1, bias=False), layer.BatchNorm2d(channels),
                     make_neuron()]
            in_channels = channels
        mods.append(layer.MaxPool2d(2, 2))
    return mods


def _head(in_features, hidden, out_features, voter, make_neuron):
    return [layer.Flatten(), layer.Dropout(0.5), layer.Linear(in_features, hidden), make_neuron(), layer.Dropout(0.5),
            layer.Linear(hidden, out_features), make_neuron(), voter]


class _PLIFNet(nn.Module):
    def forward(self, x: torch.Tensor):
        return self.conv_fc(x)


class MNISTNet(_PLIFNet):
    """28x28x1 input: {c3-BN-SN-MP}x2 - DP-FC2048-SN - DP-FC100-SN - vote(10)."""

    def __init__(self, channels=128, spiking_neuron: Callable = None, **kwargs):
        super().__init__()
        sn = lambda: spiking_neuron(**deepcopy(kwargs))
        self.conv_fc = nn.Sequential(*_conv_stack(1, channels, 2, 1, sn), *_head(channels * 7 * 7, 2048, 100, layer.VotingLayer(), sn))


class FashionMNISTNet(MNISTNet):
    """Same network as ``MNISTNet``."""


class NMNISTNet(MNISTNet):
    """34x34x2 event frames cropped to 32x32: first conv takes 2 channels, FC takes 8x8 maps."""

    def __init__(self, channels=128, spiking_neuron: Callable = None, **kwargs):
        super().__init__(channels, spiking_neuron, **kwargs)
        self.conv_fc[0] = layer.Conv2d(2, channels, kernel_size=3, padding=1, bias=False)
        self.conv_fc[-6] = layer.Linear(channels * 8 * 8, 2048)


class CIFAR10Net(_PLIFNet):
    """32x32x3 input: {{c3-BN-SN}x3-MP}x2 - DP-FC2048-SN - DP-FC100-SN - vote(10)."""

    def __init__(self, channels=256, spiking_neuron: Callable = None, **kwargs):
        super().__init__()
        sn = lambda: spiking_neuron(**deepcopy(kwargs))
        self.conv_fc = nn.Sequential(*_conv_stack(3, channels, 2, 3, sn), *_head(channels * 8 * 8, 2048, 100, layer.VotingLayer(10), sn))


class CIFAR10DVSNet(_PLIFNet):
    """128x128x2 event frames: {c3-BN-SN-MP}x4 - DP-FC512-SN - DP-FC100-SN - vote(10)."""

    def __init__(self, channels=128, spiking_neuron: Callable = None, **kwargs):
        super().__init__()
        sn = lambda: spiking_neuron(**deepcopy(kwargs))
        self.conv_fc = nn.Sequential(*_conv_stack(2, channels, 4, 1, sn), *_head(channels * 8 * 8, 512, 100, layer.VotingLayer(10), sn))


class DVSGestureNet(_PLIFNet):
    """128x128x2 event frames: {c3-BN-SN-MP}x5 - DP-FC512-SN - DP-FC110-SN - vote(10) (11 classes)."""

    def __init__(self, channels=128, spiking_neuron: Callable = None, **kwargs):
        super().__init__()
        sn = lambda: spiking_neuron(**deepcopy(kwargs))
        self.conv_fc = nn.Sequential(*_conv_stack(2, channels, 5, 1, sn), *_head(channels * 4 * 4, 512, 110, layer.VotingLayer(10), sn))


def test_models():
    """Builds every network of this file with IF neurons and runs one batch in both step modes; returns
    ``{name: (single-step output shape, multi-step output shape)}``."""
    import torch

    from ..activation_based import functional, neuron, surrogate
    shapes = {"MNISTNet": (1, 28, 28), "FashionMNISTNet": (1, 28, 28), "NMNISTNet": (2, 32, 32), "CIFAR10Net": (3, 32, 32),
              "CIFAR10DVSNet": (2, 128, 128), "DVSGestureNet": (2, 128, 128)}
    out = {}
    for name, chw in shapes.items():
        net = globals()[name](16, neuron.IFNode, surrogate_function=surrogate.ATan())
        with torch.no_grad():
            single = tuple(net(torch.rand(2, *chw)).shape)
            functional.reset_net(net)
            functional.set_step_mode(net, "m")
            multi = tuple(net(torch.rand(3, 2, *chw)).shape)
        out[name] = (single, multi)
    return out
