"""Spiking ResNets: torchvision ResNets with every ReLU replaced by a spiking neuron.

Parity: ``spikingjelly/activation_based/model/spiking_resnet.py:13-1003`` (same constructors,
module names and state_dict keys; ``in_channels`` is an added keyword with default 3).
"""
from __future__ import annotations

from typing import Callable

from . import _resnet_family as _f
from ._resnet_family import conv1x1, conv3x3  # noqa: F401

__all__ = ["SpikingResNet", "spiking_resnet18", "spiking_resnet34", "spiking_resnet50", "spiking_resnet101",
           "spiking_resnet152", "spiking_resnext50_32x4d", "spiking_resnext101_32x8d", "spiking_wide_resnet50_2",
           "spiking_wide_resnet101_2"]

BasicBlock, Bottleneck = _f.SpikingBasicBlock, _f.SpikingBottleneck
model_urls = _f.model_urls


class SpikingResNet(_f.ResidualSNN):
    """``SpikingResNet(block, layers, ..., spiking_neuron=neuron.IFNode, **neuron_kwargs)``"""

    def __init__(self, block, layers, num_classes=1000, zero_init_residual=False, groups=1, width_per_group=64,
                 replace_stride_with_dilation=None, norm_layer=None, spiking_neuron: Callable = None, **kwargs):
        super().__init__(block, layers, num_classes, zero_init_residual, groups, width_per_group, replace_stride_with_dilation,
                         norm_layer, cnf=None, spiking_neuron=spiking_neuron, **kwargs)


def _spiking_resnet(arch, block, layers, pretrained, progress, spiking_neuron, **kwargs):
    model = SpikingResNet(block, layers, spiking_neuron=spiking_neuron, **kwargs)
    if pretrained:
        _f.load_pretrained(model, arch, progress)
    return model


def _factory(arch: str, doc: str):
    def make(pretrained: bool = False, progress: bool = True, spiking_neuron: Callable = None, **kwargs):
        return _f.build(SpikingResNet, False, arch, pretrained, progress, None, spiking_neuron, **kwargs)
    make.__name__ = make.__qualname__ = f"spiking_{arch}"
    make.__doc__ = f"{doc}  ``spiking_neuron``: neuron class, built with the remaining ``**kwargs``."
    return make


spiking_resnet18 = _factory("resnet18", "Spiking ResNet-18.")
spiking_resnet34 = _factory("resnet34", "Spiking ResNet-34.")
spiking_resnet50 = _factory("resnet50", "Spiking ResNet-50.")
spiking_resnet101 = _factory("resnet101", "Spiking ResNet-101.")
spiking_resnet152 = _factory("resnet152", "Spiking ResNet-152.")
spiking_resnext50_32x4d = _factory("resnext50_32x4d", "Spiking ResNeXt-50 32x4d.")
spiking_resnext101_32x8d = _factory("resnext101_32x8d", "Spiking ResNeXt-101 32x8d.")
spiking_wide_resnet50_2 = _factory("wide_resnet50_2", "Spiking Wide ResNet-50-2.")
spiking_wide_resnet101_2 = _factory("wide_resnet101_2", "Spiking Wide ResNet-101-2.")
