"""Spike-Element-Wise ResNets (Fang et al., NeurIPS 2021).

Parity: ``spikingjelly/activation_based/model/sew_resnet.py:13-904`` (same constructors, module
names and state_dict keys; ``in_channels`` is an added keyword with default 3).
"""
from __future__ import annotations

from typing import Callable

from . import _resnet_family as _f
from ._resnet_family import conv1x1, conv3x3, sew_function  # noqa: F401

__all__ = ["SEWResNet", "sew_resnet18", "sew_resnet34", "sew_resnet50", "sew_resnet101", "sew_resnet152",
           "sew_resnext50_32x4d", "sew_resnext101_32x8d", "sew_wide_resnet50_2", "sew_wide_resnet101_2"]

BasicBlock, Bottleneck = _f.SEWBasicBlock, _f.SEWBottleneck
model_urls = _f.model_urls


class SEWResNet(_f.ResidualSNN):
    """``SEWResNet(block, layers, ..., cnf="ADD", spiking_neuron=neuron.IFNode, **neuron_kwargs)``"""


def _sew_resnet(arch, block, layers, pretrained, progress, cnf, spiking_neuron, **kwargs):
    model = SEWResNet(block, layers, cnf=cnf, spiking_neuron=spiking_neuron, **kwargs)
    if pretrained:
        _f.load_pretrained(model, arch, progress)
    return model


def _factory(arch: str, doc: str):
    def make(pretrained: bool = False, progress: bool = True, cnf: str = None, spiking_neuron: Callable = None, **kwargs):
        return _f.build(SEWResNet, True, arch, pretrained, progress, cnf, spiking_neuron, **kwargs)
    make.__name__ = make.__qualname__ = f"sew_{arch}"
    make.__doc__ = (f"{doc}  ``cnf``: 'ADD' | 'AND' | 'IAND'; ``spiking_neuron``: neuron class, built with "
                    "``**kwargs`` (keywords that ResNet itself understands, e.g. ``num_classes``, ``zero_init_residual``, "
                    "``in_channels``, are consumed by the network).")
    return make


sew_resnet18 = _factory("resnet18", "SEW ResNet-18.")
sew_resnet34 = _factory("resnet34", "SEW ResNet-34.")
sew_resnet50 = _factory("resnet50", "SEW ResNet-50.")
sew_resnet101 = _factory("resnet101", "SEW ResNet-101.")
sew_resnet152 = _factory("resnet152", "SEW ResNet-152.")
sew_resnext50_32x4d = _factory("resnext50_32x4d", "SEW ResNeXt-50 32x4d.")
sew_resnext101_32x8d = _factory("resnext101_32x8d", "SEW ResNeXt-101 32x8d.")
sew_wide_resnet50_2 = _factory("wide_resnet50_2", "SEW Wide ResNet-50-2.")
sew_wide_resnet101_2 = _factory("wide_resnet101_2", "SEW Wide ResNet-101-2.")
