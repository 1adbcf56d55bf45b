"""Residual spiking networks: one parameterised builder for both residual styles.

* ``residual="spiking"`` (Spiking ResNet): the shortcut is added to the *pre-activation* of the
  block's last neuron, ``out = sn(bn(conv(..)) + identity)``.
* ``residual="sew"`` (Spike-Element-Wise ResNet): the block's last neuron fires first and the
  shortcut (through its own neuron when it is a projection) is combined with the spikes by
  ``cnf`` in {"ADD", "AND", "IAND"}.

Module names follow torchvision's ResNet (``conv1, bn1, sn1, layer1..4, fc``; blocks
``conv1/bn1/sn1/...``, ``downsample.0/1``, SEW only: ``downsample_sn``) so that torchvision and
SpikingJelly checkpoints load unchanged.

Parity: ``spikingjelly/activation_based/model/sew_resnet.py:41-470``,
``spikingjelly/activation_based/model/spiking_resnet.py:140-480``.
"""
from __future__ import annotations

from copy import deepcopy
from typing import Callable, List, Optional, Sequence, Type

import torch
import torch.nn as nn

from ..activation_based import layer

__all__ = ["sew_function", "conv3x3", "conv1x1", "ResidualSNN", "ARCHS", "build"]


def sew_function(x: torch.Tensor, y: torch.Tensor, cnf: str) -> torch.Tensor:
    if cnf == "ADD":
        return x + y
    if cnf == "AND":
        return x * y
    if cnf == "IAND":
        return x * (1.0 - y)
    raise NotImplementedError(cnf)


def conv3x3(in_planes: int, out_planes: int, stride: int = 1, groups: int = 1, dilation: int = 1) -> layer.Conv2d:
    return layer.Conv2d(in_planes, out_planes, kernel_size=3, stride=stride, padding=dilation, groups=groups, bias=False,
                        dilation=dilation)


def conv1x1(in_planes: int, out_planes: int, stride: int = 1) -> layer.Conv2d:
    return layer.Conv2d(in_planes, out_planes, kernel_size=1, stride=stride, bias=False)


class _Block(nn.Module):
    """conv-bn-sn stages listed in ``self._stages``; subclasses say how the shortcut joins."""
    expansion = 1
    sew = False

    def _finish_init(self, downsample, cnf, spiking_neuron, kwargs, stride):
        self.downsample = downsample
        if self.sew and downsample is not None:
            self.downsample_sn = spiking_neuron(**deepcopy(kwargs))
        self.stride = stride
        self.cnf = cnf

    def forward(self, x):
        out = x
        n = len(self._stages)
        for i, (conv, bn, sn) in enumerate(self._stages):
            out = getattr(self, bn)(getattr(self, conv)(out))
            if i + 1 < n or self.sew:
                out = getattr(self, sn)(out)
        last_sn = getattr(self, self._stages[-1][2])
        if self.sew:
            identity = x if self.downsample is None else self.downsample_sn(self.downsample(x))
            # argument order kept per block type: it matters for the non-commutative IAND
            return sew_function(identity, out, self.cnf) if self._identity_first else sew_function(out, identity, self.cnf)
        identity = x if self.downsample is None else self.downsample(x)
        return last_sn(out + identity)

    def extra_repr(self) -> str:
        return f"cnf={self.cnf}" if self.sew else ""


def _make_basic(sew: bool):
    class BasicBlock(_Block):
        expansion = 1
        _stages = (("conv1", "bn1", "sn1"), ("conv2", "bn2", "sn2"))
        _identity_first = True

        def __init__(self, inplanes, planes, stride=1, downsample=None, groups=1, base_width=64, dilation=1, norm_layer=None,
                     cnf: str = None, spiking_neuron: Callable = None, **kwargs):
            super().__init__()
            norm_layer = norm_layer or layer.BatchNorm2d
            if groups != 1 or base_width != 64:
                raise ValueError("BasicBlock only supports groups=1 and base_width=64")
            if dilation > 1:
                raise NotImplementedError("Dilation > 1 not supported in BasicBlock")
            self.conv1 = conv3x3(inplanes, planes, stride)
            self.bn1 = norm_layer(planes)
            self.sn1 = spiking_neuron(**deepcopy(kwargs))
            self.conv2 = conv3x3(planes, planes)
            self.bn2 = norm_layer(planes)
            self.sn2 = spiking_neuron(**deepcopy(kwargs))
            self._finish_init(downsample, cnf, spiking_neuron, kwargs, stride)
    BasicBlock.sew = sew
    return BasicBlock


def _make_bottleneck(sew: bool):
    class Bottleneck(_Block):
        """ResNet v1.5: the stride sits on the 3x3 convolution."""
        expansion = 4
        _stages = (("conv1", "bn1", "sn1"), ("conv2", "bn2", "sn2"), ("conv3", "bn3", "sn3"))
        _identity_first = False

        def __init__(self, inplanes, planes, stride=1, downsample=None, groups=1, base_width=64, dilation=1, norm_layer=None,
                     cnf: str = None, spiking_neuron: Callable = None, **kwargs):
            super().__init__()
            norm_layer = norm_layer or layer.BatchNorm2d
            width = int(planes * (base_width / 64.0)) * groups
            self.conv1 = conv1x1(inplanes, width)
            self.bn1 = norm_layer(width)
            self.sn1 = spiking_neuron(**deepcopy(kwargs))
            self.conv2 = conv3x3(width, width, stride, groups, dilation)
            self.bn2 = norm_layer(width)
            self.sn2 = spiking_neuron(**deepcopy(kwargs))
            self.conv3 = conv1x1(width, planes * self.expansion)
            self.bn3 = norm_layer(planes * self.expansion)
            self.sn3 = spiking_neuron(**deepcopy(kwargs))
            self._finish_init(downsample, cnf, spiking_neuron, kwargs, stride)
    Bottleneck.sew = sew
    return Bottleneck


def _without_cnf(block):
    """The plain spiking ResNet blocks have no connect function, and no ``cnf`` parameter in front of ``spiking_neuron``."""
    class Block(block):
        def __init__(self, inplanes, planes, stride=1, downsample=None, groups=1, base_width=64, dilation=1, norm_layer=None,
                     spiking_neuron: Callable = None, **kwargs):
            kwargs.pop("cnf", None)
            super().__init__(inplanes, planes, stride, downsample, groups, base_width, dilation, norm_layer, None, spiking_neuron, **kwargs)
    Block.__name__, Block.__qualname__, Block.__doc__ = block.__name__, block.__qualname__, block.__doc__
    return Block


SEWBasicBlock, SEWBottleneck = _make_basic(True), _make_bottleneck(True)
SpikingBasicBlock, SpikingBottleneck = _without_cnf(_make_basic(False)), _without_cnf(_make_bottleneck(False))


class ResidualSNN(nn.Module):
    """torchvision-shaped ResNet trunk with spiking neurons.  ``in_channels`` (default 3) is an
    addition for event data (2 polarity channels); the default keeps checkpoint shapes."""

    def __init__(self, block: Type[_Block], layers: Sequence[int], num_classes: int = 1000, zero_init_residual: bool = False,
                 groups: int = 1, width_per_group: int = 64, replace_stride_with_dilation: Optional[List[bool]] = None,
                 norm_layer=None, cnf: str = None, spiking_neuron: Callable = None, in_channels: int = 3, **kwargs):
        super().__init__()
        norm_layer = norm_layer or layer.BatchNorm2d
        self._norm_layer = norm_layer
        self.inplanes, self.dilation = 64, 1
        if replace_stride_with_dilation is None:
            replace_stride_with_dilation = [False, False, False]
        if len(replace_stride_with_dilation) != 3:
            raise ValueError("replace_stride_with_dilation should be None or a 3-element tuple, got {}".format(
                replace_stride_with_dilation))
        self.groups, self.base_width = groups, width_per_group
        self.conv1 = layer.Conv2d(in_channels, self.inplanes, kernel_size=7, stride=2, padding=3, bias=False)
        self.bn1 = norm_layer(self.inplanes)
        self.sn1 = spiking_neuron(**deepcopy(kwargs))
        self.maxpool = layer.MaxPool2d(kernel_size=3, stride=2, padding=1)
        common = dict(cnf=cnf, spiking_neuron=spiking_neuron, **kwargs)
        self.layer1 = self._make_layer(block, 64, layers[0], **common)
        self.layer2 = self._make_layer(block, 128, layers[1], stride=2, dilate=replace_stride_with_dilation[0], **common)
        self.layer3 = self._make_layer(block, 256, layers[2], stride=2, dilate=replace_stride_with_dilation[1], **common)
        self.layer4 = self._make_layer(block, 512, layers[3], stride=2, dilate=replace_stride_with_dilation[2], **common)
        self.avgpool = layer.AdaptiveAvgPool2d((1, 1))
        self.fc = layer.Linear(512 * block.expansion, num_classes)
        for m in self.modules():
            if isinstance(m, layer.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")
            elif isinstance(m, (layer.BatchNorm2d, layer.GroupNorm)):
                nn.init.constant_(m.weight, 1)
                nn.init.constant_(m.bias, 0)
        if zero_init_residual:                      # residual branches start as identities
            for m in self.modules():
                if isinstance(m, _Block):
                    nn.init.constant_(getattr(m, m._stages[-1][1]).weight, 0)

    def _make_layer(self, block, planes, blocks, stride=1, dilate=False, cnf=None, spiking_neuron=None, **kwargs):
        norm_layer, downsample, previous_dilation = self._norm_layer, None, self.dilation
        if dilate:
            self.dilation *= stride
            stride = 1
        if stride != 1 or self.inplanes != planes * block.expansion:
            downsample = nn.Sequential(conv1x1(self.inplanes, planes * block.expansion, stride),
                                       norm_layer(planes * block.expansion))
        stack = [block(self.inplanes, planes, stride, downsample, self.groups, self.base_width, previous_dilation, norm_layer,
                       cnf=cnf, spiking_neuron=spiking_neuron, **kwargs)]
        self.inplanes = planes * block.expansion
        for _ in range(1, blocks):
            stack.append(block(self.inplanes, planes, groups=self.groups, base_width=self.base_width, dilation=self.dilation,
                               norm_layer=norm_layer, cnf=cnf, spiking_neuron=spiking_neuron, **kwargs))
        return nn.Sequential(*stack)

    def _forward_impl(self, x):
        x = self.maxpool(self.sn1(self.bn1(self.conv1(x))))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        x = self.avgpool(x)
        x = torch.flatten(x, 1 if self.avgpool.step_mode == "s" else 2)
        return self.fc(x)

    def forward(self, x):
        if x.is_cuda and x.ndim == 5:
            from . import _resnet_fused
            if _resnet_fused.eligible(self, x):
                return _resnet_fused.forward(self, x)
        return self._forward_impl(x)


#: arch name -> (bottleneck?, layers, extra kwargs)
ARCHS = {
    "resnet18": (False, [2, 2, 2, 2], {}),
    "resnet34": (False, [3, 4, 6, 3], {}),
    "resnet50": (True, [3, 4, 6, 3], {}),
    "resnet101": (True, [3, 4, 23, 3], {}),
    "resnet152": (True, [3, 8, 36, 3], {}),
    "resnext50_32x4d": (True, [3, 4, 6, 3], dict(groups=32, width_per_group=4)),
    "resnext101_32x8d": (True, [3, 4, 23, 3], dict(groups=32, width_per_group=8)),
    "wide_resnet50_2": (True, [3, 4, 6, 3], dict(width_per_group=128)),
    "wide_resnet101_2": (True, [3, 4, 23, 3], dict(width_per_group=128)),
}

model_urls = {
    "resnet18": "https://download.pytorch.org/models/resnet18-f37072fd.pth",
    "resnet34": "https://download.pytorch.org/models/resnet34-b627a593.pth",
    "resnet50": "https://download.pytorch.org/models/resnet50-0676ba61.pth",
    "resnet101": "https://download.pytorch.org/models/resnet101-63fe2227.pth",
    "resnet152": "https://download.pytorch.org/models/resnet152-394f9c45.pth",
    "resnext50_32x4d": "https://download.pytorch.org/models/resnext50_32x4d-7cdf4587.pth",
    "resnext101_32x8d": "https://download.pytorch.org/models/resnext101_32x8d-8ba56ff5.pth",
    "wide_resnet50_2": "https://download.pytorch.org/models/wide_resnet50_2-95faca4d.pth",
    "wide_resnet101_2": "https://download.pytorch.org/models/wide_resnet101_2-32ee1156.pth",
}


def load_pretrained(model: nn.Module, arch: str, progress: bool = True) -> None:
    """ANN weights from torchvision's model zoo (needs network access)."""
    from torch.hub import load_state_dict_from_url
    model.load_state_dict(load_state_dict_from_url(model_urls[arch], progress=progress))


def build(cls, sew: bool, arch: str, pretrained: bool, progress: bool, cnf, spiking_neuron, **kwargs):
    bottleneck, layers, extra = ARCHS[arch]
    block = (SEWBottleneck if bottleneck else SEWBasicBlock) if sew else (SpikingBottleneck if bottleneck else SpikingBasicBlock)
    kwargs = {**kwargs, **extra}
    model = cls(block, layers, cnf=cnf, spiking_neuron=spiking_neuron, **kwargs) if sew else \
        cls(block, layers, spiking_neuron=spiking_neuron, **kwargs)
    if pretrained:
        load_pretrained(model, arch, progress)
    return model
