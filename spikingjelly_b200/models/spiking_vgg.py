"""Spiking VGGs: torchvision's VGG layouts with every ReLU replaced by a spiking neuron.

Parity: ``spikingjelly/activation_based/model/spiking_vgg.py:11-680`` (same constructors,
``features.N`` / ``classifier.N`` module paths, so torchvision VGG checkpoints load unchanged).
"""
from __future__ import annotations

from copy import deepcopy
from typing import Callable

import torch
import torch.nn as nn

from ..activation_based import functional, layer, neuron

__all__ = ["SpikingVGG", "spiking_vgg11", "spiking_vgg11_bn", "spiking_vgg13", "spiking_vgg13_bn", "spiking_vgg16",
           "spiking_vgg16_bn", "spiking_vgg19", "spiking_vgg19_bn", "sequential_forward", "cfgs"]

model_urls = {
    "vgg11": "https://download.pytorch.org/models/vgg11-8a719046.pth",
    "vgg13": "https://download.pytorch.org/models/vgg13-19584684.pth",
    "vgg16": "https://download.pytorch.org/models/vgg16-397923af.pth",
    "vgg19": "https://download.pytorch.org/models/vgg19-dcbb9e9d.pth",
    "vgg11_bn": "https://download.pytorch.org/models/vgg11_bn-6002323d.pth",
    "vgg13_bn": "https://download.pytorch.org/models/vgg13_bn-abd245e5.pth",
    "vgg16_bn": "https://download.pytorch.org/models/vgg16_bn-6c64b313.pth",
    "vgg19_bn": "https://download.pytorch.org/models/vgg19_bn-c79401a0.pth",
}


def _stages(*widths_and_repeats):
    cfg = []
    for width, repeat in widths_and_repeats:
        cfg += [width] * repeat + ["M"]
    return cfg


#: torchvision's configurations A (11 layers), B (13), D (16), E (19)
cfgs = {
    "A": _stages((64, 1), (128, 1), (256, 2), (512, 2), (512, 2)),
    "B": _stages((64, 2), (128, 2), (256, 2), (512, 2), (512, 2)),
    "D": _stages((64, 2), (128, 2), (256, 3), (512, 3), (512, 3)),
    "E": _stages((64, 2), (128, 2), (256, 4), (512, 4), (512, 4)),
}


class SpikingVGG(nn.Module):
    def __init__(self, cfg, batch_norm=False, norm_layer=None, num_classes=1000, init_weights=True,
                 spiking_neuron: Callable = None, **kwargs):
        super().__init__()
        self.features = self.make_layers(cfg=cfg, batch_norm=batch_norm, norm_layer=norm_layer, neuron=spiking_neuron, **kwargs)
        self.avgpool = layer.AdaptiveAvgPool2d((7, 7))
        self.classifier = nn.Sequential(
            layer.Linear(512 * 7 * 7, 4096), spiking_neuron(**deepcopy(kwargs)), layer.Dropout(),
            layer.Linear(4096, 4096), spiking_neuron(**deepcopy(kwargs)), layer.Dropout(),
            layer.Linear(4096, num_classes))
        if init_weights:
            self._initialize_weights()

    def forward(self, x):
        if self.avgpool.step_mode == "m" and torch.is_tensor(x) and x.is_cuda and x.ndim == 5:
            from . import _conv_fused
            feats = _conv_fused.run_sequential(self.features, x)      # fuses conv -> BN -> neuron triples where eligible
        else:
            feats = self.features(x)
        x = self.avgpool(feats)
        x = torch.flatten(x, 1 if self.avgpool.step_mode == "s" else 2)
        return self.classifier(x)

    def _initialize_weights(self):
        for m in self.modules():
            if isinstance(m, layer.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")
                if m.bias is not None:
                    nn.init.constant_(m.bias, 0)
            elif isinstance(m, layer.BatchNorm2d):
                nn.init.constant_(m.weight, 1)
                nn.init.constant_(m.bias, 0)
            elif isinstance(m, layer.Linear):
                nn.init.normal_(m.weight, 0, 0.01)
                nn.init.constant_(m.bias, 0)

    @staticmethod
    def make_layers(cfg, batch_norm=False, norm_layer=None, neuron: Callable = None, **kwargs):
        norm_layer = norm_layer or layer.BatchNorm2d
        mods, in_channels = [], 3
        for v in cfg:
            if v == "M":
                mods.append(layer.MaxPool2d(kernel_size=2, stride=2))
                continue
            mods.append(layer.Conv2d(in_channels, v, kernel_size=3, padding=1))
            if batch_norm:
                mods.append(norm_layer(v))
            mods.append(neuron(**deepcopy(kwargs)))
            in_channels = v
        return nn.Sequential(*mods)


def sequential_forward(sequential: nn.Sequential, x_seq: torch.Tensor) -> torch.Tensor:
    """Run a single-step ``nn.Sequential`` on a sequence: neurons get the sequence, stateless layers
    are applied with time folded into the batch."""
    assert isinstance(sequential, nn.Sequential)
    out = x_seq
    for m in sequential:
        out = m(out) if isinstance(m, neuron.BaseNode) else functional.seq_to_ann_forward(out, m)
    return out


def _spiking_vgg(arch, cfg, batch_norm, pretrained, progress, norm_layer: Callable = None, spiking_neuron: Callable = None,
                 **kwargs):
    if pretrained:
        kwargs["init_weights"] = False
    model = SpikingVGG(cfg=cfgs[cfg], batch_norm=batch_norm, norm_layer=norm_layer if batch_norm else None,
                       spiking_neuron=spiking_neuron, **kwargs)
    if pretrained:
        from torch.hub import load_state_dict_from_url
        model.load_state_dict(load_state_dict_from_url(model_urls[arch], progress=progress))
    return model


def _plain(arch, cfg):
    def make(pretrained=False, progress=True, spiking_neuron: Callable = None, **kwargs):
        return _spiking_vgg(arch, cfg, False, pretrained, progress, None, spiking_neuron, **kwargs)
    make.__name__ = make.__qualname__ = f"spiking_{arch}"
    make.__doc__ = f"Spiking {arch.upper()} (configuration {cfg}); neurons are ``spiking_neuron(**kwargs)``."
    return make


def _with_bn(arch, cfg):
    def make(pretrained=False, progress=True, norm_layer: Callable = None, spiking_neuron: Callable = None, **kwargs):
        return _spiking_vgg(arch, cfg, True, pretrained, progress, norm_layer, spiking_neuron, **kwargs)
    make.__name__ = make.__qualname__ = f"spiking_{arch}"
    make.__doc__ = f"Spiking {arch.upper()} (configuration {cfg}, batch norm); neurons are ``spiking_neuron(**kwargs)``."
    return make


spiking_vgg11, spiking_vgg11_bn = _plain("vgg11", "A"), _with_bn("vgg11_bn", "A")
spiking_vgg13, spiking_vgg13_bn = _plain("vgg13", "B"), _with_bn("vgg13_bn", "B")
spiking_vgg16, spiking_vgg16_bn = _plain("vgg16", "D"), _with_bn("vgg16_bn", "D")
spiking_vgg19, spiking_vgg19_bn = _plain("vgg19", "E"), _with_bn("vgg19_bn", "E")
