"""VGG family for online training through time (OTTT): weight-standardised convolutions followed by an online LIF
neuron and a constant gain of 2.74 that restores unit variance after the neuron; the whole network is an
``OTTTSequential`` so that presynaptic traces travel with the spikes
(``spikingjelly/activation_based/model/spiking_vggws_ottt.py:23-579``).  Layouts: torchvision's A / B / D / E plus the
paper's 8-convolution ``S`` with average pooling."""
from __future__ import annotations

from copy import deepcopy

import torch.nn as nn

from ..activation_based import layer, neuron

__all__ = ["OTTTSpikingVGG", "ottt_spiking_vgg11", "ottt_spiking_vgg11_ws", "ottt_spiking_vgg13", "ottt_spiking_vgg13_ws",
           "ottt_spiking_vgg16", "ottt_spiking_vgg16_ws", "ottt_spiking_vgg19", "ottt_spiking_vgg19_ws", "ottt_spiking_vggws"]

WS_GAIN = 2.74


class Scale(nn.Module):
    def __init__(self, scale):
        super().__init__()
        self.scale = scale

    def forward(self, x):
        return x * self.scale


def _vgg_layout(blocks, pool="M"):
    out = []
    for width, n in blocks:
        out += [width] * n + [pool]
    return out


cfgs = {
    "A": _vgg_layout([(64, 1), (128, 1), (256, 2), (512, 2), (512, 2)]),
    "B": _vgg_layout([(64, 2), (128, 2), (256, 2), (512, 2), (512, 2)]),
    "D": _vgg_layout([(64, 2), (128, 2), (256, 3), (512, 3), (512, 3)]),
    "E": _vgg_layout([(64, 2), (128, 2), (256, 4), (512, 4), (512, 4)]),
    "S": [64, 128, "A", 256, 256, "A", 512, 512, "A", 512, 512],
}


class OTTTSpikingVGG(nn.Module):
    def __init__(self, cfg, weight_standardization=True, num_classes=1000, init_weights=True, spiking_neuron: callable = None,
                 light_classifier=True, drop_rate=0.0, **kwargs):
        super().__init__()
        self.fc_hw = kwargs.get("fc_hw", 1)
        gain = WS_GAIN if weight_standardization else 1.0
        self.neuron = spiking_neuron
        self.features = self.make_layers(cfg=cfg, weight_standardization=weight_standardization, neuron=spiking_neuron,
                                         drop_rate=drop_rate, **kwargs)
        if light_classifier:
            head = [layer.AdaptiveAvgPool2d((self.fc_hw, self.fc_hw)), layer.Flatten(1), layer.Linear(512 * self.fc_hw ** 2, num_classes)]
        else:
            Linear = layer.WSLinear if weight_standardization else layer.Linear
            head = [layer.AdaptiveAvgPool2d((7, 7)), layer.Flatten(1)]
            for fan_in in (512 * 7 * 7, 4096):
                head += [Linear(fan_in, 4096), spiking_neuron(**deepcopy(kwargs)), Scale(gain), layer.Dropout()]
            head.append(layer.Linear(4096, num_classes))
        self.classifier = layer.OTTTSequential(*head)
        if init_weights:
            self._initialize_weights()

    def forward(self, x):
        return self.classifier(self.features(x))

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
    def make_layers(cfg, weight_standardization=True, neuron: callable = None, drop_rate=0.0, **kwargs):
        Conv2d = layer.WSConv2d if weight_standardization else layer.Conv2d
        layers, in_channels = [], 3
        for v in cfg:
            if v == "M":
                layers.append(layer.MaxPool2d(kernel_size=2, stride=2))
            elif v == "A":
                layers.append(layer.AvgPool2d(kernel_size=2, stride=2))
            else:
                layers += [Conv2d(in_channels, v, kernel_size=3, padding=1), neuron(**deepcopy(kwargs))]
                if weight_standardization:
                    layers.append(Scale(WS_GAIN))
                if drop_rate > 0.0:
                    layers.append(layer.Dropout(drop_rate))
                in_channels = v
        return layer.OTTTSequential(*layers)


def _spiking_vgg(cfg, weight_standardization, spiking_neuron, **kwargs):
    return OTTTSpikingVGG(cfg=cfgs[cfg], weight_standardization=weight_standardization, spiking_neuron=spiking_neuron, **kwargs)


def ottt_spiking_vggws(spiking_neuron: callable = neuron.OTTTLIFNode, **kwargs):
    """The 8-convolution network of the OTTT paper (weight standardisation, average pooling, linear head)."""
    return _spiking_vgg("S", True, spiking_neuron, light_classifier=True, **kwargs)


def _factory(cfg: str, ws: bool, name: str):
    def build(spiking_neuron: callable = neuron.OTTTLIFNode, **kwargs):
        return _spiking_vgg(cfg, ws, spiking_neuron, light_classifier=False, **kwargs)
    build.__name__ = build.__qualname__ = name
    build.__doc__ = f"OTTT VGG, layout {cfg}, {'with' if ws else 'without'} weight standardisation, three-layer classifier."
    return build


ottt_spiking_vgg11, ottt_spiking_vgg11_ws = _factory("A", False, "ottt_spiking_vgg11"), _factory("A", True, "ottt_spiking_vgg11_ws")
ottt_spiking_vgg13, ottt_spiking_vgg13_ws = _factory("B", False, "ottt_spiking_vgg13"), _factory("B", True, "ottt_spiking_vgg13_ws")
ottt_spiking_vgg16, ottt_spiking_vgg16_ws = _factory("D", False, "ottt_spiking_vgg16"), _factory("D", True, "ottt_spiking_vgg16_ws")
ottt_spiking_vgg19, ottt_spiking_vgg19_ws = _factory("E", False, "ottt_spiking_vgg19"), _factory("E", True, "ottt_spiking_vgg19_ws")
