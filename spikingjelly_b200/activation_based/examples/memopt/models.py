"""CIFAR10-DVS VGG used by the memory-optimisation and distributed examples: eight {Conv-BN -> LIF} blocks (average pooling
folded in front of the convolution where the resolution halves) and a linear classifier applied per time step
(``examples/memopt/models.py:6-84`` of the reference)."""
import torch
import torch.nn as nn

from ... import functional, layer, neuron, surrogate


class VGGBlock(nn.Module):
    def __init__(self, in_plane, out_plane, kernel_size, stride, padding, preceding_avg_pool=False, **kwargs):
        super().__init__()
        mods = [layer.AvgPool2d(2)] if preceding_avg_pool else []
        mods += [layer.Conv2d(in_plane, out_plane, kernel_size, stride, padding), layer.BatchNorm2d(out_plane)]
        self.proj_bn = nn.Sequential(*mods)
        self.neuron = neuron.LIFNode(**kwargs)

    def forward(self, x_seq):
        from spikingjelly_b200.models import _conv_fused as fused
        conv, bn = self.proj_bn[-2], self.proj_bn[-1]
        if fused.eligible(conv, bn, self.neuron, x_seq):
            # channels-last convolution -> fused BatchNorm + LIF kernels (16-bit compute on a CUDA device)
            for m in self.proj_bn[:-2]:
                x_seq = m(x_seq)
            return fused.conv_bn_lif(conv, bn, self.neuron, x_seq)
        return self.neuron(self.proj_bn(x_seq))

    def __spatial_split__(self):
        """The stateless part and the stateful part, for checkpointing that splits a block in space."""
        return self.proj_bn, self.neuron


class CIFAR10DVSVGG(nn.Module):
    def __init__(self, dropout: float = 0.25, tau: float = 1.333, decay_input: bool = False, detach_reset: bool = True,
                 surrogate_function=surrogate.ATan(), backend="cuda", resolution: int = 48):
        super().__init__()
        kw = dict(tau=tau, decay_input=decay_input, detach_reset=detach_reset, surrogate_function=surrogate_function, backend=backend,
                  step_mode="m")
        plan = [(2, 64, False), (64, 128, False), (128, 256, True), (256, 256, False), (256, 512, True), (512, 512, False),
                (512, 512, True), (512, 512, False)]
        self.features = nn.Sequential(*[VGGBlock(i, o, 3, 1, 1, pool, **kw) for i, o, pool in plan], layer.AvgPool2d(2))
        self.features[0].x_compressor = "NullSpikeCompressor"          # the first block sees real-valued frames
        d = resolution // 16
        self.classifier = nn.Sequential(*([nn.Dropout(dropout)] if dropout > 0 else []), nn.Linear(512 * d * d, 10))
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")
        functional.set_step_mode(self, "m")

    def forward(self, input):
        functional.reset_net(self)
        x = self.features(input.transpose(0, 1).contiguous())            # [N, T, C, H, W] -> [T, N, C, H, W]
        return self.classifier(torch.flatten(x, 2))                       # [T, N, 10]
