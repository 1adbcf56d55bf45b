"""Convolutional SNN on Fashion-MNIST in multi-step mode with the native kernels: {Conv-BN-IF-MaxPool} x 2 -> FC-IF -> FC-IF,
static image repeated T times (role of ``examples/conv_fashion_mnist.py`` in the reference).

    python -m spikingjelly_b200.activation_based.examples.conv_fashion_mnist --synthetic --max-steps 30 --amp
"""
import argparse

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import functional, layer, neuron, surrogate
from ._common import add_common_args, loaders, pick_backend, pick_device, run_epochs, synthetic_images


class CSNN(nn.Module):
    def __init__(self, T: int, channels: int, backend: str):
        super().__init__()
        self.T = T
        sn = lambda: neuron.IFNode(surrogate_function=surrogate.ATan())
        self.conv_fc = nn.Sequential(
            layer.Conv2d(1, channels, 3, padding=1, bias=False), layer.BatchNorm2d(channels), sn(), layer.MaxPool2d(2, 2),
            layer.Conv2d(channels, channels, 3, padding=1, bias=False), layer.BatchNorm2d(channels), sn(), layer.MaxPool2d(2, 2),
            layer.Flatten(), layer.Linear(channels * 7 * 7, channels * 4 * 4, bias=False), sn(),
            layer.Linear(channels * 4 * 4, 10, bias=False), sn())
        functional.set_step_mode(self, "m")
        functional.set_backend(self, backend, instance=neuron.IFNode)

    def forward(self, x):
        return self.conv_fc(x.unsqueeze(0).repeat(self.T, 1, 1, 1, 1)).mean(0)

    def spiking_encoder(self):
        return self.conv_fc[0:3]


def main(argv=None):
    p = add_common_args(argparse.ArgumentParser(description=__doc__))
    p.add_argument("-T", type=int, default=4)
    p.add_argument("--channels", type=int, default=128)
    args = p.parse_args(argv)
    device = pick_device(args.device)
    if args.synthetic:
        train_set, test_set = synthetic_images(2048, (1, 28, 28), 10), synthetic_images(512, (1, 28, 28), 10, seed=1)
    else:
        import torchvision
        tf = torchvision.transforms.ToTensor()
        train_set = torchvision.datasets.FashionMNIST(args.data_dir, train=True, transform=tf, download=True)
        test_set = torchvision.datasets.FashionMNIST(args.data_dir, train=False, transform=tf, download=True)
    net = CSNN(args.T, args.channels, pick_backend(device, args.backend)).to(device)
    loss_fn = lambda out, y: F.mse_loss(out, F.one_hot(y, 10).float())
    return run_epochs(net, *loaders(train_set, test_set, args), lambda n, x: n(x), loss_fn, args, device)


if __name__ == "__main__":
    main()
