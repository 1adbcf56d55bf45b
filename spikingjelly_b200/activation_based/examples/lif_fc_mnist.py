"""One fully connected layer of LIF neurons on MNIST with Poisson-encoded inputs and a rate-coded MSE loss — the
"hello world" of the framework (role of ``examples/lif_fc_mnist.py`` in the reference).

    python -m spikingjelly_b200.activation_based.examples.lif_fc_mnist --synthetic --epochs 1 --max-steps 50
"""
import argparse

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import encoding, layer, neuron, surrogate
from ._common import add_common_args, loaders, pick_backend, pick_device, run_epochs, synthetic_images


class SNN(nn.Module):
    def __init__(self, tau: float, backend: str):
        super().__init__()
        self.layer = nn.Sequential(layer.Flatten(), layer.Linear(28 * 28, 10, bias=False),
                                   neuron.LIFNode(tau=tau, surrogate_function=surrogate.ATan(), backend=backend))

    def forward(self, x):
        return self.layer(x)


def main(argv=None):
    p = add_common_args(argparse.ArgumentParser(description=__doc__))
    p.add_argument("-T", type=int, default=100)
    p.add_argument("--tau", type=float, default=2.0)
    args = p.parse_args(argv)
    device = pick_device(args.device)
    backend = pick_backend(device, args.backend)
    if args.synthetic:
        train_set, test_set = synthetic_images(2048, (1, 28, 28), 10), synthetic_images(512, (1, 28, 28), 10, seed=1)
    else:
        import torchvision
        tf = torchvision.transforms.ToTensor()
        train_set = torchvision.datasets.MNIST(args.data_dir, train=True, transform=tf, download=True)
        test_set = torchvision.datasets.MNIST(args.data_dir, train=False, transform=tf, download=True)
    net = SNN(args.tau, "torch").to(device)              # single-step neuron inside a Python time loop: stochastic input per step
    enc = encoding.PoissonEncoder()

    def forward(net, img):
        rate = 0.0
        for _ in range(args.T):
            rate = rate + net(enc(img))
        return rate / args.T

    loss_fn = lambda out, y: F.mse_loss(out, F.one_hot(y, 10).float())
    return run_epochs(net, *loaders(train_set, test_set, args), forward, loss_fn, args, device)


if __name__ == "__main__":
    main()
