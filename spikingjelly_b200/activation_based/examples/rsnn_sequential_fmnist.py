"""Row-by-row ("sequential") image classification with recurrent spiking networks: an image ``[H, W]`` is presented as
``T = H`` time steps of ``W`` pixels.  Three models, as in the reference's ``examples/rsnn_sequential_fmnist.py`` and
``examples/spiking_lstm_sequential_mnist.py``:

* ``plain``    Linear -> LIF -> Linear -> LIF (no recurrence, memory only in the membrane potentials)
* ``feedback`` the first LIF's spikes are fed back into its input through ``layer.LinearRecurrentContainer``
* ``lstm``     ``rnn.SpikingLSTM`` followed by a linear read-out of the last hidden state

    python -m spikingjelly_b200.activation_based.examples.rsnn_sequential_fmnist --model feedback --synthetic --max-steps 20
"""
from __future__ import annotations

import argparse

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import functional, layer, neuron, rnn, surrogate
from . import _common as C


class PlainNet(nn.Module):
    def __init__(self, width: int, hidden: int, classes: int):
        super().__init__()
        self.fc = nn.Sequential(layer.Linear(width, hidden), neuron.LIFNode(surrogate_function=surrogate.ATan()),
                                layer.Linear(hidden, classes), neuron.LIFNode(surrogate_function=surrogate.ATan()))

    def forward(self, x_seq):                                   # [T, N, W] -> mean firing rate [N, classes]
        return self.fc(x_seq).mean(0)


class FeedbackNet(nn.Module):
    def __init__(self, width: int, hidden: int, classes: int):
        super().__init__()
        self.rec = layer.LinearRecurrentContainer(
            nn.Sequential(layer.Linear(width, hidden), neuron.LIFNode(surrogate_function=surrogate.ATan(), detach_reset=True)),
            in_features=width, out_features=hidden, bias=True, step_mode="m")
        self.out = nn.Sequential(layer.Linear(hidden, classes), neuron.LIFNode(surrogate_function=surrogate.ATan()))

    def forward(self, x_seq):
        return self.out(self.rec(x_seq)).mean(0)


class LSTMNet(nn.Module):
    def __init__(self, width: int, hidden: int, classes: int):
        super().__init__()
        self.lstm = rnn.SpikingLSTM(width, hidden, 1)
        self.fc = nn.Linear(hidden, classes)

    def forward(self, x_seq):
        y, _ = self.lstm(x_seq)
        return self.fc(y[-1])


def main(argv=None) -> dict:
    p = C.add_common_args(argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter))
    p.add_argument("--model", default="feedback", choices=["plain", "feedback", "lstm"])
    p.add_argument("--hidden", type=int, default=64)
    p.add_argument("--dataset", default="fmnist", choices=["fmnist", "mnist"])
    a = p.parse_args(argv)
    device = C.pick_device(a.device)
    if a.synthetic:
        train_set, test_set = C.synthetic_images(512, (28, 28), 10, 0), C.synthetic_images(128, (28, 28), 10, 0)
    else:
        import torchvision
        ds = torchvision.datasets.FashionMNIST if a.dataset == "fmnist" else torchvision.datasets.MNIST
        tf = torchvision.transforms.ToTensor()
        train_set, test_set = ds(a.data_dir, True, tf, download=True), ds(a.data_dir, False, tf, download=True)
    train, test = C.loaders(train_set, test_set, a)
    net = {"plain": PlainNet, "feedback": FeedbackNet, "lstm": LSTMNet}[a.model](28, a.hidden, 10).to(device)
    functional.set_step_mode(net, "m")
    if a.model == "plain":
        functional.set_backend(net, C.pick_backend(device, a.backend))

    def forward(net, x):
        x = x.reshape(x.shape[0], 28, 28).permute(1, 0, 2)       # [T = rows, N, W]
        return net(x)

    loss = (lambda out, y: F.cross_entropy(out, y)) if a.model == "lstm" else (lambda out, y: F.mse_loss(out, F.one_hot(y, 10).float()))
    return C.run_epochs(net, train, test, forward, loss, a, device)


if __name__ == "__main__":
    main()
