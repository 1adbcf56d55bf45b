"""Spike-based backpropagation with leak-corrected activation derivatives (Lee et al., "Enabling Spike-based
Backpropagation for Training Deep Neural Network Architectures", 2020) on a spiking ResNet-11 for CIFAR-10.  Counterpart of
the reference's ``examples/cifar10_r11_enabling_spikebased_backpropagation.py``.

How the rule works.  Images are Poisson-coded into signed spikes for ``T`` steps.  A neuron integrates, fires when its
potential exceeds the threshold (hard reset), then leaks ``(v - v_reset) / tau`` - the leak is treated as a constant in
backward.  The graph spans all ``T`` steps (potentials accumulate across them); every firing LIF neuron scales the gradient
of each of its spikes by an *accumulated* derivative computed after the last step from two running quantities: the spike
count ``a`` and the leak-corrected potential ``a_l``::

    d spike / d net = [a_l > 0] + log(1 - 1 / tau) * a_l / max(a, 1)

The output layer does not fire; its final potential divided by ``T`` is compared with the one-hot label by MSE.

    python -m spikingjelly_b200.activation_based.examples.cifar10_r11_enabling_spikebased_backpropagation --data-dir ./cifar10 -T 100

Without ``torchvision`` / the dataset on disk, ``--synthetic`` trains on generated colour-blob classes (used by the test).
``--width`` scales the channel counts (64 = the paper's network).
"""
from __future__ import annotations

import argparse
import math
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import functional, layer

__all__ = ["PassThroughSpike", "AccumulatingLIF", "FirstLayerIF", "ResNet11", "poisson_signed", "train_step", "main"]


class PassThroughSpike(torch.autograd.Function):
    """Heaviside forward; backward passes the gradient where the neuron was above threshold and blocks it elsewhere."""

    @staticmethod
    def forward(ctx, over):
        ctx.save_for_backward(over > 0)
        return (over > 0).to(over.dtype)

    @staticmethod
    def backward(ctx, g):
        (fired,) = ctx.saved_tensors
        return g * fired


class _Membrane(nn.Module):
    """State shared by the two neuron kinds.  ``reset()`` is what ``functional.reset_net`` calls."""

    def __init__(self, v_threshold: float, v_reset: float):
        super().__init__()
        self.v_threshold, self.v_reset = v_threshold, v_reset
        self.reset()

    def reset(self) -> None:
        self.v = self.v_reset
        self.count = 0.0            # spikes emitted so far
        self.leaky_count = 0.0      # leak-corrected potential + spike of the last step
        self.scale: Optional[torch.Tensor] = None

    def _fire(self) -> torch.Tensor:
        over = self.v - self.v_threshold
        spike = PassThroughSpike.apply(over)
        self.v = torch.where(over > 0, torch.full_like(self.v, self.v_reset), self.v)
        return spike


class AccumulatingLIF(_Membrane):
    """Leaky neuron of the paper.  ``fire=False``: a read-out that only integrates and leaks and returns its potential."""

    def __init__(self, tau: float = 100.0, v_threshold: float = 1.0, v_reset: float = 0.0, fire: bool = True):
        super().__init__(v_threshold, v_reset)
        self.tau, self.fire = tau, fire

    def forward(self, dv: torch.Tensor) -> torch.Tensor:
        self.v = self.v + dv
        spike = None
        if self.fire:
            spike = self._fire()
            self.count = self.count + spike.detach()
            self.leaky_count = (self.v - (self.v - self.v_reset) / self.tau + spike).detach()
        self.v = self.v - ((self.v - self.v_reset) / self.tau).detach()
        if not self.fire:
            return self.v
        if self.training and spike.requires_grad:
            spike.register_hook(lambda g: g * self.scale)
        return spike

    def finish_sequence(self) -> None:
        """Fix the accumulated derivative used by the hook of the last step (call once, after the last forward)."""
        if self.fire and torch.is_tensor(self.count):
            count = self.count + (self.count < 1e-3).to(self.count.dtype)
            self.scale = (self.leaky_count > 1e-3).to(count.dtype) + math.log(1.0 - 1.0 / self.tau) * self.leaky_count / count


class FirstLayerIF(_Membrane):
    """Non-leaky neuron after the first average pooling."""

    def __init__(self, v_threshold: float = 0.75, v_reset: float = 0.0):
        super().__init__(v_threshold, v_reset)

    def forward(self, dv: torch.Tensor) -> torch.Tensor:
        self.v = self.v + dv
        return self._fire()


def _spiking(p_drop: float) -> nn.Sequential:
    return nn.Sequential(AccumulatingLIF(), layer.Dropout(p_drop))


class _Residual(nn.Module):
    """conv3x3 -> LIF -> conv3x3 (stride) added to a 1x1 / pooling shortcut, then LIF."""

    def __init__(self, c_in: int, c_out: int, stride: int, p_drop: float):
        super().__init__()
        self.conv1 = nn.Conv2d(c_in, c_out, 3, 1, 1, bias=False)
        self.lif1 = _spiking(p_drop)
        self.conv2 = nn.Conv2d(c_out, c_out, 3, stride, 1, bias=False)
        self.shortcut = nn.Conv2d(c_in, c_out, 1, stride, bias=False) if c_in != c_out else nn.AvgPool2d(1, stride)
        self.lif2 = _spiking(p_drop)

    def forward(self, x):
        return self.lif2(self.conv2(self.lif1(self.conv1(x))) + self.shortcut(x))


class ResNet11(nn.Module):
    """conv - LIF - pool - IF, four residual stages (w -> 2w, 2w -> 4w /2, 4w -> 8w, 8w -> 8w /2), two linear layers."""

    def __init__(self, width: int = 64, image_size: int = 32, classes: int = 10, hidden: int = 1024, p_drop: float = 0.25):
        super().__init__()
        w = width
        self.stem = nn.Sequential(nn.Conv2d(3, w, 3, 1, 1, bias=False), _spiking(p_drop), nn.AvgPool2d(2), FirstLayerIF())
        self.stages = nn.Sequential(_Residual(w, 2 * w, 1, p_drop), _Residual(2 * w, 4 * w, 2, p_drop), _Residual(4 * w, 8 * w, 1, p_drop),
                                    _Residual(8 * w, 8 * w, 2, p_drop))
        side = image_size // 8
        self.fc0 = nn.Linear(8 * w * side * side, hidden, bias=False)
        self.lif_fc = _spiking(p_drop)
        self.fc1 = nn.Linear(hidden, classes, bias=False)
        self.readout = AccumulatingLIF(fire=False)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                m.weight.data.normal_(0, math.sqrt(1.0 / (m.kernel_size[0] * m.kernel_size[1] * m.in_channels)))
            elif isinstance(m, nn.Linear):
                m.weight.data.normal_(0, math.sqrt(1.0 / m.in_features))

    def forward(self, x):
        x = self.stages(self.stem(x))
        return self.readout(self.fc1(self.lif_fc(self.fc0(x.flatten(1)))))

    def firing_neurons(self) -> List[AccumulatingLIF]:
        return [m for m in self.modules() if isinstance(m, AccumulatingLIF) and m.fire]


def poisson_signed(img: torch.Tensor) -> torch.Tensor:
    """Signed Poisson spikes: probability ``|pixel|`` (pixels normalised to about [-1, 1]), sign of the pixel."""
    return (img.abs() > torch.rand_like(img)).to(img.dtype) * img.sign()


def train_step(net: ResNet11, img: torch.Tensor, label: torch.Tensor, optimizer, T: int) -> float:
    """One batch: ``T`` Poisson steps, accumulated derivatives, MSE on the read-out potential / T, one optimiser step."""
    net.train()
    optimizer.zero_grad(set_to_none=True)
    for _ in range(T):
        out = net(poisson_signed(img))
    for m in net.firing_neurons():
        m.finish_sequence()
    loss = F.mse_loss(out / T, F.one_hot(label, out.shape[1]).to(out.dtype))
    loss.backward()
    optimizer.step()
    functional.reset_net(net)
    return float(loss.detach())


@torch.no_grad()
def evaluate(net: ResNet11, loader, T: int, device) -> float:
    net.eval()
    hit = total = 0
    for img, label in loader:
        img, label = img.to(device), label.to(device)
        for _ in range(T):
            out = net(poisson_signed(img))
        hit += int((out.argmax(1) == label).sum())
        total += label.numel()
        functional.reset_net(net)
    return hit / max(total, 1)


def _synthetic(n: int, classes: int, size: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    centres = torch.rand(classes, 3, 1, 1, generator=g) * 1.6 - 0.8
    label = torch.randint(0, classes, (n,), generator=g)
    img = (centres[label] + 0.15 * torch.randn(n, 3, size, size, generator=g)).clamp(-1, 1)
    return torch.utils.data.TensorDataset(img, label)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--data-dir", default="./cifar10")
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("-T", type=int, default=100)
    ap.add_argument("-b", "--batch-size", type=int, default=32)
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--lr", type=float, default=0.01)
    ap.add_argument("--width", type=int, default=64)
    ap.add_argument("--image-size", type=int, default=32)
    ap.add_argument("--samples", type=int, default=256, help="size of the synthetic training set")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    device = torch.device(a.device)
    if a.synthetic:
        train_set, test_set = _synthetic(a.samples, 10, a.image_size, 0), _synthetic(max(a.samples // 4, 8), 10, a.image_size, 0)
    else:
        import torchvision
        import torchvision.transforms as tf
        norm = tf.Compose([tf.ToTensor(), tf.Normalize((0.5, 0.5, 0.5), (0.5, 0.5, 0.5))])
        train_set = torchvision.datasets.CIFAR10(a.data_dir, train=True, transform=tf.Compose([tf.RandomHorizontalFlip(), norm]), download=False)
        test_set = torchvision.datasets.CIFAR10(a.data_dir, train=False, transform=norm, download=False)
    train_loader = torch.utils.data.DataLoader(train_set, a.batch_size, shuffle=True, drop_last=True)
    test_loader = torch.utils.data.DataLoader(test_set, a.batch_size)
    net = ResNet11(a.width, a.image_size).to(device)
    opt = torch.optim.SGD(net.parameters(), lr=a.lr, momentum=0.9, weight_decay=5e-4)
    history = []
    for epoch in range(a.epochs):
        losses = [train_step(net, img.to(device), label.to(device), opt, a.T) for img, label in train_loader]
        acc = evaluate(net, test_loader, a.T, device)
        history.append((sum(losses) / len(losses), acc))
        print(f"epoch {epoch}: train loss {history[-1][0]:.4f}, test accuracy {acc:.3f}")
    return net, history


if __name__ == "__main__":
    main()
