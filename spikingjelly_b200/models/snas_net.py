"""SNASNet: spiking networks whose cells come out of a neural-architecture search without training
(Kim et al., "Neural Architecture Search for Spiking Neural Networks").

A cell has four nodes (input, two intermediates, output).  The connection matrix ``con_mat[row, col]`` names the
operation on the edge ``row -> col`` (upper triangle: forward edges, evaluated in the same time step; lower triangle:
backward edges, whose result is added to the source node's value at the NEXT time step):

    0  zero (multiplication by a constant 0)     3  LIF -> 3x3 convolution -> BN
    1  identity                                   4  3x3 average pooling, stride 1
    2  LIF -> 1x1 convolution -> BN

Module and parameter names equal the reference's (``spikingjelly/activation_based/model/snas_net.py:37-512``), so its
checkpoints load; the construction is table-driven instead of one copy of the operation list per cell kind.

Network: static stem (convolution + BN, evaluated once), then per time step cell1 -> BN/LIF/conv/BN -> avg-pool ->
cell2 -> BN/LIF -> avg-pool -> dropout/linear/LIF/linear, with the class scores averaged over groups of
``num_cluster`` output neurons ("population boosting") and over time.
"""
from __future__ import annotations

import argparse
from types import SimpleNamespace
from typing import Sequence, Union

import torch
import torch.nn as nn

from ..activation_based import layer, neuron, surrogate

__all__ = ["ScaleLayer", "Neuronal_Cell", "Neuronal_Cell_backward", "SNASNet", "snasnet_args"]


class ScaleLayer(nn.Module):
    """The "zero" edge: multiplies by a constant (0), so the edge passes neither signal nor gradient but keeps shapes."""

    def __init__(self):
        super().__init__()
        self.scale = torch.tensor(0.0)

    def forward(self, input):
        return input * self.scale


def _lif(args) -> neuron.LIFNode:
    return neuron.LIFNode(v_threshold=args.threshold, v_reset=0.0, tau=args.tau, surrogate_function=surrogate.ATan(),
                          detach_reset=True)


def _edge(op: int, args, in_channel: int, out_channel: int) -> nn.Module:
    op = int(op)
    if op == 0:
        return ScaleLayer()
    if op == 1:
        return nn.Identity()
    if op in (2, 3):
        k, p = (1, 0) if op == 2 else (3, 1)
        return nn.Sequential(_lif(args),
                             nn.Conv2d(in_channel, out_channel, kernel_size=(k, k), stride=(1, 1), padding=(p, p), bias=False),
                             nn.BatchNorm2d(out_channel, eps=1e-05, momentum=0.1, affine=True, track_running_stats=True))
    if op == 4:
        return nn.AvgPool2d(kernel_size=3, stride=1, padding=1)
    raise ValueError(f"unknown cell operation {op}")


class Neuronal_Cell(nn.Module):
    """Feed-forward cell.  Edge order in ``cell_architecture``: (0->1), (0->2), (1->2), (0->3), (1->3), (2->3)."""

    def __init__(self, args, in_channel, out_channel, con_mat):
        super().__init__()
        self.con_mat = con_mat
        self.cell_architecture = nn.ModuleList(
            _edge(con_mat[row, col], args, in_channel, out_channel) for col in range(1, 4) for row in range(col))

    def forward(self, x_in):
        e = self.cell_architecture
        x_1 = e[0](x_in)
        x_2 = e[1](x_in) + e[2](x_1)
        return e[3](x_in) + e[4](x_1) + e[5](x_2)


class Neuronal_Cell_backward(nn.Module):
    """Cell with backward (recurrent) edges.  ``cell_architecture_back`` order: (1->0), (2->0), (3->0), (2->1), (3->1),
    (3->2); their outputs are kept in ``last_xin / last_x1 / last_x2`` and added to the node values at the next step."""

    def __init__(self, args, in_channel, out_channel, con_mat):
        super().__init__()
        self.con_mat = con_mat
        self.cell_architecture = nn.ModuleList(
            _edge(con_mat[row, col], args, in_channel, out_channel) for col in range(1, 4) for row in range(col))
        self.cell_architecture_back = nn.ModuleList(
            _edge(con_mat[row, col], args, in_channel, out_channel) for col in range(3) for row in range(col + 1, 4))
        self.last_xin = 0.0
        self.last_x1 = 0.0
        self.last_x2 = 0.0

    def forward(self, x_in):
        f, b = self.cell_architecture, self.cell_architecture_back
        n0 = x_in + self.last_xin
        x_1 = f[0](n0)
        n1 = x_1 + self.last_x1
        x_2 = f[1](n0) + f[2](n1)
        n2 = x_2 + self.last_x2
        x_3 = f[3](n0) + f[4](n1) + f[5](n2)
        self.last_xin = b[0](n1) + b[1](n2) + b[2](x_3)
        self.last_x1 = b[3](n2) + b[4](x_3)
        self.last_x2 = b[5](x_3)
        return x_3


_DATASETS = {
    #               classes, final neurons, cluster, image, channel ratio, spatial decay factor, classifier width, stem stride
    "cifar10":      (10, 100, 10, 32, 2, 2, 1024, 1),
    "cifar100":     (100, 500, 5, 32, 1, 2, 1024, 1),
    "tinyimagenet": (200, 1000, 5, 64, 1, 4, 4096, 2),
}


def snasnet_args(dataset: str = "cifar100", timestep: int = 5, tau: float = 4 / 3, threshold: float = 1.0,
                 celltype: str = "backward", second_avgpooling: int = 2) -> SimpleNamespace:
    """The argument bundle :class:`SNASNet` reads (the reference passes an ``argparse`` namespace with these fields)."""
    return SimpleNamespace(dataset=dataset, timestep=timestep, tau=tau, threshold=threshold, celltype=celltype,
                           second_avgpooling=second_avgpooling)


class SNASNet(nn.Module):
    def __init__(self, args, con_mat: Union[torch.Tensor, Sequence[Sequence[int]]]):
        super().__init__()
        if not torch.is_tensor(con_mat):
            con_mat = torch.tensor(con_mat)
        if args.dataset not in _DATASETS:
            raise ValueError(f"Unsupported dataset: {args.dataset!r}")
        if args.celltype not in ("forward", "backward"):
            raise ValueError(f"Unsupported celltype: {args.celltype!r}")
        self.con_mat = con_mat
        self.total_timestep = args.timestep
        self.second_avgpooling = args.second_avgpooling
        (self.num_class, self.num_final_neuron, self.num_cluster, self.img_size, self.channel_ratio, decay,
         self.classifier_inter_ch, self.stem_stride) = _DATASETS[args.dataset]
        self.in_channel = 3
        self.first_out_channel = 128
        self.spatial_decay = decay * self.second_avgpooling
        c1, c2 = self.first_out_channel * self.channel_ratio, 256 * self.channel_ratio
        cell = Neuronal_Cell if args.celltype == "forward" else Neuronal_Cell_backward

        self.stem = nn.Sequential(nn.Conv2d(self.in_channel, c1, kernel_size=3, stride=self.stem_stride, padding=1, bias=False),
                                  nn.BatchNorm2d(c1, affine=True))
        self.cell1 = cell(args, c1, c1, con_mat)
        self.downconv1 = nn.Sequential(
            nn.BatchNorm2d(c1, eps=1e-05, momentum=0.1, affine=True, track_running_stats=True), _lif(args),
            nn.Conv2d(c1, c2, kernel_size=(3, 3), stride=(1, 1), padding=(1, 1), bias=False),
            nn.BatchNorm2d(c2, eps=1e-05, momentum=0.1, affine=True, track_running_stats=True))
        self.resdownsample1 = nn.AvgPool2d(2, 2)
        self.cell2 = cell(args, c2, c2, con_mat)
        self.last_act = nn.Sequential(nn.BatchNorm2d(c2, eps=1e-05, momentum=0.1, affine=True, track_running_stats=True), _lif(args))
        self.resdownsample2 = nn.AvgPool2d(self.second_avgpooling, self.second_avgpooling)
        side = self.img_size // self.spatial_decay
        self.classifier = nn.Sequential(layer.Dropout(0.5), nn.Linear(c2 * side * side, self.classifier_inter_ch, bias=False),
                                        _lif(args), nn.Linear(self.classifier_inter_ch, self.num_final_neuron, bias=True))
        self.boost = nn.AvgPool1d(self.num_cluster, self.num_cluster)

        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_uniform_(m.weight, a=2)
            elif isinstance(m, nn.BatchNorm2d):
                nn.init.constant_(m.weight, 1)
                nn.init.constant_(m.bias, 0)
            elif isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, 0, 0.01)
                if m.bias is not None:
                    nn.init.constant_(m.bias, 0)

    def neuron_init(self):
        """Forget the values carried over the backward edges (the LIF states are reset by ``functional.reset_net``)."""
        for cell in (self.cell1, self.cell2):
            cell.last_xin = cell.last_x1 = cell.last_x2 = 0.0

    def forward(self, input):
        self.neuron_init()
        static_x = self.stem(input)
        acc = 0
        for _ in range(self.total_timestep):
            x = self.resdownsample1(self.downconv1(self.cell1(static_x)))
            x = self.resdownsample2(self.last_act(self.cell2(x)))
            x = self.classifier(x.flatten(1))
            acc = acc + self.boost(x.unsqueeze(1)).squeeze(1)
        return acc / self.total_timestep


if __name__ == "__main__":
    parser = argparse.ArgumentParser("SNASNet")
    parser.add_argument("--dataset", type=str, default="cifar100", help="[cifar10, cifar100, tinyimagenet]")
    parser.add_argument("--timestep", type=int, default=5)
    parser.add_argument("--tau", type=float, default=4 / 3)
    parser.add_argument("--threshold", type=float, default=1.0)
    parser.add_argument("--celltype", type=str, default="backward", help="[forward, backward]")
    parser.add_argument("--second_avgpooling", type=int, default=2)
    net = SNASNet(parser.parse_args(), [[0, 0, 0, 2], [0, 0, 0, 0], [0, 0, 0, 0], [0, 0, 0, 0]])
    print(net)
