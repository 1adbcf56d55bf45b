"""SpikeDHS: spiking network found by differentiable hierarchical search, with the differentiable surrogate-gradient
search (DGS) of the ``dSpike`` temperature (Che et al., "Differentiable hierarchical and surrogate gradient search for
spiking neural networks").

Names of modules, parameters and public classes equal the reference's
(``spikingjelly/activation_based/model/spike_dhs.py:30-947``) so that its checkpoints load.  Differences in how it is
written: the three-candidate ("small / middle / big" temperature) machinery that the reference repeats for the stem and
for the cell node lives once in :class:`_DGSBranches`; ``dgs_alpha`` is created on the module's device instead of
being forced onto ``cuda``; the nearest-neighbour resize is a function instead of a module built on every call.

Every tensor is a sequence ``[T, N, C, H, W]`` (multi-step mode).
"""
from __future__ import annotations

import argparse
from collections import namedtuple
from math import tanh
from types import SimpleNamespace
from typing import List, Sequence

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from ..activation_based import functional, layer
from ..activation_based.neuron import LIFNode
from ..activation_based.surrogate import SurrogateFunctionBase, heaviside

__all__ = ["DSpike", "save_v_LIFNode", "SpikingConv2d", "SpikingLinear", "SpikingAvgPool2d", "SpikingAdaptiveAvgPool2d",
           "SearchSpikingConv2d_stem", "SearchSpikingConv2d_cell", "Cell", "newFeature", "AuxiliaryHeadCIFAR", "SpikeDHS",
           "network_layer_to_space", "spikedhs_args", "Genotype", "PRIMITIVES"]

Genotype = namedtuple("Genotype_2D", "cell cell_concat")
PRIMITIVES = ["skip_connect", "snn_b3", "snn_b5"]


def network_layer_to_space(net_arch: Sequence[int]) -> np.ndarray:
    """Path through the 4-level resolution trellis -> one-hot ``[layers, 4, 3]``: entry ``[i, level, move]`` with move
    0 = came from the level above (down-sampled), 1 = same level, 2 = came from the level below (up-sampled)."""
    space = np.zeros((len(net_arch), 4, 3))
    prev = None
    for i, level in enumerate(net_arch):
        if prev is None:
            move = 0
        elif level == prev + 1:
            move = 0
        elif level == prev:
            move = 1
        elif level == prev - 1:
            move = 2
        else:
            raise ValueError("consecutive layers may differ by at most one level")
        space[i][level][move] = 1
        prev = level
    return space


# ------------------------------------------------------------------------------------------------ surrogate + neuron
class _DSpikeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, alpha):
        if x.requires_grad:
            ctx.save_for_backward(x)
            ctx.alpha = alpha
        return heaviside(x)

    @staticmethod
    def backward(ctx, grad_output):
        (x,) = ctx.saved_tensors
        alpha = ctx.alpha
        const = alpha / (2.0 * tanh(alpha / 2.0))
        g = grad_output * const / torch.cosh(alpha * x).square()
        return g.masked_fill(x.abs() > 0.5, 0), None


def dSpike_backward(grad_output: torch.Tensor, x: torch.Tensor, alpha: float):
    """``(grad_x, None)``: the gradient :class:`DSpike` applies, as a function of the saved input."""
    const = alpha / (2.0 * tanh(alpha / 2.0))
    return (grad_output * const / torch.cosh(alpha * x).square()).masked_fill(x.abs() > 0.5, 0), None


dSpike = _DSpikeFn          # the autograd function under the reference's name: ``dSpike.apply(x, alpha)``


class Nearest(nn.Module):
    """Nearest-neighbour resize to a fixed spatial ``shape``."""

    def __init__(self, shape) -> None:
        super().__init__()
        self._shape = shape

    def forward(self, x):
        return F.interpolate(x, self._shape, mode="nearest")


class DSpike(SurrogateFunctionBase):
    """Heaviside forward; backward ``alpha / (2 tanh(alpha / 2)) / cosh^2(alpha x)`` inside ``|x| <= 1/2`` and zero
    outside: the derivative of a tanh ramp whose temperature ``alpha`` moves it between a box and a delta."""

    def __init__(self, alpha: float = 3, spiking=True):
        assert alpha > 0, "alpha must be lager than 0."
        super().__init__(spiking, alpha=alpha)

    @staticmethod
    def spiking_function(x, alpha):
        return _DSpikeFn.apply(x, alpha)

    @staticmethod
    def primitive_function(x, alpha):
        return (torch.tanh(alpha * x.clamp(-0.5, 0.5)) / (2.0 * tanh(alpha / 2.0)) + 0.5)


class save_v_LIFNode(LIFNode):
    """LIF that also records ``mean(h - v_threshold)`` of the last step in ``v_before_spike`` (the search reads it)."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.v_before_spike = None

    def _step_with_observation(self, x, v):
        charged = functional.lif_charge(x, v, self.tau, self.decay_input, self.v_reset)
        observed = (charged - self.v_threshold).mean()
        spike = self.surrogate_function(charged - self.v_threshold)
        v = functional.voltage_reset(charged, spike, self.v_threshold, self.v_reset, self.detach_reset)
        return spike, v, observed

    def single_step_functional_forward(self, inputs, states, **kwargs):
        spike, v, _ = self._step_with_observation(inputs[0], states[0])
        return (spike,), (v, *states[1:])

    def single_step_forward(self, x):
        states = self.materialize_states((x,), tuple(self._memories.values()), "s")
        spike, v, self.v_before_spike = self._step_with_observation(x, states[0])
        self.v = v
        return spike

    def multi_step_forward(self, x_seq):
        v = self.materialize_states((x_seq,), tuple(self._memories.values()), "m")[0]
        spikes, seen = [], []
        for x in x_seq:
            spike, v, obs = self._step_with_observation(x, v)
            spikes.append(spike)
            seen.append(obs)
        self.v = v
        self.v_before_spike = seen[-1]
        if self.store_v_seq:
            self.v_seq = torch.stack(seen)
        return torch.stack(spikes)


def _node(cls=LIFNode, v_threshold: float = 0.5):
    return cls(tau=1.25, decay_input=False, v_threshold=v_threshold, detach_reset=True, surrogate_function=DSpike(),
               step_mode="m")


def getSpikingNode(v_threshold=0.5):
    return _node(LIFNode, v_threshold)


def get_save_v_SpikingNode(v_threshold=0.5):
    return _node(save_v_LIFNode, v_threshold)


# --------------------------------------------------------------------------------------------------------- components
class SpikingConv2d(nn.Module):
    def __init__(self, input_c, output_c, kernel_size=3, stride=1, padding=1, b=3, spiking=True, v_threshold=0.5):
        super().__init__()
        self.conv = layer.Conv2d(input_c, output_c, kernel_size=kernel_size, stride=stride, padding=padding, step_mode="m")
        self.bn = layer.BatchNorm2d(output_c, step_mode="m")
        self.spiking = spiking
        if spiking:
            self.spike = getSpikingNode(v_threshold=v_threshold)

    def forward(self, x):
        x = self.bn(self.conv(x))
        return self.spike(x) if self.spiking else x


OPS = {
    "skip_connect": lambda Cin, Cout, stride, signal: (SpikingConv2d(Cin, Cout, stride=stride, padding=1, spiking=False)
                                                       if signal == 1 else nn.Identity()),
    "snn_b3": lambda Cin, Cout, stride, signal: SpikingConv2d(Cin, Cout, kernel_size=3, stride=stride, padding=1, spiking=False),
    "snn_b5": lambda Cin, Cout, stride, signal: SpikingConv2d(Cin, Cout, kernel_size=3, stride=stride, padding=1, spiking=False),
}


class _DGSBranches(nn.Module):
    """Surrogate-gradient search over one spiking node.  Outside a search stage only the "middle" branch (suffix
    ``_m``) runs.  During a stage (``dgs_init_stage``) two copies of its weights run beside it with the ``dSpike``
    temperature moved by ``-dgs_step`` (``_s``) and ``+dgs_step`` (``_b``), mixed by ``softmax(dgs_alpha)``; the stage
    ends by moving the middle temperature in the winning direction (``dgs_finish_stage``), floored at 0.2.

    Subclasses list in ``_paths`` the (conv, bn) attribute prefixes whose ``_m/_b/_s`` variants they created."""

    _paths: tuple = ()
    dgs_step = 0.2

    def _make_search_state(self):
        self.spike_m, self.spike_b, self.spike_s = (get_save_v_SpikingNode() for _ in range(3))
        self.is_DGS = False
        self.dgs_alpha = nn.Parameter(1e-3 * torch.ones(3), requires_grad=True)
        self.dgs_step = 0.2

    def dgs_init_stage(self):
        self.is_DGS = True
        for conv, bn in self._paths:
            for tag in ("_s", "_b"):
                getattr(self, conv + tag).load_state_dict(getattr(self, conv + "_m").state_dict())
                getattr(self, bn + tag).load_state_dict(getattr(self, bn + "_m").state_dict())
        mid = self.spike_m.surrogate_function.alpha
        self.spike_s.surrogate_function.alpha = mid - self.dgs_step
        self.spike_b.surrogate_function.alpha = mid + self.dgs_step
        self.dgs_alpha = nn.Parameter(1e-3 * torch.ones(3, device=self.dgs_alpha.device), requires_grad=True)
        for p in self.parameters():
            p.requires_grad_(True)

    def dgs_finish_stage(self, dgs_direction):
        self.is_DGS = False
        sg = self.spike_m.surrogate_function
        sg.alpha = max(sg.alpha + (-self.dgs_step, 0, self.dgs_step)[dgs_direction], 0.2)

    def _current(self, tag: str, xs):
        total = None
        for (conv, bn), x in zip(self._paths, xs):
            y = getattr(self, bn + tag)(getattr(self, conv + tag)(x))
            total = y if total is None else total + y
        return getattr(self, "spike" + tag)(total)

    def _run(self, *xs):
        if not self.is_DGS:
            return self._current("_m", xs)
        w = F.softmax(self.dgs_alpha, dim=0)
        return w[0] * self._current("_s", xs) + w[1] * self._current("_m", xs) + w[2] * self._current("_b", xs)


class SearchSpikingConv2d_stem(_DGSBranches):
    _paths = (("conv", "bn"),)

    def __init__(self, input_c, output_c, kernel_size=3, stride=1, padding=1, b=3, spiking=True, v_threshold=0.5):
        super().__init__()
        for tag in ("_m", "_b", "_s"):
            setattr(self, "conv" + tag, layer.Conv2d(input_c, output_c, kernel_size=kernel_size, stride=stride, padding=padding, step_mode="m"))
        for tag in ("_m", "_b", "_s"):
            setattr(self, "bn" + tag, layer.BatchNorm2d(output_c, step_mode="m"))
        self._make_search_state()

    def forward(self, x):
        return self._run(x)


class SearchSpikingConv2d_cell(_DGSBranches):
    """One cell node: two incoming edges, each convolution + BN, summed in front of ONE spiking neuron."""
    _paths = (("conv1", "bn1"), ("conv2", "bn2"))

    def __init__(self, io_c, kernel_size=3, stride=1, padding=1, b=3, spiking=True, v_threshold=0.5):
        super().__init__()
        for k, (cin, cout, _primitive) in enumerate(io_c, start=1):
            for tag in ("_m", "_b", "_s"):
                setattr(self, f"conv{k}{tag}", layer.Conv2d(cin, cout, kernel_size=kernel_size, stride=stride, padding=padding, step_mode="m"))
            for tag in ("_m", "_b", "_s"):
                setattr(self, f"bn{k}{tag}", layer.BatchNorm2d(cout, step_mode="m"))
        self._make_search_state()

    def forward(self, x1, x2):
        return self._run(x1, x2)


class SpikingLinear(nn.Module):
    def __init__(self, input_c, output_c, spiking=True):
        super().__init__()
        self.linear = layer.Linear(input_c, output_c, step_mode="m")
        self.bn = layer.SeqToANNContainer(nn.BatchNorm1d(output_c))
        self.spiking = spiking
        if spiking:
            self.spike = getSpikingNode()

    def forward(self, x):
        x = self.bn(self.linear(x))
        return self.spike(x) if self.spiking else x


class SpikingAvgPool2d(nn.Module):
    def __init__(self, kernel_size=5, stride=3, padding=0, b=3, spiking=True):
        super().__init__()
        self.pooling = layer.SeqToANNContainer(nn.AvgPool2d(kernel_size=kernel_size, stride=stride, padding=padding, count_include_pad=False))
        self.spike = getSpikingNode()

    def forward(self, x):
        return self.spike(self.pooling(x))


class SpikingAdaptiveAvgPool2d(nn.Module):
    def __init__(self, dimension, b=3, spiking=True):
        super().__init__()
        self.pooling = layer.SeqToANNContainer(nn.AdaptiveAvgPool2d(dimension))
        self.spike = getSpikingNode()

    def forward(self, x):
        return self.spike(self.pooling(x))


def _resize_nearest(x_seq: torch.Tensor, size) -> torch.Tensor:
    t, n = x_seq.shape[:2]
    return F.interpolate(x_seq.flatten(0, 1), list(size), mode="nearest").unflatten(0, (t, n))


# -------------------------------------------------------------------------------------------------------------- model
class Cell(nn.Module):
    """Three nodes; node ``j`` reads two of the earlier states (the two cell inputs and the nodes before it).
    ``cell_arch`` rows are ``[edge id, primitive]``; edge ids 0, 2, 5 start at the input before last, 1, 3, 6 at the
    last input, the others at a node of this cell.  The output concatenates the last ``block_multiplier`` states."""

    def __init__(self, steps, block_multiplier, prev_prev_fmultiplier, prev_filter_multiplier, cell_arch, network_arch,
                 filter_multiplier, downup_sample, args=None):
        super().__init__()
        self.C_in = block_multiplier * filter_multiplier
        self.C_out = filter_multiplier
        self.C_prev = int(block_multiplier * prev_filter_multiplier)
        self.C_prev_prev = int(block_multiplier * prev_prev_fmultiplier)
        self.downup_sample = int(downup_sample)
        self._steps = steps
        self.block_multiplier = block_multiplier
        if self.downup_sample == -1:
            self.scale = 0.5
        elif self.downup_sample == 1:
            self.scale = 2
        self.cell_arch = torch.sort(torch.as_tensor(cell_arch), dim=0)[0].to(torch.uint8)
        self._ops = nn.ModuleList()
        pair: List[list] = []
        for edge, prim in self.cell_arch.tolist():
            c_in = self.C_prev_prev if edge in (0, 2, 5) else self.C_prev if edge in (1, 3, 6) else self.C_out
            pair.append([c_in, self.C_out, PRIMITIVES[prim]])
            if len(pair) == 2:
                self._ops.append(SearchSpikingConv2d_cell(io_c=pair))
                pair = []
        self.spikes = nn.ModuleList([getSpikingNode() for _ in range(self._steps)])

    @staticmethod
    def scale_dimension(dim, scale):
        return int((float(dim) - 1.0) * scale + 1.0) if dim % 2 == 1 else int(float(dim) * scale)

    def forward(self, prev_prev_input, prev_input):
        s0, s1 = prev_prev_input, prev_input
        if self.downup_sample != 0:
            s1 = _resize_nearest(s1, (self.scale_dimension(s1.shape[3], self.scale), self.scale_dimension(s1.shape[4], self.scale)))
        if s0.shape[3:] != s1.shape[3:]:
            s0 = _resize_nearest(s0, s1.shape[3:])
        states = [s0, s1]
        states.append(self._ops[0](states[0], states[1]))
        states.append(self._ops[1](states[0], states[1]))
        states.append(self._ops[2](states[2], states[3]))
        return prev_input, torch.cat(states[-self.block_multiplier:], dim=2)


class AuxiliaryHeadCIFAR(nn.Module):
    """Auxiliary classifier on an 8 x 8 feature map."""

    def __init__(self, C, num_classes):
        super().__init__()
        self.pooling = SpikingAvgPool2d(kernel_size=5, stride=3, padding=0)
        self.conv1 = SpikingConv2d(C, 128, 1, padding=0, b=3)
        self.conv2 = SpikingConv2d(128, 768, 2, padding=0, b=3)
        self.classifier = SpikingLinear(768, num_classes, spiking=False)

    def forward(self, x):
        x = self.conv2(self.conv1(self.pooling(x)))
        return self.classifier(x.flatten(2))


class newFeature(nn.Module):
    def __init__(self, frame_rate, network_arch, cell_arch, cell=Cell, args=None):
        super().__init__()
        self.args = args
        self.network_arch = torch.from_numpy(np.asarray(network_arch))
        self.cell_arch = torch.from_numpy(np.asarray(cell_arch))
        self._step = args.fea_step
        self._num_layers = args.fea_num_layers
        self._block_multiplier = args.fea_block_multiplier
        self._filter_multiplier = args.fea_filter_multiplier
        fm, bm = int(self._filter_multiplier), self._block_multiplier
        self.stem0 = SearchSpikingConv2d_stem(frame_rate, fm * bm, kernel_size=3, stride=1, padding=1, b=3)
        self.auxiliary_head = AuxiliaryHeadCIFAR(576, 100)
        width = {0: 1, 1: 2, 2: 4, 3: 8}
        levels = [int(torch.argmax(self.network_arch[i].sum(dim=1))) for i in range(self._num_layers)]
        self.cells = nn.ModuleList()
        for i in range(self._num_layers):
            if i == 0:
                move = -levels[0]
                pp, p = fm, fm
            else:
                move = int(torch.argmax(self.network_arch[i].sum(dim=0))) - 1
                pp = fm if i == 1 else int(fm * width[levels[i - 2]])
                p = int(fm * width[levels[i - 1]])
            self.cells.append(cell(self._step, bm, pp, p, self.cell_arch, self.network_arch[i], int(fm * width[levels[i]]), move, args))

    def forward(self, x):
        stem = self.stem0(x)
        out = (stem, stem)
        logits_aux = None
        for i in range(self._num_layers):
            out = self.cells[i](out[0], out[1])
            if i == 2 * 8 // 3 and self.training:
                logits_aux = self.auxiliary_head(out[-1])
        return out[-1], (logits_aux if self.training else None)

    def get_params(self):
        return [p for _, p in self.named_parameters()], []


def spikedhs_args(fea_num_layers: int = 8, fea_filter_multiplier: int = 48, fea_block_multiplier: int = 3, fea_step: int = 3) -> SimpleNamespace:
    """The fields :class:`SpikeDHS` reads from its ``args`` (the reference passes an ``argparse`` namespace)."""
    return SimpleNamespace(fea_num_layers=fea_num_layers, fea_filter_multiplier=fea_filter_multiplier,
                           fea_block_multiplier=fea_block_multiplier, fea_step=fea_step)


class SpikeDHS(nn.Module):
    """CIFAR-100 classifier: fixed searched path ``[0, 0, 1, 1, 1, 2, 2, 2]`` through the resolution trellis and the
    searched cell; 6 time steps on a repeated image.  ``forward(image [N, C, H, W]) -> (logits, aux logits | None)``."""

    def __init__(self, init_channels=3, args=None):
        super().__init__()
        args = args if args is not None else spikedhs_args()
        net_arch = network_layer_to_space(np.array([0, 0, 1, 1, 1, 2, 2, 2][:args.fea_num_layers]))
        cell_arch = np.array([[1, 1], [0, 1], [3, 2], [2, 1], [7, 1], [8, 1]])
        self.feature = newFeature(init_channels, net_arch, cell_arch, args=args)
        self.global_pooling = SpikingAdaptiveAvgPool2d(1)
        self.classifier = SpikingLinear(576, 100, spiking=False)
        self._time_step = 6

    def weight_parameters(self):
        return list(self.parameters())

    def forward(self, input):
        x = input.unsqueeze(0).expand(self._time_step, -1, -1, -1, -1)
        feature_out, logits_aux = self.feature(x)
        pooled = self.global_pooling(feature_out)
        logits = self.classifier(pooled.flatten(2)).mean(0)
        if self.training:
            return logits, (logits_aux.mean(0) if logits_aux is not None else None)
        return logits, None

    def dgs_freeze_weights(self):
        for p in self.parameters():
            p.requires_grad_(False)

    def dgs_unfreeze_weights(self):
        for p in self.parameters():
            p.requires_grad_(True)


if __name__ == "__main__":
    parser = argparse.ArgumentParser("cifar")
    parser.add_argument("--fea_num_layers", type=int, default=8)
    parser.add_argument("--fea_filter_multiplier", type=int, default=48)
    parser.add_argument("--fea_block_multiplier", type=int, default=3)
    parser.add_argument("--fea_step", type=int, default=3)
    print(SpikeDHS(init_channels=3, args=parser.parse_args()))
