"""Layers for online training through time (OTTT), where activations travel as a ``[spike, trace]`` pair: the forward
value of a weighted layer comes from the spike, its weight gradient from the presynaptic trace
(``spikingjelly/activation_based/layer/online_learning.py:14-254``).
"""
import torch
import torch.nn as nn

__all__ = ["ReplaceforGrad", "GradwithTrace", "SpikeTraceOp", "OTTTSequential"]


class ReplaceforGrad(torch.autograd.Function):
    """``y = x_r`` in the forward pass; in the backward pass the incoming gradient goes to ``x`` AND ``x_r``.  Lets one
    tensor carry the value while another one carries the graph."""

    @staticmethod
    def forward(ctx, x, x_r):
        return x_r

    @staticmethod
    def backward(ctx, grad):
        return grad, grad


def _weighted(layer: nn.Module, spike: torch.Tensor, trace: torch.Tensor) -> torch.Tensor:
    """``layer(spike)`` as the value, differentiated as if the input had been ``trace``."""
    graph_side = layer(ReplaceforGrad.apply(spike, trace))      # value of layer(trace), gradient also reaches spike
    with torch.no_grad():
        value_side = layer(spike)
    return ReplaceforGrad.apply(graph_side, value_side)


def _unweighted(layer: nn.Module, spike: torch.Tensor, trace: torch.Tensor) -> list:
    """Pooling, flatten and the like act on both members; only the spike keeps a graph."""
    with torch.no_grad():
        moved_trace = layer(trace)
    return [layer(spike), moved_trace]


class GradwithTrace(nn.Module):
    """Around a layer with weights: ``[spike, trace]`` in, one tensor out."""

    def __init__(self, module):
        super().__init__()
        self.module = module

    def forward(self, x):
        return _weighted(self.module, *x)


class SpikeTraceOp(nn.Module):
    """Around a layer without weights: ``[spike, trace]`` in, ``[spike', trace']`` out."""

    def __init__(self, module):
        super().__init__()
        self.module = module

    def forward(self, x):
        return _unweighted(self.module, *x)


class OTTTSequential(nn.Sequential):
    """``nn.Sequential`` for OTTT networks.  While the running value is a ``[spike, trace]`` list, a child that owns
    parameters consumes the pair (:func:`_weighted`) and a parameter-free child maps both members; plain tensors go
    through the children as usual."""

    def forward(self, input):
        for child in self:
            if not isinstance(input, list):
                input = child(input)
                continue
            owns_weights = any(True for _ in child.parameters())
            input = _weighted(child, *input) if owns_weights else _unweighted(child, *input)
        return input
