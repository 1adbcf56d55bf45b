"""Building blocks of online training through time (OTTT): layers that forward a
``[spike, trace]`` pair and route gradients through the presynaptic trace.

Parity: ``spikingjelly/activation_based/layer/online_learning.py:14-254``.
"""
import torch
import torch.nn as nn

__all__ = ["ReplaceforGrad", "GradwithTrace", "SpikeTraceOp", "OTTTSequential"]


class ReplaceforGrad(torch.autograd.Function):
    """Forward returns the second argument; backward sends the gradient to both."""

    @staticmethod
    def forward(ctx, x, x_r):
        return x_r

    @staticmethod
    def backward(ctx, grad):
        return grad, grad


def _with_trace_grad(module: nn.Module, pair):
    """Output value computed from the spike, weight gradient computed from the trace."""
    spike, trace = pair
    with torch.no_grad():
        value = module(spike)
    carrier = module(ReplaceforGrad.apply(spike, trace))
    return ReplaceforGrad.apply(carrier, value)


def _on_both(module: nn.Module, pair):
    spike, trace = pair
    spike = module(spike)
    with torch.no_grad():
        trace = module(trace)
    return [spike, trace]


class GradwithTrace(nn.Module):
    """Wrap a weighted layer: input ``[spike, trace]`` -> tensor."""

    def __init__(self, module):
        super().__init__()
        self.module = module

    def forward(self, x):
        return _with_trace_grad(self.module, x)


class SpikeTraceOp(nn.Module):
    """Wrap a parameter-free layer (pooling, flatten): applied to spike and trace alike."""

    def __init__(self, module):
        super().__init__()
        self.module = module

    def forward(self, x):
        return _on_both(self.module, x)


class OTTTSequential(nn.Sequential):
    """Sequential that understands ``[spike, trace]`` lists: parameter-free children act on
    both entries, weighted children consume the pair."""

    def forward(self, input):
        for module in self:
            if isinstance(input, list):
                has_params = next(module.parameters(), None) is not None
                input = _with_trace_grad(module, input) if has_params else _on_both(module, input)
            else:
                input = module(input)
        return input
