"""Small stateful and stateless helpers: a synaptic low-pass filter, a delay line, population voting, and the pair of layers
that turn integer spike counts into binary sub-steps and back (``spikingjelly/activation_based/layer/misc.py:22-629``)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ...logger import logger
from .. import base, functional

__all__ = ["SynapseFilter", "PrintShapeModule", "VotingLayer", "Delay", "SpikeCountToBinary", "TemporalBinSum"]


def _state_like(state, frame: Tensor) -> Tensor:
    """A state tensor shaped like one input frame: a scalar reset value is broadcast, a tensor of another shape starts
    over from zero, a tensor elsewhere (dtype / device) is moved."""
    if not isinstance(state, Tensor):
        return torch.full_like(frame, float(state))
    if state.shape != frame.shape:
        return torch.zeros_like(frame)
    return state.to(dtype=frame.dtype, device=frame.device)


class SynapseFilter(base.MemoryModule):
    """First-order synapse: the current decays with time constant ``tau`` between spikes and is topped up by each spike,
    ``i <- i - (1 - s) * i / tau + s``.  ``learnable=True`` trains the time constant through ``1 / tau = sigmoid(w)``."""

    def __init__(self, tau=100.0, learnable=False, step_mode="s"):
        super().__init__()
        assert tau > 1, "tau must exceed 1 (sigmoid parametrisation)"
        self.step_mode, self.learnable = step_mode, learnable
        if learnable:
            self.w = nn.Parameter(torch.tensor(-math.log(tau - 1.0)))
        else:
            self.tau = tau
        self.register_memory("out_i", 0.0)

    def _decay(self):
        return torch.sigmoid(self.w) if self.learnable else 1.0 / self.tau

    def extra_repr(self):
        shown = self.tau if not self.learnable else 1.0 / float(torch.sigmoid(self.w.detach()))
        return f"tau={shown}, learnable={self.learnable}, step_mode={self.step_mode}"

    def materialize_states(self, inputs, states, step_mode):
        frame = inputs[0]
        if step_mode == "m" and frame.dim() > 0 and len(frame) > 0:
            frame = frame[0]
        return (_state_like(states[0], frame),)

    def single_step_functional_forward(self, inputs, states, **kwargs):
        current = functional.synapse_filter_step(inputs[0], states[0], self._decay())
        return (current,), (current,)


class PrintShapeModule(nn.Module):
    """Passes its input on unchanged and writes its shape to the package logger (level DEBUG)."""

    def __init__(self, ext_str="PrintShapeModule"):
        super().__init__()
        self.ext_str = ext_str

    def forward(self, x: Tensor):
        logger.debug("%s: tensor of shape %s", self.ext_str, tuple(x.shape))
        return x


class VotingLayer(nn.Module, base.StepModule):
    """Population decoding: every run of ``voting_size`` output neurons votes for one class (their mean is the score)."""

    def __init__(self, voting_size: int = 10, step_mode="s"):
        super().__init__()
        self.voting_size, self.step_mode = voting_size, step_mode

    def extra_repr(self):
        return f"voting_size={self.voting_size}, step_mode={self.step_mode}"

    def single_step_forward(self, x: torch.Tensor):
        pooled = F.avg_pool1d(x[:, None, :], kernel_size=self.voting_size, stride=self.voting_size)
        return pooled[:, 0, :]

    def forward(self, x: torch.Tensor):
        if self.step_mode == "m":
            return functional.seq_to_ann_forward(x, self.single_step_forward)
        return self.single_step_forward(x)


class Delay(base.MemoryModule):
    """Delay line: what goes in comes out ``delay_steps`` steps later (zeros before that).  Memory ``queue`` holds the frames
    in flight."""

    def __init__(self, delay_steps: int, step_mode="s"):
        super().__init__()
        assert isinstance(delay_steps, int) and delay_steps >= 0, "delay_steps is a non-negative int"
        self._delay_steps, self.step_mode = delay_steps, step_mode
        self.register_memory("queue", [])

    @property
    def delay_steps(self):
        return self._delay_steps

    def single_step_functional_forward(self, inputs, states, **kwargs):
        out, in_flight = functional.delay_step(inputs[0], tuple(states[0]), self._delay_steps)
        return (out,), (list(in_flight),)

    def multi_step_functional_forward(self, inputs, states, **kwargs):
        in_flight = tuple(states[0])
        outs = []
        for frame in inputs[0]:
            out, in_flight = functional.delay_step(frame, in_flight, self._delay_steps)
            outs.append(out)
        return (torch.stack(outs),), (list(in_flight),)

    def single_step_forward(self, x: Tensor) -> Tensor:
        (out,), (in_flight,) = self.single_step_functional_forward((x,), (self.queue,))
        self.queue[:] = in_flight              # in place: references to the memory stay valid
        return out


class _SlotLayer(nn.Module, base.MultiStepModule):
    """Common part of the count <-> binary layers: ``num_slots`` sub-steps per step; identity while training unless
    ``always_convert``."""

    def __init__(self, num_slots: int, always_convert: bool = False) -> None:
        super().__init__()
        if num_slots < 1:
            raise ValueError(f"num_slots: at least one sub-step per step is needed, got {num_slots}")
        self.num_slots, self.always_convert = num_slots, always_convert
        self._step_mode = "m"

    def _active(self, x_seq: Tensor) -> bool:
        if self.training and not self.always_convert:
            return False
        if x_seq.ndim < 2 or x_seq.shape[0] == 0:
            raise ValueError(f"x_seq: expected [T, N, *] with T > 0, got shape {tuple(x_seq.shape)}")
        return True


class SpikeCountToBinary(_SlotLayer):
    """``[T, N, *]`` integer spike counts -> ``[T * num_slots, N, *]`` binary spikes: a count ``c`` becomes ``c`` ones
    followed by ``num_slots - c`` zeros.  The backward pass treats every sub-step as ``count / num_slots``."""

    def forward(self, x_seq: torch.Tensor) -> torch.Tensor:
        if not self._active(x_seq):
            return x_seq
        counts = x_seq[:, None]                                               # [T, 1, N, *]
        slot = torch.arange(self.num_slots, device=x_seq.device).reshape(1, self.num_slots, *([1] * (x_seq.ndim - 1)))
        binary = (counts > slot).to(x_seq.dtype)
        smooth = counts / self.num_slots
        return (binary + smooth - smooth.detach()).flatten(0, 1)


class TemporalBinSum(_SlotLayer):
    """``[T * num_slots, N, *]`` -> ``[T, N, *]``: adds up each run of ``num_slots`` steps (a ragged tail is zero padded)."""

    def forward(self, x_seq: torch.Tensor) -> torch.Tensor:
        if not self._active(x_seq):
            return x_seq
        missing = -x_seq.shape[0] % self.num_slots
        if missing:
            x_seq = torch.cat([x_seq, x_seq.new_zeros(missing, *x_seq.shape[1:])])
        return x_seq.unflatten(0, (-1, self.num_slots)).sum(1)
