"""Spiking recurrent networks: vanilla RNN, LSTM and GRU cells whose gate non-linearities are
surrogate (Heaviside in forward) functions, and the stacked / bidirectional wrappers.

Layout and parameter names follow ``torch.nn.RNN*`` conventions per cell (``linear_ih``,
``linear_hh``); multi-layer state tensors are ``[num_layers * num_directions, B, H]`` (a tuple of two
for the LSTM).  State-dict keys: ``cells.<l>.linear_ih.weight`` ... (and ``cells_reverse.<l>...``).

The stacked wrappers hoist the input projection of a whole sequence out of the time loop — one
``[T*B, in] x [in, G*H]`` GEMM per layer and direction — so that only the ``[B, H] x [H, G*H]``
recurrent product remains sequential.

Parity: ``spikingjelly/activation_based/rnn.py:10-1630``.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import surrogate

__all__ = ["directional_rnn_cell_forward", "bidirectional_rnn_cell_forward", "SpikingRNNCellBase", "SpikingRNNBase",
           "SpikingLSTMCell", "SpikingLSTM", "SpikingVanillaRNNCell", "SpikingVanillaRNN", "SpikingGRUCell", "SpikingGRU"]


def _first(ss, single_state: bool):
    return ss if single_state else ss[0]


def directional_rnn_cell_forward(cell: nn.Module, x: torch.Tensor, states: torch.Tensor):
    """Run ``cell`` over ``x [T, B, in]`` from ``states`` (``[B, H]``, or ``[n_states, B, H]``).
    Returns ``(outputs [T, B, H], final states)``; with several states the first one is the output."""
    if states.dim() not in (2, 3):
        raise ValueError(f"states must be 2D or 3D, but got shape {states.shape}")
    single = states.dim() == 2
    ss, outputs = states, []
    for t in range(x.shape[0]):
        ss = cell(x[t], ss)
        outputs.append(_first(ss, single))
    return torch.stack(outputs), ss


def bidirectional_rnn_cell_forward(cell: nn.Module, cell_reverse: nn.Module, x: torch.Tensor, states: torch.Tensor,
                                   states_reverse: torch.Tensor):
    """Forward cell over ``x`` and ``cell_reverse`` over the reversed sequence; outputs are
    concatenated on the feature axis (``[T, B, 2H]``, the reverse half re-aligned in time)."""
    if states.dim() not in (2, 3) or states_reverse.dim() != states.dim():
        raise ValueError("states and states_reverse must have the same rank, either 2D or 3D")
    single = states.dim() == 2
    T = x.shape[0]
    ss, ss_r, out, out_r = states, states_reverse, [], []
    for t in range(T):
        ss = cell(x[t], ss)
        ss_r = cell_reverse(x[T - t - 1], ss_r)
        out.append(_first(ss, single))
        out_r.append(_first(ss_r, single))
    return torch.cat((torch.stack(out), torch.stack(out_r).flip(0)), dim=-1), ss, ss_r


class SpikingRNNCellBase(nn.Module):
    """Holds ``linear_ih`` / ``linear_hh`` (created by subclasses); parameters ~ U(-1/sqrt(H), 1/sqrt(H))."""

    def __init__(self, input_size: int, hidden_size: int, bias=True):
        super().__init__()
        self.input_size, self.hidden_size, self.bias = input_size, hidden_size, bias

    def reset_parameters(self):
        k = math.sqrt(1 / self.hidden_size)
        for p in self.parameters():
            nn.init.uniform_(p, -k, k)

    def weight_ih(self):
        return self.linear_ih.weight

    def weight_hh(self):
        return self.linear_hh.weight

    def bias_ih(self):
        return self.linear_ih.bias

    def bias_hh(self):
        return self.linear_hh.bias

    # -- split form used by the stacked wrappers: forward(x, s) == step(linear_ih(x), s)
    def step(self, ih: torch.Tensor, state):
        raise NotImplementedError

    def _zeros(self, x: torch.Tensor) -> torch.Tensor:
        return torch.zeros(x.shape[0], self.hidden_size, dtype=x.dtype, device=x.device)


class SpikingVanillaRNNCell(SpikingRNNCellBase):
    """``h' = Theta(W_ih x + b_ih + W_hh h + b_hh)``"""

    def __init__(self, input_size: int, hidden_size: int, bias=True, surrogate_function=surrogate.Erf()):
        super().__init__(input_size, hidden_size, bias)
        self.linear_ih = nn.Linear(input_size, hidden_size, bias=bias)
        self.linear_hh = nn.Linear(hidden_size, hidden_size, bias=bias)
        self.surrogate_function = surrogate_function
        self.reset_parameters()

    def step(self, ih, h):
        return self.surrogate_function(ih + self.linear_hh(h))

    def forward(self, x: torch.Tensor, h=None):
        return self.step(self.linear_ih(x), self._zeros(x) if h is None else h)


class SpikingLSTMCell(SpikingRNNCellBase):
    """Spiking LSTM (Lotfi Rezaabad & Vishwanath, 2020): all four gates are spikes,
    ``c' = min(c f + i g, 1)``, ``h' = c' o``.  ``surrogate_function2`` (optional) is used for ``g``."""

    def __init__(self, input_size: int, hidden_size: int, bias=True, surrogate_function1=surrogate.Erf(),
                 surrogate_function2=None):
        super().__init__(input_size, hidden_size, bias)
        self.linear_ih = nn.Linear(input_size, 4 * hidden_size, bias=bias)
        self.linear_hh = nn.Linear(hidden_size, 4 * hidden_size, bias=bias)
        self.surrogate_function1, self.surrogate_function2 = surrogate_function1, surrogate_function2
        if surrogate_function2 is not None:
            assert surrogate_function1.spiking == surrogate_function2.spiking
        self.reset_parameters()

    def step(self, ih, hc):
        h, c = hc[0], hc[1]
        pre = ih + self.linear_hh(h)
        if self.surrogate_function2 is None:
            i, f, g, o = torch.split(self.surrogate_function1(pre), self.hidden_size, dim=1)
        else:
            assert self.surrogate_function1.spiking == self.surrogate_function2.spiking
            i, f, g, o = torch.split(pre, self.hidden_size, dim=1)
            i, f, o = self.surrogate_function1(i), self.surrogate_function1(f), self.surrogate_function1(o)
            g = self.surrogate_function2(g)
        c = c * f + i * g
        with torch.no_grad():
            torch.clamp_max_(c, 1.0)         # the cell state stays binary
        return c * o, c

    def forward(self, x: torch.Tensor, hc=None):
        if hc is None:
            z = self._zeros(x)
            hc = (z, torch.zeros_like(z))
        return self.step(self.linear_ih(x), hc)


class SpikingGRUCell(SpikingRNNCellBase):
    """``r, z = Theta(.)``; ``n = Theta(W_in x + r (W_hn h))``; ``h' = (1 - z) n + z h``."""

    def __init__(self, input_size: int, hidden_size: int, bias=True, surrogate_function1=surrogate.Erf(),
                 surrogate_function2=None):
        super().__init__(input_size, hidden_size, bias)
        self.linear_ih = nn.Linear(input_size, 3 * hidden_size, bias=bias)
        self.linear_hh = nn.Linear(hidden_size, 3 * hidden_size, bias=bias)
        self.surrogate_function1, self.surrogate_function2 = surrogate_function1, surrogate_function2
        if surrogate_function2 is not None:
            assert surrogate_function1.spiking == surrogate_function2.spiking
        self.reset_parameters()

    def step(self, ih, h):
        y_ih = torch.split(ih, self.hidden_size, dim=1)
        y_hh = torch.split(self.linear_hh(h), self.hidden_size, dim=1)
        r = self.surrogate_function1(y_ih[0] + y_hh[0])
        z = self.surrogate_function1(y_ih[1] + y_hh[1])
        sg_n = self.surrogate_function1 if self.surrogate_function2 is None else self.surrogate_function2
        n = sg_n(y_ih[2] + r * y_hh[2])
        return (1.0 - z) * n + z * h

    def forward(self, x: torch.Tensor, h=None):
        return self.step(self.linear_ih(x), self._zeros(x) if h is None else h)


class SpikingRNNBase(nn.Module):
    """``num_layers`` stacked (optionally bidirectional) cells with inter-layer dropout.
    ``invariant_dropout_mask``: one mask per layer shared by all time-steps of a forward call.

    ``forward(x [T, B, in], states=None) -> (y [T, B, H * dirs], final states)``; ``states`` /
    final states: ``[layers * dirs, B, H]`` or a tuple of ``states_num()`` such tensors."""

    def __init__(self, input_size, hidden_size, num_layers, bias=True, dropout_p=0, invariant_dropout_mask=False,
                 bidirectional=False, *args, **kwargs):
        super().__init__()
        self.input_size, self.hidden_size, self.num_layers, self.bias = input_size, hidden_size, num_layers, bias
        self.dropout_p, self.invariant_dropout_mask, self.bidirectional = dropout_p, invariant_dropout_mask, bidirectional
        if bidirectional:
            self.cells, self.cells_reverse = self.create_cells(*args, **kwargs)
        else:
            self.cells = self.create_cells(*args, **kwargs)

    def create_cells(self, *args, **kwargs):
        cell_type = self.base_cell()
        wide = self.hidden_size * (2 if self.bidirectional else 1)
        sizes = [self.input_size] + [wide] * (self.num_layers - 1)

        def stack():
            return nn.Sequential(*(cell_type(n, self.hidden_size, self.bias, *args, **kwargs) for n in sizes))
        return (stack(), stack()) if self.bidirectional else stack()

    @staticmethod
    def base_cell():
        raise NotImplementedError

    @staticmethod
    def states_num():
        raise NotImplementedError

    @staticmethod
    def _run(cell, x, state, reverse: bool):
        """One direction of one layer -> (outputs [T, B, H], final state)."""
        single = torch.is_tensor(state) and state.dim() == 2
        T = x.shape[0]
        if isinstance(cell, SpikingRNNCellBase) and type(cell).step is not SpikingRNNCellBase.step:
            ih = cell.linear_ih(x)                      # whole sequence at once
            feed, advance = ih, cell.step
        else:
            feed, advance = x, cell
        outs = [None] * T
        order = range(T - 1, -1, -1) if reverse else range(T)
        for t in order:
            state = advance(feed[t], state)
            outs[t] = _first(state, single)
        return torch.stack(outs), state

    def forward(self, x: torch.Tensor, states=None):
        B, n_states = x.shape[1], self.states_num()
        dirs = 2 if self.bidirectional else 1
        rows = self.num_layers * dirs
        if states is None:
            st = x.new_zeros(n_states, rows, B, self.hidden_size)
        elif isinstance(states, tuple):
            st = torch.stack(states)
        elif isinstance(states, torch.Tensor) and states.dim() == 3:
            st = states.unsqueeze(0)
        else:
            raise TypeError("states must be None, a 3-D torch.Tensor, or a tuple of tensors, "
                            f"but got {type(states).__name__}.")
        if st.dim() != 4 or st.shape[0] != n_states or st.shape[1] != rows:
            raise ValueError(f"states must have shape [{n_states}, {rows}, batch_size, hidden_size], but got {tuple(st.shape)}.")

        masks = None
        if self.training and self.dropout_p > 0 and self.invariant_dropout_mask and self.num_layers > 1:
            masks = F.dropout(x.new_ones(self.num_layers - 1, B, self.hidden_size * dirs), p=self.dropout_p, training=True)

        def pick(row):
            s = st[:, row]
            return s[0] if n_states == 1 else s

        def put(out, row, final):
            if n_states > 1 and isinstance(final, (tuple, list)):
                final = torch.stack(final)
            out[:, row] = final.unsqueeze(0) if n_states == 1 else final

        y, finals = x, torch.empty_like(st)
        for l in range(self.num_layers):
            fwd, s_f = self._run(self.cells[l], y, pick(l), reverse=False)
            put(finals, l, s_f)
            if self.bidirectional:
                bwd, s_b = self._run(self.cells_reverse[l], y, pick(l + self.num_layers), reverse=True)
                put(finals, l + self.num_layers, s_b)
                y = torch.cat((fwd, bwd), dim=-1)
            else:
                y = fwd
            if self.training and self.dropout_p > 0 and l < self.num_layers - 1:
                y = F.dropout(y, p=self.dropout_p, training=True) if masks is None else y * masks[l]
        return (y, finals[0]) if n_states == 1 else (y, tuple(finals))


class SpikingLSTM(SpikingRNNBase):
    def __init__(self, input_size, hidden_size, num_layers, bias=True, dropout_p=0, invariant_dropout_mask=False,
                 bidirectional=False, surrogate_function1=surrogate.Erf(), surrogate_function2=None):
        super().__init__(input_size, hidden_size, num_layers, bias, dropout_p, invariant_dropout_mask, bidirectional,
                         surrogate_function1, surrogate_function2)

    @staticmethod
    def base_cell():
        return SpikingLSTMCell

    @staticmethod
    def states_num():
        return 2


class SpikingVanillaRNN(SpikingRNNBase):
    def __init__(self, input_size, hidden_size, num_layers, bias=True, dropout_p=0, invariant_dropout_mask=False,
                 bidirectional=False, surrogate_function=surrogate.Erf()):
        super().__init__(input_size, hidden_size, num_layers, bias, dropout_p, invariant_dropout_mask, bidirectional,
                         surrogate_function)

    @staticmethod
    def base_cell():
        return SpikingVanillaRNNCell

    @staticmethod
    def states_num():
        return 1


class SpikingGRU(SpikingRNNBase):
    def __init__(self, input_size, hidden_size, num_layers, bias=True, dropout_p=0, invariant_dropout_mask=False,
                 bidirectional=False, surrogate_function1=surrogate.Erf(), surrogate_function2=None):
        super().__init__(input_size, hidden_size, num_layers, bias, dropout_p, invariant_dropout_mask, bidirectional,
                         surrogate_function1, surrogate_function2)

    @staticmethod
    def base_cell():
        return SpikingGRUCell

    @staticmethod
    def states_num():
        return 1
