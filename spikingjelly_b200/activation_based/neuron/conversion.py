"""Neurons used by ANN-to-SNN conversion: few-spike (FS) coding and the SpikeZIP ternary IF.

A few-spike neuron approximates a nonlinearity ``f`` with ``K`` time steps: at step ``k`` it fires
``z_k = H(v - theta_k)``, emits ``d_k z_k`` and subtracts ``h_k z_k`` from ``v``; the table
``(theta, h, d)`` encodes ``f``.  Variants select the table per element (by magnitude or by
region).  Parity: ``neuron/few_spike.py:52-639``, ``neuron/spikezip.py:14-228``.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Union

import weakref

import torch
import torch.nn as nn

from .. import base, functional, surrogate

__all__ = ["FewSpikeNode", "FewSpikeTable", "HGNode", "OutlierAwareThresholdNode", "STBIFNeuron"]

TensorLike1D = Union[torch.Tensor, Sequence[float]]


def _vec(name: str, value: TensorLike1D) -> torch.Tensor:
    t = torch.as_tensor(value)
    if t.dim() != 1:
        raise ValueError(f"{name} must be a 1-D tensor or sequence, but got shape {tuple(t.shape)}.")
    if t.numel() == 0:
        raise ValueError(f"{name} must be non-empty.")
    if torch.is_complex(t):
        raise TypeError(f"{name} must be a real-valued tensor or sequence.")
    if not torch.is_floating_point(t):
        t = t.to(torch.get_default_dtype())
    if not torch.isfinite(t).all():
        raise ValueError(f"{name} must contain only finite values.")
    return t.detach().clone()


class FewSpikeTable:
    """``K`` triples ``(theta_k, h_k, d_k)``: firing threshold, reset amount, output weight."""

    def __init__(self, theta: TensorLike1D, h: TensorLike1D, d: TensorLike1D):
        self.theta, self.h, self.d = _vec("theta", theta), _vec("h", h), _vec("d", d)
        if not (self.theta.shape == self.h.shape == self.d.shape):
            raise ValueError("theta, h and d must have the same shape, but got "
                             f"{tuple(self.theta.shape)}, {tuple(self.h.shape)}, {tuple(self.d.shape)}.")

    @property
    def K(self) -> int:
        return self.theta.numel()


def _require_table(name: str, table, K: Optional[int] = None):
    if not isinstance(table, FewSpikeTable):
        raise TypeError(f"{name} must be FewSpikeTable, but got {type(table).__name__}.")
    if K is not None and table.K != K:
        raise ValueError(f"{name}.K must be {K}, but got {table.K}.")


class FewSpikeNode(nn.Module, base.StepModule):
    """Single-step: returns ``sum_k d_k z_k`` for input ``x``.  Multi-step: input ``[K, ...]`` is
    summed over time into the gate and the output is the sequence ``d_k z_k``."""

    def __init__(self, table: FewSpikeTable, surrogate_function: Optional[surrogate.SurrogateFunctionBase] = None,
                 step_mode: str = "s"):
        super().__init__()
        _require_table("table", table)
        self.register_buffer("theta", table.theta.clone())
        self.register_buffer("h", table.h.clone())
        self.register_buffer("d", table.d.clone())
        self.surrogate_function = surrogate.Sigmoid() if surrogate_function is None else surrogate_function
        self.step_mode = step_mode

    @property
    def K(self) -> int:
        return self.theta.numel()

    @staticmethod
    def _check_input(x, name: str):
        if not isinstance(x, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor.")
        if not torch.is_floating_point(x):
            raise TypeError(f"{name} must be a floating point tensor.")

    def _tables_at(self, k: int, gate):
        """(theta_k, h_k, d_k) broadcastable to ``gate``; overridden by the selecting variants."""
        return self.theta[k], self.h[k], self.d[k]

    def _prepare(self, gate):
        """Returns (initial potential, output multiplier)."""
        return gate, None

    def _forward_from_gate(self, gate: torch.Tensor, return_sequence: bool) -> torch.Tensor:
        v, mult = self._prepare(gate)
        outs = []
        for k in range(self.K):
            theta_k, h_k, d_k = self._tables_at(k, gate)
            z = self.surrogate_function(v - theta_k)
            outs.append(d_k * z)
            v = v - h_k * z
        y = torch.stack(outs, dim=0) if return_sequence else sum(outs[1:], outs[0])
        if mult is not None:
            y = y * (mult.unsqueeze(0) if return_sequence else mult)
        return y

    def single_step_forward(self, x):
        self._check_input(x, "x")
        return self._forward_from_gate(x, return_sequence=False)

    def multi_step_forward(self, x_seq):
        self._check_input(x_seq, "x_seq")
        if x_seq.shape[0] != self.K:
            raise ValueError(f"x_seq.shape[0] must equal K={self.K}, but got {x_seq.shape[0]}.")
        return self._forward_from_gate(x_seq.sum(dim=0), return_sequence=True)

    def forward(self, x):
        return self.single_step_forward(x) if self.step_mode == "s" else self.multi_step_forward(x)

    def extra_repr(self) -> str:
        return f"K={self.K}, step_mode={self.step_mode}"


class OutlierAwareThresholdNode(FewSpikeNode):
    """Sign-symmetric FS neuron with a second table for magnitudes above ``split_threshold``
    (optionally clamped at ``clamp_value``)."""

    def __init__(self, table: FewSpikeTable, outlier_table: FewSpikeTable, split_threshold: float,
                 clamp_value: Optional[float] = None, surrogate_function=None, step_mode: str = "s"):
        _require_table("table", table)
        _require_table("outlier_table", outlier_table, table.K)
        split_threshold = float(split_threshold)
        if not math.isfinite(split_threshold) or split_threshold < 0:
            raise ValueError("split_threshold must be a finite non-negative value.")
        if clamp_value is not None:
            clamp_value = float(clamp_value)
            if not math.isfinite(clamp_value) or clamp_value <= 0:
                raise ValueError("clamp_value must be finite and positive when it is not None.")
            if clamp_value < split_threshold:
                raise ValueError("clamp_value must be no smaller than split_threshold.")
        super().__init__(table, surrogate_function, step_mode)
        for name, src, ref in (("outlier_theta", outlier_table.theta, table.theta), ("outlier_h", outlier_table.h, table.h),
                               ("outlier_d", outlier_table.d, table.d)):
            self.register_buffer(name, src.to(device=ref.device, dtype=ref.dtype).clone())
        self.split_threshold, self.clamp_value = split_threshold, clamp_value

    def _forward_from_gate(self, gate, return_sequence):
        if self.clamp_value is not None:
            gate = gate.clamp(min=-self.clamp_value, max=self.clamp_value)
        self._inlier = gate.abs() <= self.split_threshold
        try:
            return super()._forward_from_gate(gate, return_sequence)
        finally:
            del self._inlier

    def _prepare(self, gate):
        return gate.abs(), torch.sign(gate).detach()

    def _tables_at(self, k, gate):
        m = self._inlier
        return (torch.where(m, self.theta[k], self.outlier_theta[k]), torch.where(m, self.h[k], self.outlier_h[k]),
                torch.where(m, self.d[k], self.outlier_d[k]))

    def extra_repr(self) -> str:
        return super().extra_repr() + f", split_threshold={self.split_threshold}, clamp_value={self.clamp_value}"


class HGNode(FewSpikeNode):
    """FS neuron with one table per input region; regions are separated by ``gate_thresholds``."""

    def __init__(self, tables: Sequence[FewSpikeTable], gate_thresholds: TensorLike1D, surrogate_function=None,
                 step_mode: str = "s"):
        if len(tables) == 0:
            raise ValueError("tables must contain at least one FewSpikeTable.")
        for i, t in enumerate(tables):
            _require_table(f"tables[{i}]", t, tables[0].K if i else None)
        th = torch.as_tensor(gate_thresholds)
        if th.dim() != 1:
            raise ValueError("gate_thresholds must be a 1-D tensor or sequence.")
        if torch.is_complex(th):
            raise TypeError("gate_thresholds must be real-valued.")
        ref = tables[0].theta
        th = th.to(device=ref.device, dtype=ref.dtype)
        if th.numel() != len(tables) - 1:
            raise ValueError("gate_thresholds must have length len(tables) - 1, but got "
                             f"{th.numel()} for {len(tables)} tables.")
        if not torch.isfinite(th).all():
            raise ValueError("gate_thresholds must contain only finite values.")
        if th.numel() > 1 and not torch.all(th[1:] > th[:-1]):
            raise ValueError("gate_thresholds must be strictly increasing.")
        nn.Module.__init__(self)
        self.surrogate_function = surrogate.Sigmoid() if surrogate_function is None else surrogate_function
        self.step_mode = step_mode
        for name, attr in (("region_theta", "theta"), ("region_h", "h"), ("region_d", "d")):
            self.register_buffer(name, torch.stack([getattr(t, attr).to(device=ref.device, dtype=ref.dtype) for t in tables]))
        self.register_buffer("gate_thresholds", th)

    @property
    def K(self) -> int:
        return self.region_theta.shape[1]

    def _forward_from_gate(self, gate, return_sequence):
        self._region = torch.bucketize(gate.detach(), self.gate_thresholds)
        try:
            return super()._forward_from_gate(gate, return_sequence)
        finally:
            del self._region

    def _tables_at(self, k, gate):
        r = self._region
        return self.region_theta[:, k][r], self.region_h[:, k][r], self.region_d[:, k][r]

    def extra_repr(self) -> str:
        return super().extra_repr() + f", regions={self.region_theta.shape[0]}, gate_thresholds={self.gate_thresholds}"


def _scalar(value) -> torch.Tensor:
    return (value if torch.is_tensor(value) else torch.tensor(value)).detach().clone()


class STBIFNeuron(base.MemoryModule):
    """SpikeZIP ternary IF neuron: emits ``+q_threshold``, ``-q_threshold`` or 0; the running count
    ``acc_q`` stays within ``[neg_min, pos_max]`` so that the time-summed output equals the
    ``level``-level quantiser of the converted ANN."""

    def __init__(self, q_threshold, level: int, sym: bool = False, pos_max=None, neg_min=None, step_mode: str = "s"):
        super().__init__()
        self.level = int(level)
        if isinstance(level, bool) or self.level < 2:
            raise ValueError("SpikeZIP quantizer level must be >= 2.")
        self.sym = bool(sym)
        self.register_buffer("q_threshold", _scalar(q_threshold).float())
        self.register_buffer("pos_max", _scalar((self.level // 2 - 1 if self.sym else self.level - 1)
                                                if pos_max is None else pos_max).float())
        self.register_buffer("neg_min", _scalar((-self.level // 2 if self.sym else 0) if neg_min is None else neg_min).float())
        self.step_mode = step_mode
        self.register_memory("q", None)
        self.register_memory("acc_q", None)
        self.register_memory("cur_output", None)
        self.register_memory("is_work", False)

    @classmethod
    def from_quantizer(cls, quantizer: nn.Module) -> "STBIFNeuron":
        pos_max, neg_min = quantizer.pos_max, quantizer.neg_min
        default_level = int(_scalar(pos_max).item()) - int(_scalar(neg_min).item()) + 1
        return cls(quantizer.s, level=int(getattr(quantizer, "level", default_level)), sym=bool(quantizer.sym),
                   pos_max=pos_max, neg_min=neg_min)

    @property
    def supported_backends(self):
        return ("torch", "cuda", "triton")

    def materialize_states(self, inputs, states, step_mode):
        x = inputs[0] if step_mode == "s" else inputs[0][0]
        q, acc_q, cur, work = states
        if q is None or q.shape != x.shape:
            q, acc_q, cur = torch.full_like(x, 0.5), torch.zeros_like(x), torch.zeros_like(x)
        else:
            q, acc_q, cur = q.to(x), acc_q.to(x), cur.to(x)
        return q, acc_q, cur, work

    def single_step_functional_forward(self, inputs, states, **kwargs):
        x = inputs[0]
        q, acc_q, cur, _ = states
        out, q, acc_q, cur = functional.stbif_step(x, q, acc_q, self.q_threshold, self.pos_max, self.neg_min)
        return (out,), (q, acc_q, cur, bool((x != 0).any() | (out != 0).any()))

    def _scalars(self):
        """Python copies of the three scalar buffers, refreshed when a buffer is written (no sync per call)."""
        buffers = (self.q_threshold, self.pos_max, self.neg_min)
        if any(b.is_inference() for b in buffers):          # no version counter to watch: read the values every time
            return tuple(float(b) for b in buffers)
        stamp = (self.q_threshold._version, self.pos_max._version, self.neg_min._version, self.q_threshold.data_ptr())
        if getattr(self, "_scalar_stamp", None) != stamp:
            self._scalar_values = (float(self.q_threshold), float(self.pos_max), float(self.neg_min))
            self._scalar_stamp = stamp
        return self._scalar_values

    def _compiled_run(self, x_seq, q, acc_q, cur):
        """The kernel carries a fourth state in registers: 1 once this element has seen a non-zero input or emitted a
        spike.  The activity flag of the call is then a reduction over one step's worth of values instead of two passes
        over the input and output sequences."""
        from ._compiled import CompiledSequence, compiled_for
        ref = weakref.ref(self)

        def step(x, q, acc, c, seen):
            out, q, acc, c = functional.stbif_step(x, q, acc, *ref()._scalars())
            return out, q, acc, c, torch.where((x != 0) | (out != 0), torch.ones_like(seen), seen)

        seq = compiled_for(self, lambda: CompiledSequence(step, 4, lambda: ("stbif", *ref()._scalars()), "stbif"))
        with torch.no_grad():
            res = seq.run(x_seq, (q, acc_q, cur, torch.zeros_like(q)))
        if res is None:
            return None
        out_seq, (q, acc_q, cur, seen), _ = res
        return out_seq, (q, acc_q, cur), seen.any()

    def multi_step_functional_forward(self, inputs, states, **kwargs):
        x_seq = inputs[0]
        q, acc_q, cur, _ = states
        if x_seq.is_cuda and not (torch.is_grad_enabled() and x_seq.requires_grad):
            res = self._compiled_run(x_seq, q, acc_q, cur)
            if res is not None:
                out_seq, (q, acc_q, cur), active = res
                # the activity flag stays on the device (a 0-d bool tensor): reading it here would stall the stream once
                # per neuron and call
                return (out_seq,), (q, acc_q, cur, active)
        outs = []
        for t in range(x_seq.shape[0]):
            o, q, acc_q, cur = functional.stbif_step(x_seq[t], q, acc_q, self.q_threshold, self.pos_max, self.neg_min)
            outs.append(o)
        out_seq = torch.stack(outs)
        return (out_seq,), (q, acc_q, cur, bool((x_seq != 0).any() | (out_seq != 0).any()))

    @property
    def accumulated(self) -> torch.Tensor:
        if self.acc_q is None:
            raise RuntimeError("STBIFNeuron has no accumulated state before forward.")
        return self.acc_q * self.q_threshold.to(dtype=self.acc_q.dtype)
