"""Stateless neuron dynamics.

``*_step(x, v, …) -> (spike, v_next)`` are the eager single-step rules (numerical
oracle, any device).  ``*_multi_step_cuda(x_seq, v, …, store_v_seq) -> (spike_seq,
v_last, v_seq | None)`` run the whole sequence in one sm_100a kernel; the names the
reference uses for its GPU paths (``*_multi_step_cupy/_triton/_inductor``,
``*_step_cupy``) are aliases of them.

Parity: ``spikingjelly/activation_based/functional/neuron.py`` — ``voltage_reset``
:173-228, ``if_step`` :242-312, ``qif_step`` :315-399, ``eif_step`` :402-488,
``lif_charge``/``lif_step`` :797-933, ``liaf_step`` :936-1027, ``ilif_step``
:1030-1099, ``plif_step`` :1215-1297, ``izhikevich_step`` :1412-1522, ``klif_step``
:1525-1622, ``cuba_lif_step`` :1625-1706, PSN steps :2852-3021, ``gated_lif_step``
:3024-3141, ``stbif_step`` :3144-3247 and the backend shims :1709-2849.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch

from .. import surrogate as _sg

__all__ = [
    "voltage_reset", "if_step", "qif_step", "eif_step", "activation_aware_if_step", "lif_charge", "lif_step",
    "liaf_step", "ilif_step", "plif_step", "izhikevich_step", "klif_step", "cuba_lif_step", "lava_cuba_lif_step",
    "sliding_psn_step", "masked_psn_step", "gated_lif_step", "stbif_step",
    "if_multi_step_cuda", "lif_multi_step_cuda", "plif_multi_step_cuda", "qif_multi_step_cuda",
    "eif_multi_step_cuda", "if_step_cuda", "lif_step_cuda", "torch_multi_step",
    "if_multi_step_cupy", "lif_multi_step_cupy", "plif_multi_step_cupy", "qif_multi_step_cupy",
    "eif_multi_step_cupy", "if_multi_step_triton", "lif_multi_step_triton", "plif_multi_step_triton",
    "if_multi_step_inductor", "lif_multi_step_inductor", "plif_multi_step_inductor", "if_step_cupy",
    "lif_step_cupy", "izhikevich_multi_step_cupy", "izhikevich_multi_step_eager", "activation_aware_if_multi_step_triton",
    "activation_aware_if_sequence",
    "stbif_single_step_triton", "stbif_multi_step_triton", "ilif_multi_step_triton",
]


#: what the functional forms accept as ``surrogate_function``
SurrogateFunction = Callable[[torch.Tensor], torch.Tensor]


def voltage_reset(v, spike, v_threshold: float, v_reset: Optional[float], detach_reset: bool):
    """Soft (``v_reset is None``): ``v - s*v_th``; hard: ``s*v_reset + (1-s)*v``."""
    s = spike.detach() if detach_reset else spike
    if v_reset is None:
        return v - s * v_threshold
    return s * v_reset + (1.0 - s) * v


def if_step(x, v, v_threshold, v_reset, surrogate_function, detach_reset=False):
    h = v + x
    spike = surrogate_function(h - v_threshold)
    return spike, voltage_reset(h, spike, v_threshold, v_reset, detach_reset)


def qif_step(x, v, tau, a0, v_rest, v_c, v_threshold, v_reset, surrogate_function, detach_reset=False):
    h = v + (x + a0 * (v - v_rest) * (v - v_c)) / tau
    spike = surrogate_function(h - v_threshold)
    return spike, voltage_reset(h, spike, v_threshold, v_reset, detach_reset)


def eif_step(x, v, tau, delta_t, theta_rh, v_rest, v_threshold, v_reset, surrogate_function, detach_reset=False):
    h = v + (x + v_rest - v + delta_t * torch.exp((v - theta_rh) / delta_t)) / tau
    spike = surrogate_function(h - v_threshold)
    return spike, voltage_reset(h, spike, v_threshold, v_reset, detach_reset)


def activation_aware_if_step(x, v, v_threshold, v_offset, v_reset, surrogate_function, detach_reset=False):
    """IF with per-channel tensor threshold/offset: fire on ``h + v_offset - v_th``."""
    h = v + x
    spike = surrogate_function(h + v_offset - v_threshold)
    s = spike.detach() if detach_reset else spike
    v_next = h - s * v_threshold if v_reset is None else s * v_reset + (1.0 - s) * h
    return spike, v_next


def lif_charge(x, v, tau: float, decay_input: bool, v_reset: Optional[float]):
    vr = 0.0 if v_reset is None else v_reset
    if decay_input:
        return v + (x - (v - vr)) / tau
    return v - (v - vr) / tau + x


def lif_step(x, v, tau, decay_input, v_threshold, v_reset, surrogate_function, detach_reset=False):
    h = lif_charge(x, v, tau, decay_input, v_reset)
    spike = surrogate_function(h - v_threshold)
    return spike, voltage_reset(h, spike, v_threshold, v_reset, detach_reset)


def liaf_step(x, v, tau, decay_input, v_threshold, v_reset, act, threshold_related, surrogate_function,
              detach_reset=False):
    """Analog output ``act(h [- v_th])``; the spike only drives the reset."""
    h = lif_charge(x, v, tau, decay_input, v_reset)
    out = act(h - v_threshold if threshold_related else h)
    spike = surrogate_function(h - v_threshold)
    return out, voltage_reset(h, spike, v_threshold, v_reset, detach_reset)


def ilif_step(x, v, tau, v_threshold, surrogate_function, detach_reset=False):
    """Integer-valued spikes ``sg(h / v_th)``; always soft reset, input not decayed."""
    h = lif_charge(x, v, tau, False, None)
    spike = surrogate_function(h / v_threshold)
    return spike, voltage_reset(h, spike, v_threshold, None, detach_reset)


def plif_step(x, v, w, decay_input, v_threshold, v_reset, surrogate_function, detach_reset=False):
    r = w.sigmoid()
    vr = 0.0 if v_reset is None else v_reset
    h = v + (x - (v - vr)) * r if decay_input else v - (v - vr) * r + x
    spike = surrogate_function(h - v_threshold)
    return spike, voltage_reset(h, spike, v_threshold, v_reset, detach_reset)


def izhikevich_step(x, v, w, tau, a0, v_rest, v_c, tau_w, a, b, v_threshold, v_reset, surrogate_function,
                    detach_reset=False):
    h = v + (x + a0 * (v - v_rest) * (v - v_c) - w) / tau
    w_next = w + (a * (h - v_rest) - w) / tau_w
    spike = surrogate_function(h - v_threshold)
    s = spike.detach() if detach_reset else spike
    v_next = h - s * v_threshold if v_reset is None else (1.0 - s) * h + spike * v_reset
    return spike, v_next, w_next + b * spike


def klif_step(x, v, k, tau, decay_input, scale_reset, v_threshold, v_reset, surrogate_function, detach_reset=False):
    h = torch.relu(k * lif_charge(x, v, tau, decay_input, v_reset))
    spike = surrogate_function(h - v_threshold)
    if scale_reset:
        return spike, voltage_reset(h / k, spike, v_threshold / k, v_reset, detach_reset)
    return spike, voltage_reset(h, spike, v_threshold, v_reset, detach_reset)


def cuba_lif_step(x, current, v, current_decay, voltage_decay, v_threshold, v_reset, surrogate_function,
                  detach_reset=False):
    current_next = current * current_decay + x
    h = v * voltage_decay + current_next
    spike = surrogate_function(h - v_threshold)
    return spike, current_next, voltage_reset(h, spike, v_threshold, v_reset, detach_reset)


def lava_cuba_lif_step(x, current_state, voltage_state, current_decay, voltage_decay, s_scale, v_threshold,
                       v_threshold_eps, v_reset, surrogate_function, detach_reset=False):
    from ..lava_exchange import LeakyIntegratorStep, step_quantize
    cur = LeakyIntegratorStep.apply(x, step_quantize(current_decay), current_state.contiguous(), s_scale)
    h = LeakyIntegratorStep.apply(cur, step_quantize(voltage_decay), voltage_state.contiguous(), s_scale)
    spike = surrogate_function(h - (v_threshold + v_threshold_eps))
    return spike, cur, voltage_reset(h, spike, v_threshold, v_reset, detach_reset)


def sliding_psn_step(x, queue, weight, bias, surrogate_function):
    """One step of the sliding parallel spiking neuron: weighted sum of the last
    ``k = weight.numel()`` inputs (a FIFO ``queue`` of flattened tensors)."""
    k = weight.numel()
    queue = (*queue, x.flatten())[-k:]
    w = weight[k - len(queue):k].unsqueeze(-1)
    h = torch.sum(w * torch.stack(queue), 0)
    return surrogate_function(h + bias).view(x.shape), queue


def masked_psn_step(x, time_step, queue, masked_weight, bias, k, surrogate_function):
    queue = (*queue, x.flatten())[-k:]
    w = masked_weight[time_step, time_step + 1 - len(queue):time_step + 1]
    h = torch.sum(w.unsqueeze(-1) * torch.stack(queue), 0)
    return surrogate_function(h + bias[time_step]).view(x.shape), time_step + 1, queue


def gated_lif_step(x, v, spike, alpha, beta, gamma, tau, v_threshold, linear_decay, v_subreset, conduct,
                   surrogate_function):
    cur = x * (1 - beta * (1 - conduct))
    keep = 1 - alpha * (1 - tau)
    v_next = (keep * v - (1 - alpha) * linear_decay) + cur
    v_next = v_next - keep * v * gamma * spike - (1 - gamma) * v_subreset * spike
    return surrogate_function(v_next - v_threshold), v_next


def stbif_step(x, q, acc_q, q_threshold, pos_max, neg_min):
    """SpikeZIP ternary IF: emits +1/-1/0 (times ``q_threshold``), with the running
    count ``acc_q`` clamped to ``[neg_min, pos_max]``."""
    q_threshold, pos_max, neg_min = (t.to(x) if isinstance(t, torch.Tensor) else t for t in (q_threshold, pos_max, neg_min))
    q_next = q + (x / q_threshold).detach()
    acc = torch.round(acc_q)
    pos = (q_next - 1 >= 0) & (acc < pos_max)
    neg = (q_next < 0) & (acc > neg_min)
    cur = pos.to(x.dtype) - neg.to(x.dtype)
    acc = acc + cur
    q_next = torch.where(pos, q_next - 1, q_next)
    q_next = torch.where(neg, q_next + 1, q_next)
    return cur * q_threshold, q_next, acc, cur


# ------------------------------------------------------------ native dispatch
def _spec(kind, v_threshold, v_reset, surrogate_function, detach_reset, tau=2.0, q=(0.0, 0.0, 0.0)):
    from ...ops.neuron_scan import KIND, NeuronSpec
    sg = _sg.surrogate_spec(surrogate_function)
    if sg is None:
        if surrogate_function is _sg.heaviside:
            sg = (15, 0.0, 0.0)   # forward-only use: derivative irrelevant
        else:
            raise NotImplementedError(
                f"{surrogate_function!r} has no native-kernel form; use backend='torch' for it")
    return NeuronSpec(KIND[kind], float(v_threshold), None if v_reset is None else float(v_reset), float(tau),
                      tuple(float(t) for t in q), sg, bool(detach_reset))


def _native(x_seq, v, spec, store_v_seq, r=None):
    from ...ops.neuron_scan import multistep_neuron
    spike, v_last, v_seq, _ = multistep_neuron(x_seq, v, spec, r=r, store_v_seq=store_v_seq)
    return spike, v_last, v_seq


def torch_multi_step(step_fn: Callable, x_seq, v, store_v_seq: bool):
    """Eager loop used when a tensor is not on a CUDA device."""
    spikes, vs = [], []
    for t in range(x_seq.shape[0]):
        s, v = step_fn(x_seq[t], v)
        spikes.append(s)
        if store_v_seq:
            vs.append(v)
    return torch.stack(spikes), v, (torch.stack(vs) if store_v_seq else None)


def _v_like(v, x0):
    return torch.full_like(x0, v) if not isinstance(v, torch.Tensor) else v


def if_multi_step_cuda(x_seq, v, v_threshold, v_reset, surrogate_function, detach_reset=False, store_v_seq=False):
    if not x_seq.is_cuda:
        return torch_multi_step(lambda x, vv: if_step(x, vv, v_threshold, v_reset, surrogate_function, detach_reset),
                                x_seq, _v_like(v, x_seq[0]), store_v_seq)
    return _native(x_seq, v, _spec("if", v_threshold, v_reset, surrogate_function, detach_reset), store_v_seq)


def lif_multi_step_cuda(x_seq, v, tau, decay_input, v_threshold, v_reset, surrogate_function, detach_reset=False,
                        store_v_seq=False):
    if not x_seq.is_cuda:
        return torch_multi_step(
            lambda x, vv: lif_step(x, vv, tau, decay_input, v_threshold, v_reset, surrogate_function, detach_reset),
            x_seq, _v_like(v, x_seq[0]), store_v_seq)
    kind = "lif_di" if decay_input else "lif_ndi"
    return _native(x_seq, v, _spec(kind, v_threshold, v_reset, surrogate_function, detach_reset, tau), store_v_seq)


def plif_multi_step_cuda(x_seq, v, reciprocal_tau, decay_input, v_threshold, v_reset, surrogate_function,
                         detach_reset=False, store_v_seq=False):
    """``reciprocal_tau`` is the tensor ``sigmoid(w)`` (its gradient flows back to ``w``)."""
    if not x_seq.is_cuda:
        vr = 0.0 if v_reset is None else v_reset

        def step(x, vv):
            h = vv + (x - (vv - vr)) * reciprocal_tau if decay_input else vv - (vv - vr) * reciprocal_tau + x
            s = surrogate_function(h - v_threshold)
            return s, voltage_reset(h, s, v_threshold, v_reset, detach_reset)
        return torch_multi_step(step, x_seq, _v_like(v, x_seq[0]), store_v_seq)
    kind = "plif_di" if decay_input else "plif_ndi"
    r = reciprocal_tau.to(torch.float32).reshape(1)
    return _native(x_seq, v, _spec(kind, v_threshold, v_reset, surrogate_function, detach_reset), store_v_seq, r=r)


def qif_multi_step_cuda(x_seq, v, tau, v_c, a0, v_threshold, v_rest, v_reset, surrogate_function,
                        detach_reset=False, store_v_seq=False):
    if not x_seq.is_cuda:
        return torch_multi_step(
            lambda x, vv: qif_step(x, vv, tau, a0, v_rest, v_c, v_threshold, v_reset, surrogate_function, detach_reset),
            x_seq, _v_like(v, x_seq[0]), store_v_seq)
    spec = _spec("qif", v_threshold, v_reset, surrogate_function, detach_reset, tau, (a0, v_rest, v_c))
    return _native(x_seq, v, spec, store_v_seq)


def eif_multi_step_cuda(x_seq, v, tau, v_threshold, v_reset, v_rest, theta_rh, delta_T, surrogate_function,
                        detach_reset=False, store_v_seq=False):
    if not x_seq.is_cuda:
        return torch_multi_step(
            lambda x, vv: eif_step(x, vv, tau, delta_T, theta_rh, v_rest, v_threshold, v_reset, surrogate_function,
                                   detach_reset), x_seq, _v_like(v, x_seq[0]), store_v_seq)
    spec = _spec("eif", v_threshold, v_reset, surrogate_function, detach_reset, tau, (delta_T, theta_rh, v_rest))
    return _native(x_seq, v, spec, store_v_seq)


def if_step_cuda(x, v, v_threshold, v_reset, surrogate_function, detach_reset=False):
    """Single step through the scan kernel (T = 1)."""
    s, v_next, _ = if_multi_step_cuda(x.unsqueeze(0), v, v_threshold, v_reset, surrogate_function, detach_reset)
    return s[0], v_next


def lif_step_cuda(x, v, tau, decay_input, v_threshold, v_reset, surrogate_function, detach_reset=False):
    s, v_next, _ = lif_multi_step_cuda(x.unsqueeze(0), v, tau, decay_input, v_threshold, v_reset,
                                       surrogate_function, detach_reset)
    return s[0], v_next


def izhikevich_multi_step_eager(x_seq, v, w, tau, v_threshold, v_reset, v_rest, v_c, a0, tau_w, a, b,
                                surrogate_function, detach_reset=False, store_v_seq=False):
    """Two-state neuron: runs the eager rule per step on whatever device holds the data."""
    spikes, vs, ws = [], [], []
    for t in range(x_seq.shape[0]):
        s, v, w = izhikevich_step(x_seq[t], v, w, tau, a0, v_rest, v_c, tau_w, a, b, v_threshold, v_reset,
                                  surrogate_function, detach_reset)
        spikes.append(s)
        if store_v_seq:
            vs.append(v)
            ws.append(w)
    return (torch.stack(spikes), v, w, torch.stack(vs) if store_v_seq else None,
            torch.stack(ws) if store_v_seq else None)


def activation_aware_if_sequence(x_seq, v, v_threshold, v_offset, v_reset, store_v_seq=False):
    """Inference-only per-channel-threshold IF over a sequence; ``v_threshold`` / ``v_offset`` broadcast against one step."""
    with torch.no_grad():
        spikes, vs = [], []
        for t in range(x_seq.shape[0]):
            s, v = activation_aware_if_step(x_seq[t], v, v_threshold, v_offset, v_reset, _sg.heaviside)
            spikes.append(s)
            if store_v_seq:
                vs.append(v)
        return torch.stack(spikes), v, (torch.stack(vs) if store_v_seq else None)


def activation_aware_if_multi_step_triton(x_seq, v, v_threshold, v_offset, channel_size: int, inner_size: int, v_reset, store_v_seq=False):
    """The reference's calling convention: one step of ``x_seq`` is laid out as ``[outer, channel_size, inner_size]`` (flattened or
    not) and ``v_threshold`` / ``v_offset`` hold one value per channel (or one value in all)."""
    step = x_seq.shape[1:]
    if channel_size * inner_size == 0 or x_seq[0].numel() % (channel_size * inner_size):
        raise ValueError(f"a step of {x_seq[0].numel()} elements is not a multiple of channel_size * inner_size = {channel_size * inner_size}")
    per = lambda t: t if not torch.is_tensor(t) or t.numel() == 1 else t.reshape(1, 1, channel_size, 1)          # noqa: E731
    xs = x_seq.reshape(x_seq.shape[0], -1, channel_size, inner_size)
    s, v_last, v_seq = activation_aware_if_sequence(xs, v.reshape(xs.shape[1:]), per(v_threshold), per(v_offset), v_reset, store_v_seq)
    return s.reshape(x_seq.shape), v_last.reshape(step), (None if v_seq is None else v_seq.reshape(x_seq.shape))


def ilif_multi_step_triton(x_seq, v, tau, v_threshold, surrogate_function, detach_reset=False, store_v_seq=False):
    return torch_multi_step(lambda x, vv: ilif_step(x, vv, tau, v_threshold, surrogate_function, detach_reset),
                            x_seq, _v_like(v, x_seq[0]), store_v_seq)


def stbif_single_step_triton(x, q, acc_q, q_threshold, pos_max, neg_min):
    out, q, acc, cur = stbif_step(x, q, acc_q, q_threshold, pos_max, neg_min)
    return out, q, acc, cur, cur.ne(0).any().reshape(1)


def stbif_multi_step_triton(x_seq, q, acc_q, q_threshold, pos_max, neg_min):
    outs = []
    cur = torch.zeros_like(x_seq[0])
    for t in range(x_seq.shape[0]):
        o, q, acc_q, cur = stbif_step(x_seq[t], q, acc_q, q_threshold, pos_max, neg_min)
        outs.append(o)
    return torch.stack(outs), q, acc_q, cur


# Names of the reference's GPU paths: all served by the native kernels.
if_multi_step_cupy = if_multi_step_triton = if_multi_step_inductor = if_multi_step_cuda
lif_multi_step_cupy = lif_multi_step_triton = lif_multi_step_inductor = lif_multi_step_cuda


# The remaining back-end names take their arguments in the reference's order (functional/neuron.py:1300-2800 there).
def plif_multi_step_cupy(x_seq, v, w, decay_input, v_threshold, v_reset, surrogate_function, detach_reset=False, store_v_seq=False):
    """``w``: the raw learnable parameter; ``1 / tau = sigmoid(w)`` is taken here."""
    return plif_multi_step_cuda(x_seq, v, w.sigmoid(), decay_input, v_threshold, v_reset, surrogate_function, detach_reset, store_v_seq)


plif_multi_step_triton = plif_multi_step_inductor = plif_multi_step_cupy


def qif_multi_step_cupy(x_seq, v, tau, v_threshold, v_reset, v_rest, v_c, a0, detach_reset, surrogate_function, store_v_seq=False):
    return qif_multi_step_cuda(x_seq, v, tau, v_c, a0, v_threshold, v_rest, v_reset, surrogate_function, detach_reset, store_v_seq)


def eif_multi_step_cupy(x_seq, v, tau, v_threshold, v_reset, v_rest, theta_rh, delta_t, detach_reset, surrogate_function, store_v_seq=False):
    return eif_multi_step_cuda(x_seq, v, tau, v_threshold, v_reset, v_rest, theta_rh, delta_t, surrogate_function, detach_reset, store_v_seq)


def izhikevich_multi_step_cupy(x_seq, v, w, tau, v_threshold, v_reset, v_rest, a, b, tau_w, v_c, a0, detach_reset, surrogate_function,
                               store_state_seq=False):
    """``(spike_seq, v, w, v_seq | None, w_seq | None)``; on a CUDA tensor the sequence runs as one generated kernel."""
    from ..cuda_kernel.neuron_kernel.multi_step.izhikevich import izhikevich_multi_step
    if x_seq.is_cuda:
        s, v_seq, w_seq = izhikevich_multi_step(x_seq, v, w, tau, v_threshold, v_reset, v_rest, a, b, tau_w, v_c, a0, detach_reset, surrogate_function)
        return s, v_seq[-1], w_seq[-1], (v_seq if store_state_seq else None), (w_seq if store_state_seq else None)
    return izhikevich_multi_step_eager(x_seq, v, w, tau, v_threshold, v_reset, v_rest, v_c, a0, tau_w, a, b, surrogate_function, detach_reset,
                                       store_state_seq)


if_step_cupy = if_step_cuda
lif_step_cupy = lif_step_cuda
