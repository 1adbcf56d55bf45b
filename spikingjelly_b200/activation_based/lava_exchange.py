"""Bridge to Lava-DL (Loihi): fixed-point CUBA LIF neuron that reproduces the chip's integer arithmetic in PyTorch,
the weight / batch-norm quantisers that go with it, a synapse+neuron container that trains under that arithmetic,
and converters to ``lava.lib.dl.slayer`` blocks (available when the ``lava`` package is importable).

Arithmetic (``spikingjelly/activation_based/lava_exchange.py:15-240``): states are held at a fixed-point scale
``s_scale = 64 * scale``; one leaky-integrator step is ``y = trunc(state * s_scale * (4096 - decay) / 4096) / s_scale
+ x`` with truncation toward zero (an arithmetic right shift of the magnitude), decays are integers in
``[0, 4096]``, weights are even multiples of ``1 / scale`` in ``[-256, 254] / scale``.
"""
from __future__ import annotations

from typing import Callable, Optional, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..logger import logger
from . import base, neuron, surrogate
from .functional import neuron as functional

__all__ = ["step_quantize_forward", "step_quantize", "quantize_8b", "quantize_8bit", "right_shift_to_zero", "BatchNorm2d",
           "LeakyIntegratorStep", "CubaLIFNode", "SumPool2d", "BlockContainer", "TNX_to_NXT", "NXT_to_TNX",
           "lava_neuron_forward", "to_lava_neuron_param_dict", "to_lava_neuron", "linear_to_lava_synapse_dense",
           "conv2d_to_lava_synapse_conv", "avgpool2d_to_lava_synapse_pool", "to_lava_block_dense", "to_lava_block_conv",
           "to_lava_block_pool", "to_lava_block_flatten", "to_lava_blocks", "slayer"]

_hw_bits = 12

try:
    import lava.lib.dl.slayer as slayer
except (ImportError, OSError) as _e:          # pragma: no cover - depends on the environment
    logger.debug("lava_exchange: lava-dl is not importable (%s); converters to slayer blocks are disabled", _e)
    slayer = None


def _need_lava():
    if slayer is None:
        raise ImportError("this function needs the `lava-dl` package (lava.lib.dl.slayer)")
    return slayer


# ------------------------------------------------------------------------------- quantisers
def step_quantize_forward(x: torch.Tensor, step: float):
    """Nearest multiple of ``step`` (ties to even, as ``torch.round``)."""
    return torch.round(x / step) * step


class step_quantize_atgf(torch.autograd.Function):
    """Straight-through estimator around :func:`step_quantize_forward`."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, step: float = 1.0):
        return step_quantize_forward(x, step)

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output, None


def step_quantize(x: torch.Tensor, step: float = 1.0):
    return step_quantize_atgf.apply(x, step)


def quantize_8b(x, scale, descale=False):
    """8-bit weights as Loihi stores them: even multiples of ``1 / scale``, clamped to ``[-256, 255] / scale``;
    ``descale`` returns the integer mantissa instead."""
    q = step_quantize(x, step=2 / scale).clamp(-256 / scale, 255 / scale)
    return q * scale if descale else q


quantize_8bit = quantize_8b


def right_shift_to_zero(x: torch.Tensor, bits: int):
    """Integer division by ``2 ** bits`` that truncates toward zero for negative values too."""
    if x.dtype not in (torch.int32, torch.int64):
        raise AssertionError("right_shift_to_zero expects int32 or int64")
    return (torch.sign(x) * (torch.abs(x) >> bits)).to(x.dtype)


def _listep_forward(x, decay, state, w_scale: int, dtype: torch.dtype = torch.int32, hw_bits: int = 12):
    kept = right_shift_to_zero((state * w_scale).to(dtype) * ((1 << hw_bits) - decay.to(dtype)), hw_bits)
    return (kept + (w_scale * x).to(dtype)) / w_scale


def _listep_backward(grad_output, decay, state, hw_bits: int = 12):
    unit = 1 << hw_bits
    return grad_output, (-state / unit * grad_output).sum(), (1 - decay / unit) * grad_output


class LeakyIntegratorStep(torch.autograd.Function):
    """``y = state * (1 - decay / 4096) + x`` in the chip's integer arithmetic; gradients of the real-valued formula."""

    @staticmethod
    def forward(ctx, x, decay, state, w_scale):
        out = _listep_forward(x, decay, state, w_scale, dtype=torch.int64, hw_bits=_hw_bits)
        ctx.save_for_backward(decay, state)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        decay, state = ctx.saved_tensors
        gx, gd, gs = _listep_backward(grad_output, decay, state, hw_bits=_hw_bits)
        return gx, gd, gs, None


class BatchNorm2d(nn.Module):
    """Weight-scale batch norm of Lava-DL: subtract the (8-bit quantised) channel mean, divide by ONE standard deviation
    for the whole tensor rounded up to a power of two in ``2 ** [-weight_exp_bits, weight_exp_bits]`` (a shift)."""

    def __init__(self, num_features: int, eps: float = 1e-05, momentum: float = 0.1, track_running_stats: bool = True,
                 weight_exp_bits: int = 3, pre_hook_fx: Callable = lambda x: x):
        super().__init__()
        self.num_features, self.eps, self.momentum = num_features, eps, momentum
        self.track_running_stats, self.weight_exp_bits, self.pre_hook_fx = track_running_stats, weight_exp_bits, pre_hook_fx
        self.register_buffer("running_mean", torch.zeros(num_features))
        self.register_buffer("running_var", torch.zeros(1))

    def to_lava(self):
        bn = _need_lava().neuron.norm.WgtScaleBatchNorm(num_features=self.num_features, momentum=self.momentum,
                                                        weight_exp_bits=self.weight_exp_bits, eps=self.eps,
                                                        pre_hook_fx=self.pre_hook_fx)
        bn.load_state_dict(self.state_dict())
        return bn

    def forward(self, x: torch.Tensor):
        if self.track_running_stats and self.training:
            mean = torch.mean(x, dim=(0, 2, 3), keepdim=True)
            var = torch.var(x, unbiased=False)
            n = x.numel() / self.num_features
            with torch.no_grad():
                self.running_mean = (1.0 - self.momentum) * self.running_mean + self.momentum * mean.squeeze()
                self.running_var = (1.0 - self.momentum) * self.running_var + self.momentum * var * n / (n + 1)
        else:
            mean, var = self.running_mean.view(1, -1, 1, 1), self.running_var.view(1, -1, 1, 1)
        shift = torch.ceil(torch.log2(torch.sqrt(var + self.eps))).clamp(-self.weight_exp_bits, self.weight_exp_bits)
        return (x - self.pre_hook_fx(mean)) / torch.pow(2.0, shift)


# ------------------------------------------------------------------------------- neuron
class CubaLIFNode(neuron.BaseNode):
    """Current-based LIF with Loihi's fixed-point state updates: ``i[t] = (1 - a_i) i[t-1] + x[t]``,
    ``v[t] = (1 - a_v) v[t-1] + i[t]``, spike when ``v > v_threshold`` (realised as ``v + eps >= v_threshold``), hard
    reset to 0.  ``current_decay`` / ``voltage_decay`` are given in ``[0, 1]`` and stored times 4096."""

    def __init__(self, current_decay: Union[float, torch.Tensor], voltage_decay: Union[float, torch.Tensor],
                 v_threshold: float = 1.0, v_reset: float = 0.0, scale=1 << 6, requires_grad=False,
                 surrogate_function: Callable = surrogate.Sigmoid(), norm: Optional[BatchNorm2d] = None, detach_reset=False,
                 step_mode="s", backend="torch", store_v_seq: bool = False, store_i_seq: bool = False):
        self.lava_cuba_neuron_params = {"threshold": v_threshold, "current_decay": current_decay,
                                        "voltage_decay": voltage_decay, "scale": scale}
        super().__init__(v_threshold=v_threshold, v_reset=v_reset, surrogate_function=surrogate_function,
                         detach_reset=detach_reset, step_mode=step_mode, backend=backend, store_v_seq=store_v_seq)
        self.store_i_seq = store_i_seq
        if v_reset != 0.0:
            raise AssertionError("CubaLIFNode only supports for hard reset with v_reset = 0. !")
        self.requires_grad = requires_grad
        self._scale, self._s_scale, self._p_scale = int(scale), int(scale * (1 << 6)), 1 << _hw_bits
        self.v_threshold_eps = 0.01 / self.s_scale
        cd = torch.as_tensor(self.p_scale * current_decay, dtype=torch.float32).clone()
        vd = torch.as_tensor(self.p_scale * voltage_decay, dtype=torch.float32).clone()
        if requires_grad:
            self.current_decay, self.voltage_decay = nn.Parameter(cd), nn.Parameter(vd)
        else:
            self.register_buffer("current_decay", cd)
            self.register_buffer("voltage_decay", vd)
        self.register_memory("current_state", 0.0)
        self.register_memory("voltage_state", 0.0)
        self.clamp_decay_parameters()
        self.norm = norm
        if norm is not None:
            if not isinstance(norm, BatchNorm2d):
                raise NotImplementedError(norm)
            norm.pre_hook_fx = self.quantize_8bit

    def quantize_8bit(self, x, descale=False):
        return quantize_8b(x, scale=self.scale, descale=descale)

    def clamp_decay_parameters(self):
        with torch.no_grad():
            self.current_decay.data.clamp_(min=0.0, max=self.p_scale)
            self.voltage_decay.data.clamp_(min=0.0, max=self.p_scale)

    @property
    def scale(self):
        """Weight scale: weights are multiples of ``2 / scale``."""
        return self._scale

    @property
    def s_scale(self):
        """State scale: currents and voltages are multiples of ``1 / s_scale``."""
        return self._s_scale

    @property
    def p_scale(self):
        """Decay scale: ``4096`` means a decay of 1."""
        return self._p_scale

    @property
    def store_i_seq(self):
        return self._store_i_seq

    @store_i_seq.setter
    def store_i_seq(self, value: bool):
        self._store_i_seq = value
        self.i_seq = None

    def reset(self):
        super().reset()
        self.i_seq = None

    @property
    def supported_backends(self):
        if self.step_mode in ("s", "m"):
            return ("torch",)
        raise ValueError(f"self.step_mode should be 's' or 'm', but get {self.step_mode} instead.")

    def materialize_states(self, inputs, states, step_mode):
        x = inputs[0][0] if step_mode == "m" else inputs[0]
        fixed = []
        for st in states[-2:]:
            if not isinstance(st, torch.Tensor) or st.shape != x.shape:
                st = torch.zeros_like(x)
            elif st.dtype != x.dtype or st.device != x.device:
                st = st.to(dtype=x.dtype, device=x.device)
            fixed.append(st)
        return (*states[:-2], *fixed)

    def single_step_functional_forward(self, inputs, states, **kwargs):
        x = inputs[0]
        cur, vol = states[-2:]
        cd = self.current_decay.clamp(min=0.0, max=self.p_scale) if self.requires_grad else self.current_decay
        vd = self.voltage_decay.clamp(min=0.0, max=self.p_scale) if self.requires_grad else self.voltage_decay
        if self.norm is None:
            spike, cur, vol = functional.lava_cuba_lif_step(x, cur, vol, cd, vd, self.s_scale, self.v_threshold,
                                                            self.v_threshold_eps, self.v_reset, self.surrogate_function,
                                                            self.detach_reset)
            return (spike,), (*states[:-2], cur, vol)
        cur = self.norm(LeakyIntegratorStep.apply(x, step_quantize(cd), cur.contiguous(), self.s_scale))
        vol = LeakyIntegratorStep.apply(cur, step_quantize(vd), vol.contiguous(), self.s_scale)
        spike = self.surrogate_function(vol - (self.v_threshold + self.v_threshold_eps))
        vol = functional.voltage_reset(vol, spike, self.v_threshold, self.v_reset, self.detach_reset)
        return (spike,), (*states[:-2], cur, vol)

    def single_step_forward(self, x: torch.Tensor, *args, **kwargs):
        states = self.materialize_states((x,), tuple(self._memories.values()), "s")
        outs, states = self.single_step_functional_forward((x,), states, **kwargs)
        self._commit(states)
        return outs[0]

    def multi_step_forward(self, x_seq: torch.Tensor, *args, **kwargs):
        states = self.materialize_states((x_seq,), tuple(self._memories.values()), "m")
        spikes, v_steps, i_steps = [], [], []
        for t in range(x_seq.shape[0]):
            outs, states = self.single_step_functional_forward((x_seq[t],), states, **kwargs)
            spikes.append(outs[0])
            if self.store_v_seq:
                v_steps.append(states[-1])
            if self.store_i_seq:
                i_steps.append(states[-2])
        self._commit(states)
        if self.store_v_seq:
            self.v_seq = torch.stack(v_steps)
        if self.store_i_seq:
            self.i_seq = torch.stack(i_steps)
        return torch.stack(spikes)


# ------------------------------------------------------------------------------- layout helpers
def TNX_to_NXT(x_seq: torch.Tensor):
    """``[T, N, *] -> [N, *, T]`` (Lava keeps time last)."""
    return x_seq.permute(*range(1, x_seq.dim()), 0)


def NXT_to_TNX(x_seq: torch.Tensor):
    return x_seq.permute(x_seq.dim() - 1, *range(x_seq.dim() - 1))


def lava_neuron_forward(lava_neuron: nn.Module, x_seq: torch.Tensor, v: Union[torch.Tensor, float]):
    """Runs a slayer neuron on a ``[T, N, *]`` sequence and returns ``(spikes [T, N, *], final voltage)``."""
    squeeze = x_seq.dim() == 2
    if squeeze:
        x_seq = x_seq.unsqueeze(1)
    if isinstance(v, float):
        v = torch.full_like(x_seq[0], v)
    shape = x_seq.shape
    lava_neuron.voltage_state = v
    spike = lava_neuron(x_seq.flatten(2).permute(1, 2, 0)).permute(2, 0, 1).reshape(shape)
    v = lava_neuron.voltage_state.reshape(shape[1:])
    return (spike.squeeze(1), v.squeeze(1)) if squeeze else (spike, v)


# ------------------------------------------------------------------------------- converters
def check_instance(m, instance):
    if not isinstance(m, instance):
        raise ValueError(f"expected {m} with type {instance}, but got {m} with type {type(m)}!")


def check_no_bias(m):
    if m.bias is not None:
        raise ValueError(f"lava does not support for {type(m)} with bias!")


def to_lava_neuron_param_dict(sj_ms_neuron: nn.Module):
    """Parameters of ``slayer.neuron.cuba.Neuron`` equivalent to an IF node or to a LIF node with
    ``decay_input=False`` (both with ``v_reset = 0``)."""
    if not isinstance(sj_ms_neuron, (neuron.IFNode, neuron.LIFNode)):
        raise NotImplementedError(sj_ms_neuron)
    if sj_ms_neuron.v_reset != 0.0:
        raise ValueError("lava only supports for v_reset == 0!")
    voltage_decay = 0.0
    if isinstance(sj_ms_neuron, neuron.LIFNode):
        if sj_ms_neuron.decay_input:
            raise ValueError("lava only supports for decay_input == False!")
        voltage_decay = 1.0 / sj_ms_neuron.tau
    return {"threshold": sj_ms_neuron.v_threshold, "current_decay": 1.0, "voltage_decay": voltage_decay, "tau_grad": 1,
            "scale_grad": 1, "scale": sj_ms_neuron.lava_s_cale, "norm": None, "dropout": None, "shared_param": True,
            "persistent_state": True, "requires_grad": False, "graded_spike": False}


def to_lava_neuron(sj_ms_neuron: nn.Module):
    return _need_lava().neuron.cuba.Neuron(**to_lava_neuron_param_dict(sj_ms_neuron))


def linear_to_lava_synapse_dense(fc: nn.Linear):
    check_instance(fc, nn.Linear)
    check_no_bias(fc)
    dense = _need_lava().synapse.Dense(fc.in_features, fc.out_features)
    dense.weight.data[:, :, 0, 0, 0] = fc.weight.data.clone()            # slayer synapses are Conv3d over [C, H, W, T]
    return dense


def _conv_kwargs(conv: nn.Conv2d) -> dict:
    return dict(in_features=conv.in_channels, out_features=conv.out_channels, kernel_size=conv.kernel_size, stride=conv.stride,
                padding=conv.padding, dilation=conv.dilation, groups=conv.groups)


def conv2d_to_lava_synapse_conv(conv2d_nn: nn.Conv2d):
    check_instance(conv2d_nn, nn.Conv2d)
    check_no_bias(conv2d_nn)
    conv = _need_lava().synapse.Conv(**_conv_kwargs(conv2d_nn))
    conv.weight.data[:, :, :, :, 0] = conv2d_nn.weight.data.clone()
    return conv


def _warn_sum_pool():
    logger.warning("The lava slayer pool layer applies sum pooling, rather than average pooling; a sum pooling layer is returned.")


def avgpool2d_to_lava_synapse_pool(pool2d_nn: nn.AvgPool2d):
    check_instance(pool2d_nn, nn.AvgPool2d)
    _warn_sum_pool()
    return _need_lava().synapse.Pool(pool2d_nn.kernel_size, pool2d_nn.stride, pool2d_nn.padding)


def _block_extra(quantize_to_8bit: bool) -> dict:
    # slayer blocks quantise weights to 8 bits by default; pre_hook_fx=None switches that off
    return dict(delay_shift=False) if quantize_to_8bit else dict(delay_shift=False, pre_hook_fx=None)


def to_lava_block_dense(fc: nn.Linear, sj_ms_neuron: nn.Module, quantize_to_8bit: bool = True):
    check_instance(fc, nn.Linear)
    check_no_bias(fc)
    block = _need_lava().block.cuba.Dense(to_lava_neuron_param_dict(sj_ms_neuron), fc.in_features, fc.out_features,
                                          **_block_extra(quantize_to_8bit))
    block.synapse.weight.data[:, :, 0, 0, 0] = fc.weight.data.clone()
    return block


def to_lava_block_conv(conv2d_nn: nn.Conv2d, sj_ms_neuron: nn.Module, quantize_to_8bit: bool = True):
    check_instance(conv2d_nn, nn.Conv2d)
    check_no_bias(conv2d_nn)
    block = _need_lava().block.cuba.Conv(to_lava_neuron_param_dict(sj_ms_neuron), **_conv_kwargs(conv2d_nn),
                                         **_block_extra(quantize_to_8bit))
    block.synapse.weight.data[:, :, :, :, 0] = conv2d_nn.weight.data.clone()
    return block


def to_lava_block_pool(pool2d_nn: nn.AvgPool2d, sj_ms_neuron: nn.Module, quantize_to_8bit: bool = True):
    check_instance(pool2d_nn, nn.AvgPool2d)
    block = _need_lava().block.cuba.Pool(to_lava_neuron_param_dict(sj_ms_neuron), pool2d_nn.kernel_size, pool2d_nn.stride,
                                         pool2d_nn.padding, **_block_extra(quantize_to_8bit))
    _warn_sum_pool()
    return block


def to_lava_block_flatten(flatten_nn: nn.Flatten):
    check_instance(flatten_nn, nn.Flatten)
    if flatten_nn.start_dim != 1:
        raise ValueError("lava only supports for flatten_nn.start_dim == 1!")
    return _need_lava().block.cuba.Flatten()


def to_lava_blocks(net: Union[list, tuple, nn.Sequential]):
    """``[synapse, neuron, synapse, neuron, ..., Flatten, ...]`` -> list of slayer blocks.  Slayer pools sum instead of
    averaging, so the weights of the layer that follows a pool are divided by the pool's window size."""
    blocks, i, pending_div = [], 0, None
    spiking = (neuron.IFNode, neuron.LIFNode)
    while i < len(net):
        m = net[i]
        if isinstance(m, nn.Flatten):
            blocks.append(to_lava_block_flatten(m))
            i += 1
            continue
        if not isinstance(m, (nn.Linear, nn.Conv2d, nn.AvgPool2d)) or i + 1 >= len(net) or not isinstance(net[i + 1], spiking):
            raise ValueError(type(m))
        if isinstance(m, (nn.Linear, nn.Conv2d)) and pending_div is not None:
            m.weight.data /= pending_div
            pending_div = None
        if isinstance(m, nn.Linear):
            blocks.append(to_lava_block_dense(m, net[i + 1]))
        elif isinstance(m, nn.Conv2d):
            blocks.append(to_lava_block_conv(m, net[i + 1]))
        else:
            blocks.append(to_lava_block_pool(m, net[i + 1]))
            k = m.kernel_size
            pending_div = float(k * k) if isinstance(k, int) else float(k[0] * k[1])
        i += 2
    return blocks


class SumPool2d(nn.Module):
    """Sum over the pooling window (what a slayer pool computes)."""

    def __init__(self, kernel_size, stride=None, padding=0, dilation=1):
        super().__init__()
        probe = nn.Conv2d(1, 1, kernel_size=kernel_size, stride=stride if stride is not None else kernel_size, padding=padding,
                          dilation=dilation, bias=False)
        self.kernel_size, self.stride, self.padding, self.dilation = probe.kernel_size, probe.stride, probe.padding, probe.dilation
        self.register_buffer("weight", torch.ones_like(probe.weight.data), persistent=False)

    def forward(self, x: torch.Tensor):
        if self.dilation == (1, 1):
            return F.avg_pool2d(x, self.kernel_size, self.stride, self.padding) * self.weight.numel()
        N, C, H, W = x.shape
        y = F.conv2d(x.reshape(N * C, 1, H, W), self.weight.to(x), None, self.stride, self.padding, self.dilation)
        return y.view(N, C, y.shape[2], y.shape[3])


class BlockContainer(nn.Module, base.StepModule):
    """A synapse (Linear / Conv2d without bias, ``SumPool2d``, Flatten) followed by a :class:`CubaLIFNode`, computing with
    8-bit quantised weights in the forward pass — train here, then ``to_lava_block()``."""

    def __init__(self, synapse: Union[nn.Conv2d, nn.Linear, nn.AvgPool2d, nn.Flatten], neu: Optional[CubaLIFNode], step_mode: str = "s"):
        super().__init__()
        if isinstance(synapse, nn.Flatten):
            if neu is not None:
                raise AssertionError("a Flatten block has no neuron")
            if synapse.start_dim != 1:
                raise ValueError("lava only supports for torch.nn.Flatten with start_dim == 1!")
        else:
            if isinstance(neu, (neuron.IFNode, neuron.LIFNode)) and not isinstance(neu, CubaLIFNode):
                p = to_lava_neuron_param_dict(neu)
                neu = CubaLIFNode(current_decay=1.0, voltage_decay=p["voltage_decay"], v_threshold=neu.v_threshold, scale=neu.lava_s_cale)
            elif not isinstance(neu, CubaLIFNode):
                raise AssertionError("expected an IFNode, a LIFNode or a CubaLIFNode")
            if isinstance(synapse, (nn.Conv2d, nn.Linear)) and synapse.bias is not None:
                raise AssertionError("synapses must not have a bias")
        self.synapse, self.neuron = synapse, neu
        self.step_mode = step_mode

    @property
    def step_mode(self):
        return self._step_mode

    @step_mode.setter
    def step_mode(self, value: str):
        if value not in self.supported_step_mode():
            raise ValueError(f'step_mode can only be {self.supported_step_mode()}, but got "{value}"!')
        self._step_mode = value
        for m in (self.neuron, self.synapse):
            if isinstance(m, base.StepModule):
                m.step_mode = value

    def forward(self, x: torch.Tensor):
        multi = self.step_mode == "m"
        if multi:
            T, N = x.shape[0], x.shape[1]
            x = x.flatten(0, 1)
        s = self.synapse
        if isinstance(s, nn.Conv2d):
            x = F.conv2d(x, self.neuron.quantize_8bit(s.weight), s.bias, s.stride, s.padding, s.dilation, s.groups)
        elif isinstance(s, nn.Linear):
            x = F.linear(x, self.neuron.quantize_8bit(s.weight), s.bias)
        elif isinstance(s, (SumPool2d, nn.Flatten)):
            x = s(x)
        else:
            raise NotImplementedError(type(s))
        if multi:
            x = x.view([T, N, *x.shape[1:]])
        return x if self.neuron is None else self.neuron(x)

    def to_lava_block(self):
        sl = _need_lava()
        s = self.synapse
        if isinstance(s, nn.Flatten):
            return sl.block.cuba.Flatten()
        params = self.neuron.lava_cuba_neuron_params
        if isinstance(s, nn.Linear):
            block = sl.block.cuba.Dense(params, s.in_features, s.out_features, delay_shift=False)
            block.synapse.weight.data[:, :, 0, 0, 0] = s.weight.data.clone()
        elif isinstance(s, nn.Conv2d):
            block = sl.block.cuba.Conv(params, **_conv_kwargs(s), delay_shift=False)
            block.synapse.weight.data[:, :, :, :, 0] = s.weight.data.clone()
        elif isinstance(s, SumPool2d):
            block = sl.block.cuba.Pool(params, s.kernel_size, s.stride, s.padding, s.dilation, delay_shift=False)
        else:
            raise NotImplementedError(type(s))
        if self.neuron.norm is not None:
            block.neuron.norm = self.neuron.norm.to_lava()
        return block
