"""Parameter mapping between this framework's modules and NIR primitives, independent of the ``nir`` package: a node
is described as ``(kind, {field: numpy array or python value})`` and only wrapped into / read from ``nir`` classes at
the boundary.  Conventions (``spikingjelly/activation_based/nir_exchange/to_nir.py:80-222``):

* time constants are continuous: ``tau_nir = tau * dt``; an IF neuron has ``r = 1 / dt``;
* ``LIF.r = 1`` when the input is decayed with the membrane (``decay_input=True``), else ``r = tau``;
* ``v_leak = v_reset`` (0 for soft reset); soft reset itself is not representable and exports as reset to 0;
* shapes drop the batch (and time) dimensions; ``Flatten`` dims shift by one for the same reason.
"""
from __future__ import annotations

from typing import Dict, Sequence, Tuple

import numpy as np
import torch
import torch.nn as nn

from .. import layer, neuron

__all__ = ["module_to_spec", "spec_to_module", "SUPPORTED_MODULES"]

SUPPORTED_MODULES = (nn.Linear, layer.Linear, nn.Conv2d, layer.Conv2d, nn.AvgPool2d, layer.AvgPool2d, nn.Flatten, layer.Flatten,
                     neuron.IFNode, neuron.LIFNode, neuron.ParametricLIFNode)


def _np(x: torch.Tensor) -> np.ndarray:
    return x.detach().cpu().numpy()


def _feature_shape(shape: Sequence[int], module) -> Tuple[int, ...]:
    return tuple(shape[2 if getattr(module, "step_mode", "s") == "m" else 1:])


def module_to_spec(module: nn.Module, input_shape: Sequence[int], output_shape: Sequence[int], dt: float) -> Tuple[str, Dict]:
    if isinstance(module, nn.Linear):
        if module.bias is None:
            return "Linear", {"weight": _np(module.weight)}
        return "Affine", {"weight": _np(module.weight), "bias": _np(module.bias)}
    if isinstance(module, nn.Conv2d):
        bias = np.zeros(module.weight.shape[0]) if module.bias is None else _np(module.bias)
        return "Conv2d", {"input_shape": tuple(input_shape[-2:]), "weight": _np(module.weight), "stride": module.stride,
                          "padding": module.padding, "dilation": module.dilation, "groups": module.groups, "bias": bias}
    if isinstance(module, nn.AvgPool2d):
        return "AvgPool2d", {"kernel_size": module.kernel_size, "stride": module.stride, "padding": module.padding}
    if isinstance(module, nn.Flatten):
        shift = lambda d: d - 1 if d > 0 else d
        return "Flatten", {"input_type": _feature_shape(input_shape, module), "start_dim": shift(module.start_dim), "end_dim": shift(module.end_dim)}
    if isinstance(module, (neuron.IFNode, neuron.LIFNode, neuron.ParametricLIFNode)):
        in_t, out_t = _feature_shape(input_shape, module), _feature_shape(output_shape, module)
        reset = 0.0 if module.v_reset is None else module.v_reset
        common = {"v_threshold": np.full(in_t, module.v_threshold), "v_reset": np.full(in_t, reset), "input_type": in_t, "output_type": out_t}
        if isinstance(module, neuron.IFNode):
            return "IF", {"r": np.full(in_t, 1 / dt), **common}
        tau = float(1.0 / module.w.detach().sigmoid()) if isinstance(module, neuron.ParametricLIFNode) else module.tau
        return "LIF", {"tau": np.full(in_t, tau * dt), "r": np.full(in_t, 1.0 if module.decay_input else tau), "v_leak": np.full(in_t, reset), **common}
    raise NotImplementedError(f"{type(module).__name__} has no NIR counterpart")


def _scalar(a, what: str):
    u = np.unique(np.asarray(a))
    if u.size != 1:
        raise AssertionError(f"`{what}` must be the same for all neurons!")
    v = u[0]
    return int(v) if isinstance(v, (int, np.integer)) else float(v)


def _tuple(x):
    if isinstance(x, (int, np.integer)):
        return int(x)
    if isinstance(x, (float, np.floating)):
        return float(x)
    return tuple(np.asarray(x).tolist())


def spec_to_module(kind: str, p: Dict, dt: float) -> nn.Module:
    """Single-step module for one NIR node."""
    if kind in ("Affine", "Linear"):
        w = np.asarray(p["weight"])
        m = layer.Linear(w.shape[-1], w.shape[-2], bias=kind == "Affine")
        m.weight.data = torch.from_numpy(w.copy())
        if kind == "Affine":
            m.bias.data = torch.from_numpy(np.asarray(p["bias"]).copy())
        return m
    if kind == "Conv2d":
        w = np.asarray(p["weight"])
        # weight is [out, in / groups, kh, kw]
        m = layer.Conv2d(w.shape[-3] * _tuple(p["groups"]), w.shape[-4], tuple(w.shape[-2:]),
                         stride=_tuple(p["stride"]), padding=_tuple(p["padding"]), dilation=_tuple(p["dilation"]), groups=_tuple(p["groups"]), bias=True)
        m.weight.data = torch.from_numpy(w.copy())
        m.bias.data = torch.from_numpy(np.asarray(p["bias"]).copy())
        return m
    if kind == "AvgPool2d":
        return layer.AvgPool2d(kernel_size=_tuple(p["kernel_size"]), stride=_tuple(p["stride"]), padding=_tuple(p["padding"]))
    if kind == "Flatten":
        shift = lambda d: d + 1 if d >= 0 else d
        return layer.Flatten(shift(p["start_dim"]), shift(p["end_dim"]))
    if kind == "IF":
        if not np.allclose(np.unique(p["r"]), 1.0 / dt):
            raise AssertionError("`nir.IF.r` mismatch 1.0/dt !")
        return neuron.IFNode(v_threshold=_scalar(p["v_threshold"], "v_threshold"), v_reset=_scalar(p["v_reset"], "v_reset"))
    if kind == "LIF":
        tau = _scalar(p["tau"], "tau") / dt
        r = _scalar(p["r"], "r")
        v_reset, v_leak = _scalar(p["v_reset"], "v_reset"), _scalar(p["v_leak"], "v_leak")
        if v_leak != v_reset:
            raise AssertionError("`v_leak` should be equal to `v_reset`!")
        decay_input = False if r == tau else r == 1.0
        return neuron.LIFNode(tau=tau, decay_input=decay_input, v_reset=v_reset, v_threshold=_scalar(p["v_threshold"], "v_threshold"))
    raise NotImplementedError(f"NIR node {kind} is not supported")
