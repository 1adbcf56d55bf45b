"""Delayed read-out for rate-coded networks: the first spikes of a deep network arrive after a
latency of roughly ``sum over layers of (charge needed for one spike) / (mean input per step)``.
``estimate_delay_start`` measures that on calibration data and returns the step at which to start
accumulating the output.  Parity: ``spikingjelly/activation_based/ann2snn/delay.py:21-302``."""
from __future__ import annotations

import math
import time
import warnings
from typing import Dict, Iterable, List, Tuple, Union

import torch
import torch.nn as nn
from torch import fx

from ...logger import logger
from ..functional.net_config import reset_net
from ..neuron.base_node import BaseNode
from .modules import ChannelVoltageScaler, VoltageScaler

__all__ = ["estimate_delay_start"]

Scaler = Union[VoltageScaler, ChannelVoltageScaler]
_MIN_READOUT_STEPS = 4


def _model_input(batch):
    if isinstance(batch, torch.Tensor):
        return batch
    if isinstance(batch, (tuple, list)) and batch:
        return batch[0]
    raise TypeError("estimate_delay_start supports dataloaders that yield a tensor or a non-empty tuple/list whose first element "
                    "is the model input.")


def _delay_ratio(module: BaseNode, post: Scaler, x: torch.Tensor) -> torch.Tensor:
    """steps a neuron needs before its first spike at the mean drive it sees, in ANN activation units"""
    th = torch.as_tensor(module.v_threshold, device=x.device, dtype=x.dtype)
    if th.numel() != 1:
        raise ValueError("Delay estimation requires scalar neuron v_threshold.")
    if not torch.isfinite(th).all() or (th <= 0).any():
        raise ValueError("Delay estimation requires finite positive v_threshold.")
    v0 = module.get_reset_value("v") if hasattr(module, "get_reset_value") else getattr(module, "v_reset", 0.0)
    v0 = torch.as_tensor(0.0 if v0 is None else v0, device=x.device, dtype=x.dtype)
    channel_dim = None
    scale = post.scale.to(x)
    if isinstance(post, ChannelVoltageScaler) and scale.dim() == 1:
        channel_dim = post.channel_dim % x.dim()
        shape = [1] * x.dim()
        shape[channel_dim] = scale.numel()
        scale = scale.reshape(shape)
    act = torch.clamp(x.detach(), min=0) * scale / th
    need = torch.clamp(th - v0, min=0) * scale / th
    if channel_dim is None:
        drive, charge = act.mean(), need.mean()
    else:
        dims = tuple(d for d in range(act.dim()) if d != channel_dim)
        drive, charge = act.mean(dim=dims).max(), need.expand_as(act).mean(dim=dims).max()
    return torch.zeros((), device=x.device, dtype=x.dtype) if drive <= 0 else (charge / drive).detach()


def _scaler_neuron_scaler_paths(model: nn.Module) -> List[Tuple[BaseNode, Scaler]]:
    if not isinstance(model, fx.GraphModule):
        return []
    mods = dict(model.named_modules())
    out = []
    for node in model.graph.nodes:
        m = mods.get(node.target) if node.op == "call_module" else None
        if not isinstance(m, BaseNode) or len(node.args) != 1 or not isinstance(node.args[0], fx.Node):
            continue
        pre = node.args[0]
        if pre.op != "call_module" or not isinstance(mods.get(pre.target), (VoltageScaler, ChannelVoltageScaler)):
            continue
        posts = [mods[u.target] for u in node.users if u.op == "call_module" and isinstance(mods.get(u.target), (VoltageScaler, ChannelVoltageScaler))]
        if len(posts) == 1:
            out.append((m, posts[0]))
    return out


def estimate_delay_start(model: nn.Module, dataloader: Iterable, device, time_steps: int, num_batches: int = 1) -> int:
    """First step (0-based) from which the output of a rate-coded ``model`` should be accumulated;
    always leaves at least 4 read-out steps, 0 when the model has no ``scaler -> neuron -> scaler`` paths."""
    if time_steps <= 0:
        raise ValueError("time_steps must be positive.")
    if num_batches <= 0:
        raise ValueError("num_batches must be positive.")
    t0 = time.perf_counter()
    paths = _scaler_neuron_scaler_paths(model)
    if not paths:
        logger.info("ann2snn_delay_summary matched_paths=0 batches=0 raw_delay_start=0 delay_start=0 readout_clamped=False elapsed_ms=%.3f",
                    (time.perf_counter() - t0) * 1e3)
        return 0
    tensors = list(model.parameters()) + list(model.buffers())
    home = tensors[0].device if tensors else torch.device("cpu")
    flags = {m: m.training for m in model.modules()}
    ratios: Dict[BaseNode, List[float]] = {m: [] for m, _ in paths}
    handles, done = [], 0

    def make_hook(m, post):
        def hook(_m, inputs, _out):
            x = inputs[0]
            ratios[m].append(float(_delay_ratio(m, post, x)))
            return torch.clamp(x, min=0, max=float(torch.as_tensor(m.v_threshold)))   # propagate the rate, not a spike
        return hook

    try:
        model.eval().to(device)
        handles = [m.register_forward_hook(make_hook(m, post)) for m, post in paths]
        with torch.no_grad():
            for i, batch in enumerate(dataloader):
                if i >= num_batches:
                    break
                reset_net(model)
                model(_model_input(batch).to(device))
                done += 1
        delay = sum(sum(v) / len(v) for v in ratios.values() if v)
        if not any(ratios.values()):
            warnings.warn("estimate_delay_start did not collect any delay ratios; no delayed readout will be applied.", RuntimeWarning, stacklevel=2)
    finally:
        for h in handles:
            h.remove()
        reset_net(model)
        model.to(home)
        for m, f in flags.items():
            m.training = f
    raw = math.ceil(delay) if math.isfinite(delay) else time_steps
    clamped = time_steps < raw + _MIN_READOUT_STEPS
    if clamped:
        warnings.warn(f"estimate_delay_start: time_steps is too small to keep {_MIN_READOUT_STEPS} readout steps after the estimated "
                      "delay; disabling delayed readout.", RuntimeWarning, stacklevel=2)
        result = max(time_steps - _MIN_READOUT_STEPS - 1, 0)
    else:
        result = min(raw, time_steps - 1)
    logger.info("ann2snn_delay_summary matched_paths=%s batches=%s raw_delay_start=%s delay_start=%s readout_clamped=%s elapsed_ms=%.3f",
                len(paths), done, raw, result, clamped, (time.perf_counter() - t0) * 1e3)
    return result
