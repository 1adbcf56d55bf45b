"""Export to Lynxi (KA200 / HP series) brain-inspired chips: stateless re-statements of IF / LIF whose multi-step
mode takes the time axis folded into the batch (the chip compiler traces plain tensors), a module rewriter that maps
this framework's stateful layers to compiler-friendly ``torch.nn`` ones, and thin wrappers around the vendor runtime
(``lyngor`` / ``lynpy``) that exist when those packages do (``spikingjelly/activation_based/lynxi_exchange.py:22-849``).
"""
from __future__ import annotations

import copy
import os
from typing import Dict, Optional, Union

import torch
import torch.nn as nn

from ..logger import logger
from . import layer, neuron

__all__ = ["BaseNode", "IFNode", "LIFNode", "to_lynxi_supported_module", "to_lynxi_supported_modules",
           "torch_tensor_to_lynxi", "lynxi_tensor_to_torch", "compile_lynxi_model", "load_lynxi_model"]


class BaseNode(nn.Module):
    """No hidden state: the membrane potential goes in and (optionally) comes out.  In multi-step mode the input is
    ``[T * N, ...]`` (time-major) and ``T`` is fixed at construction, because the compiled graph is static."""

    def __init__(self, v_threshold: float = 1.0, v_reset: Optional[float] = 0.0, step_mode="s", T: int = None, return_v: bool = False):
        super().__init__()
        self.v_threshold, self.v_reset, self.step_mode, self.T, self.return_v = v_threshold, v_reset, step_mode, T, return_v

    def neuronal_charge(self, x: torch.Tensor, v: torch.Tensor):
        raise NotImplementedError

    def single_step_forward(self, x: torch.Tensor, v: torch.Tensor = None):
        v = self.neuronal_charge(x, torch.zeros_like(x) if v is None else v)
        spike = (v >= self.v_threshold).to(x)
        v = v - spike * self.v_threshold if self.v_reset is None else (1.0 - spike) * v + spike * self.v_reset
        return spike, v

    def multi_step_forward(self, x_seq: torch.Tensor, v_init: torch.Tensor = None):
        v = torch.zeros_like(x_seq[0]) if v_init is None else v_init
        spikes = []
        for t in range(self.T):
            s, v = self.single_step_forward(x_seq[t], v)
            spikes.append(s.unsqueeze(0))
        return torch.cat(spikes), v

    def forward(self, x: torch.Tensor, v: torch.Tensor = None):
        if self.step_mode == "s":
            spike, v = self.single_step_forward(x, v)
            return (spike, v) if self.return_v else spike
        if self.step_mode == "m":
            shape = x.shape
            spikes, v = self.multi_step_forward(x.reshape(self.T, shape[0] // self.T, -1), None if v is None else v.flatten())
            spikes = spikes.flatten(0, 1).reshape(shape)
            return (spikes, v.reshape([shape[0] // self.T, *shape[1:]])) if self.return_v else spikes
        raise ValueError(self.step_mode)


class IFNode(BaseNode):
    def neuronal_charge(self, x: torch.Tensor, v: torch.Tensor):
        return x + v


class LIFNode(BaseNode):
    def __init__(self, tau: float = 2.0, decay_input: bool = True, v_threshold: float = 1.0, v_reset: Optional[float] = 0.0,
                 step_mode="s", T: int = None, return_v: bool = False):
        super().__init__(v_threshold, v_reset, step_mode, T, return_v)
        self.decay, self.decay_input = 1.0 / tau, decay_input

    def neuronal_charge(self, x: torch.Tensor, v: torch.Tensor):
        v = (1.0 - self.decay) * (v if self.v_reset is None else v - self.v_reset)
        return v + (x * self.decay if self.decay_input else x)


def to_lynxi_supported_module(m_in: nn.Module, T: int):
    """Stateful / step-mode-aware layer -> plain ``torch.nn`` layer with the same parameters; IF / LIF nodes -> the
    stateless nodes above.  Anything else is deep-copied to the CPU unchanged (and reported)."""
    if isinstance(m_in, layer.Conv2d):
        m_out = nn.Conv2d(m_in.in_channels, m_in.out_channels, m_in.kernel_size, m_in.stride, m_in.padding, m_in.dilation,
                          m_in.groups, m_in.bias is not None, m_in.padding_mode)
        m_out.load_state_dict(m_in.state_dict())
    elif isinstance(m_in, layer.BatchNorm2d):
        m_out = nn.BatchNorm2d(m_in.num_features, m_in.eps, m_in.momentum, m_in.affine, m_in.affine)
        m_out.load_state_dict(m_in.state_dict())
    elif isinstance(m_in, layer.MaxPool2d):
        m_out = nn.MaxPool2d(m_in.kernel_size, m_in.stride, m_in.padding, m_in.dilation, m_in.return_indices, m_in.ceil_mode)
    elif isinstance(m_in, layer.AvgPool2d):
        m_out = nn.AvgPool2d(m_in.kernel_size, m_in.stride, m_in.padding, m_in.ceil_mode, m_in.count_include_pad, m_in.divisor_override)
    elif isinstance(m_in, layer.AdaptiveAvgPool2d):
        m_out = nn.AdaptiveAvgPool2d(m_in.output_size)
    elif isinstance(m_in, layer.Flatten):
        m_out = nn.Flatten(m_in.start_dim, m_in.end_dim)
    elif isinstance(m_in, neuron.LIFNode):
        m_out = LIFNode(m_in.tau, m_in.decay_input, m_in.v_threshold, m_in.v_reset, m_in.step_mode, T, False)
    elif isinstance(m_in, neuron.IFNode):
        m_out = IFNode(m_in.v_threshold, m_in.v_reset, m_in.step_mode, T, False)
    else:
        logger.critical("%s is not processed and the origin module is used for lynxi compiling.", type(m_in))
        m_out = copy.deepcopy(m_in).cpu()
    return m_out


def to_lynxi_supported_modules(net: Union[list, tuple, nn.Sequential], T: int):
    return [to_lynxi_supported_module(m, T) for m in net]


def _vendor():
    try:
        import lyngor
        import lynpy
    except (ImportError, OSError) as e:
        raise ImportError("the Lynxi runtime (`lyngor`, `lynpy`) is not installed") from e
    return lyngor, lynpy


def torch_tensor_to_lynxi(x: torch.Tensor, device_id: int = 0, to_apu: bool = True):
    _, lynpy = _vendor()
    t = lynpy.Tensor(dev_id=device_id, size=x.element_size() * x.numel()).from_numpy(x.cpu().detach().numpy())
    return t.apu() if to_apu else t


def lynxi_tensor_to_torch(x, shape: Union[tuple, list] = None, dtype: str = None):
    if shape is not None and dtype is not None:
        x = x.view_as(shape, dtype)
    if x.devptr is not None:
        x = x.cpu()
    return torch.from_numpy(x.numpy())


def compile_lynxi_model(output_dir: str, net: nn.Module, in_data_type: str = "float32", out_data_type: str = "float32",
                        input_shape_dict: Dict = {}):
    lyngor, _ = _vendor()
    model = lyngor.DLModel()
    model.load(net, model_type="Pytorch", in_type=in_data_type, out_type=out_data_type, inputs_dict=input_shape_dict)
    out_path = lyngor.Builder(target="apu", is_map=True).build(model.graph, model.params, out_path=output_dir, apu_only=True)
    logger.info("Lynxi model artifacts generated at %s", out_path)
    return os.path.join(out_path, "Net_0")


def load_lynxi_model(device_id: int, model_path: str):
    _, lynpy = _vendor()
    return lynpy.Model(dev_id=device_id, path=model_path)
