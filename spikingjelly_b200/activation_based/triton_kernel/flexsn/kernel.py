"""Builders under the reference's names (``triton_kernel/flexsn/kernel.py:53-400``).  Each returns the compiled object(s) and a
``FlexSNInfo``; the inference builders compile the forward direction only."""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch

from .info import FlexSNInfo, extract_info

__all__ = ["build_inference_kernel", "build_inference_final_state_kernel", "build_training_kernels"]


def _build(core_fn, num_inputs, num_states, num_outputs, example_inputs, requires_grad, training):
    from ....ops import flexsn as K
    kernel = K.build_kernel(core_fn, num_inputs, num_states, num_outputs, example_inputs, requires_grad, training)
    return kernel, extract_info(kernel.graphs.forward.graph, num_inputs, num_states, num_outputs)


def build_inference_kernel(core_fn: Callable, num_inputs: int, num_states: int, num_outputs: int,
                           example_inputs: Optional[Tuple[torch.Tensor, ...]] = None):
    """``(kernel, info)``; run it with ``wrapper.flexsn_inference(kernel, info, *inputs, *states)``."""
    return _build(core_fn, num_inputs, num_states, num_outputs, example_inputs, None, False)


def build_inference_final_state_kernel(core_fn: Callable, num_inputs: int, num_states: int, num_outputs: int,
                                       example_inputs: Optional[Tuple[torch.Tensor, ...]] = None):
    """The same compiled object as :func:`build_inference_kernel`: whether state sequences are written is a launch argument."""
    return _build(core_fn, num_inputs, num_states, num_outputs, example_inputs, None, False)


def build_training_kernels(core_fn: Callable, num_inputs: int, num_states: int, num_outputs: int,
                           example_inputs: Optional[Tuple[torch.Tensor, ...]] = None, requires_grad: Optional[Tuple[bool, ...]] = None):
    """``(forward kernel, backward kernel, info)``: one object plays both parts."""
    kernel, info = _build(core_fn, num_inputs, num_states, num_outputs, example_inputs, requires_grad, True)
    return kernel, kernel, info
