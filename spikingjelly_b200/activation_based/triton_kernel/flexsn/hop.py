"""Scan entry points under the reference's names (``triton_kernel/flexsn/hop.py``).  The reference offers several ways to hand a
Python time loop to ``torch.compile`` (a higher-order operator, ``scan`` and ``while_loop`` lowerings); this package compiles
the loop itself into a CUDA kernel, so the lowering probes answer ``False`` and every scan function runs the eager loop,
which is also what the FlexSN module falls back to on the CPU."""
from __future__ import annotations

from typing import Callable, Tuple, Union

import torch

from ...neuron.flexsn import eager_scan as _eager_scan

__all__ = ["FlexSNScan", "lowerable_scan_available", "dynamo_hop_available", "lowerable_while_loop_available", "eager_scan",
           "eager_scan_final_state", "lowerable_scan", "lowerable_scan_final_state", "lowerable_while_loop_scan",
           "lowerable_while_loop_scan_final_state"]


def lowerable_scan_available() -> bool:
    return False


def dynamo_hop_available() -> bool:
    return False


def lowerable_while_loop_available() -> bool:
    return False


def eager_scan(core_fn: Callable, num_inputs: int, num_states: int, num_outputs: int, *flat_args: torch.Tensor,
               output_template_specs=None) -> Tuple[torch.Tensor, ...]:
    """``(*output sequences, *state sequences)`` for ``flat_args = (*input sequences, *initial states)``."""
    return tuple(_eager_scan(core_fn, num_inputs, num_states, num_outputs, True, *flat_args))


def eager_scan_final_state(core_fn: Callable, num_inputs: int, num_states: int, num_outputs: int, *flat_args: torch.Tensor,
                           output_template_specs=None) -> Tuple[torch.Tensor, ...]:
    """``(*output sequences, *final states)``."""
    return tuple(_eager_scan(core_fn, num_inputs, num_states, num_outputs, False, *flat_args))


lowerable_scan = lowerable_while_loop_scan = eager_scan
lowerable_scan_final_state = lowerable_while_loop_scan_final_state = eager_scan_final_state


class FlexSNScan:
    """Callable with the higher-order operator's calling convention: ``FlexSNScan()(core_fn, ni, ns, no, *flat_args)``."""

    def __call__(self, core_fn: Callable, num_inputs: int, num_states: int, num_outputs: int, *flat_args, final_state_only: bool = False):
        return (eager_scan_final_state if final_state_only else eager_scan)(core_fn, num_inputs, num_states, num_outputs, *flat_args)


flex_sn_scan = FlexSNScan()
#: ``(shape, dtype)`` or ``(shape, dtype, device)`` of one output of a step, used to build empty outputs for ``T = 0``
OutputTemplateSpec = Union[Tuple[Tuple[int, ...], torch.dtype], Tuple[Tuple[int, ...], torch.dtype, torch.device]]
OutputTemplateSpecs = Tuple[OutputTemplateSpec, ...]
