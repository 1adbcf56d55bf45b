"""Launch wrappers under the reference's names (``triton_kernel/flexsn/wrapper.py:32-420``).  ``f`` is the compiled object a
builder of ``kernel.py`` returned, ``args`` the flat tuple ``(*input sequences, *initial states)``."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .info import FlexSNInfo

__all__ = ["flexsn_backward_ncl_bucket", "flexsn_inference", "flexsn_inference_final_state", "flexsn_forward", "flexsn_backward"]

_BUCKET_TOPS = (4096, 131072, 1048576, 8388608)


def flexsn_backward_ncl_bucket(ncl: int) -> int:
    """Size class 0..4 of a step's element count (the reference picks Triton launch configurations by it; the CUDA generator
    has one configuration, the classes are kept for reports)."""
    if ncl < 0:
        raise ValueError("ncl must be non-negative")
    return sum(ncl > top for top in _BUCKET_TOPS)


def _split(info: FlexSNInfo, args):
    return list(args[:info.num_inputs]), list(args[info.num_inputs:info.num_inputs + info.num_states])


def flexsn_inference(f, info: FlexSNInfo, *args) -> tuple:
    """``(*output sequences, *state sequences)``."""
    inputs, states = _split(info, args)
    with torch.no_grad():
        outs, seqs, _ = f.forward(inputs, states, True)
    return (*outs, *seqs)


def flexsn_inference_final_state(f, info: FlexSNInfo, *args) -> tuple:
    """``(*output sequences, *final states)``: no state sequence is written."""
    inputs, states = _split(info, args)
    with torch.no_grad():
        outs, _, last = f.forward(inputs, states, False)
    return (*outs, *last)


def flexsn_forward(f, info: FlexSNInfo, *args) -> tuple:
    """Training forward: ``(*output sequences, *state sequences)``; the state sequences are what backward needs."""
    return flexsn_inference(f, info, *args)


def flexsn_backward(f, info: FlexSNInfo, *args, input_templates: Optional[Tuple[torch.Tensor, ...]] = None,
                    state_templates: Optional[Tuple[torch.Tensor, ...]] = None) -> tuple:
    """``args = (*grad output sequences, *grad state sequences, *input sequences, *initial states, *state sequences)``
    -> ``(*grad input sequences, *grad initial states)``.  The saved tensors are the forward's arguments and its state
    sequences (no intermediates exist); the templates are not needed because the gradients take the shapes of the saved tensors."""
    ni, ns, no = info.num_inputs, info.num_states, info.num_outputs
    if len(args) != no + ns + ni + ns + ns:
        raise ValueError(f"expected {no + ns + ni + 2 * ns} tensors (grads of outputs and state sequences, inputs, initial states, state "
                         f"sequences), got {len(args)}")
    g_out, g_seq = list(args[:no]), list(args[no:no + ns])
    inputs, states, seqs = list(args[no + ns:no + ns + ni]), list(args[no + ns + ni:no + 2 * ns + ni]), list(args[no + 2 * ns + ni:])
    needs = list(f.graphs.needs_grad)
    res = f.backward(inputs, states, seqs, g_out, g_seq, [None] * ns, needs)
    return tuple(r if r is not None else torch.zeros_like(t) for r, t in zip(res, [*inputs, *states]))
