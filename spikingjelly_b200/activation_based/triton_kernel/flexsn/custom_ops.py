"""Integer handles for compiled step functions and the operators that take them, under the reference's names
(``triton_kernel/flexsn/custom_ops.py:89-1130``).  A handle lets a compiled kernel (a Python object) travel through an operator
schema as an ``int``; the registry and the operators (``sjb200_flexsn::forward`` / ``::backward``, with fake implementations for
tracers) live in ``ops/flexsn/runtime.py``.  The reference keeps two reference counts per handle (owners and calls in
flight); here a call in flight holds the kernel object itself, so one count is enough and the ``*_active_*`` functions are
the same operations as the owner ones."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ....ops.flexsn import runtime as _rt
from .info import FlexSNInfo

__all__ = ["FlexSNKernelHandle", "register_flexsn_kernel_handle", "retain_flexsn_kernel_handle", "retain_owner_flexsn_kernel_handle",
           "release_flexsn_kernel_handle", "release_active_flexsn_kernel_handle", "flexsn_kernel_registry_info",
           "flexsn_inductor_inference", "flexsn_inductor_inference_final_state", "flexsn_inductor_training",
           "flexsn_inductor_training_final_state", "flexsn_inductor_backward", "attach_flexsn_handle_finalizer"]


@dataclass
class FlexSNKernelHandle:
    """What one handle stands for, in the reference's field layout: every kernel field names the same compiled object."""
    inference_kernel: Optional[object]
    inference_info: Optional[FlexSNInfo]
    inference_final_state_kernel: Optional[object]
    inference_final_state_info: Optional[FlexSNInfo]
    forward_kernel: Optional[object]
    backward_kernel: Optional[object]
    training_info: Optional[FlexSNInfo]
    owner_refs: int = 1
    active_refs: int = 0


def register_flexsn_kernel_handle(*, inference_kernel=None, inference_info=None, inference_final_state_kernel=None,
                                  inference_final_state_info=None, forward_kernel=None, backward_kernel=None, training_info=None) -> int:
    """Registers the first compiled object among the arguments (training kernels win: they can also run gradient-free)."""
    kernel = next((k for k in (forward_kernel, backward_kernel, inference_kernel, inference_final_state_kernel) if k is not None), None)
    if not isinstance(kernel, _rt.FlexSNKernel):
        raise TypeError("expected a compiled FlexSNKernel (see triton_kernel.flexsn.kernel.build_*)")
    return _rt.register_kernel_handle(kernel)


def _handle(handle) -> int:
    if isinstance(handle, torch.Tensor):
        if handle.numel() != 1:
            raise ValueError("a kernel handle tensor must hold one integer")
        handle = handle.item()
    if isinstance(handle, bool) or not isinstance(handle, int):
        raise TypeError(f"a kernel handle is an int, got {type(handle).__name__}")
    return handle


def retain_flexsn_kernel_handle(handle) -> None:
    _rt.lookup_kernel_handle(_handle(handle))          # raises KeyError for an unknown handle
    _rt.retain_kernel_handle(_handle(handle))


def release_flexsn_kernel_handle(handle) -> None:
    _rt.release_kernel_handle(_handle(handle))


retain_owner_flexsn_kernel_handle = retain_flexsn_kernel_handle
release_active_flexsn_kernel_handle = release_flexsn_kernel_handle
attach_flexsn_handle_finalizer = _rt.attach_handle_finalizer


def flexsn_kernel_registry_info() -> Dict[str, int]:
    with _rt._registry_lock:
        return {"entries": len(_rt._registry), "owner_refs": sum(e[1] for e in _rt._registry.values()), "active_refs": 0}


def flexsn_inductor_inference(handle: int, flat_args: List[torch.Tensor]) -> List[torch.Tensor]:
    """``[*output sequences, *state sequences]``."""
    outs, seqs, _ = _rt.flexsn_forward(_handle(handle), list(flat_args), True)
    return [*outs, *seqs]


def flexsn_inductor_inference_final_state(handle: int, flat_args: List[torch.Tensor]) -> List[torch.Tensor]:
    """``[*output sequences, *final states]``."""
    outs, _, last = _rt.flexsn_forward(_handle(handle), list(flat_args), False)
    return [*outs, *last]


def flexsn_inductor_training(handle: int, flat_args: List[torch.Tensor]) -> List[torch.Tensor]:
    """Differentiable: ``[*output sequences, *state sequences]``."""
    outs, seqs, _ = _rt.flexsn_training(_handle(handle), list(flat_args))
    return [*outs, *seqs]


def flexsn_inductor_training_final_state(handle: int, flat_args: List[torch.Tensor]) -> List[torch.Tensor]:
    """Differentiable: ``[*output sequences, *final states]`` (the state sequences are still kept for backward)."""
    outs, _, last = _rt.flexsn_training(_handle(handle), list(flat_args))
    return [*outs, *last]


def flexsn_inductor_backward(handle: int, grad_outputs: List[Optional[torch.Tensor]], saved_tensors: List[torch.Tensor],
                             input_templates: Optional[List[torch.Tensor]] = None) -> List[torch.Tensor]:
    """``saved_tensors = [*input sequences, *initial states, *state sequences]``, ``grad_outputs`` the gradients of the output
    and state sequences; returns ``[*grad inputs, *grad initial states]``."""
    k = _rt.lookup_kernel_handle(_handle(handle))
    n = k.NI + k.NS
    args, seqs = list(saved_tensors[:n]), list(saved_tensors[n:])
    grads = [*grad_outputs, *([None] * (k.NO + 2 * k.NS - len(grad_outputs)))]
    res = k.backward(args[:k.NI], args[k.NI:], seqs, grads[:k.NO], grads[k.NO:k.NO + k.NS], grads[k.NO + k.NS:], list(k.graphs.needs_grad))
    return [r if r is not None else torch.zeros_like(a) for r, a in zip(res, args)]
