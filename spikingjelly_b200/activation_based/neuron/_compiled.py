"""Native multi-step execution for neurons that have no hand-written kernel: the node's own single-step rule is
captured as ATen graphs (forward and joint backward) and compiled by the FlexSN code generator into one CUDA kernel per
direction, with every state in registers across ``T``.  Hyper-parameters are constants of the generated code, so a
kernel is keyed by their values and rebuilt when one changes.  Used by Izhikevich, current-based LIF, integer LIF and
the ternary IF neuron (the reference has CuPy / Triton strings for these: ``cuda_kernel/neuron_kernel/izhikevich.py``,
``triton_kernel/neuron_kernel/{ilif,stbif}.py``)."""
from __future__ import annotations

import weakref
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ...logger import logger

__all__ = ["CompiledSequence", "compiled_for", "scalar_signature"]


class CompiledSequence:
    """``step(x, *states) -> (output, *new_states)``; all tensors share one shape.  ``run`` returns
    ``(output sequence, final states, state sequences or None)`` or ``None`` when the rule cannot be compiled (the caller
    then takes its eager path)."""

    def __init__(self, step: Callable, num_states: int, signature: Callable[[], tuple], name: str):
        self._step, self._ns, self._signature, self._name = step, num_states, signature, name
        self._kernels: Dict[tuple, Optional[int]] = {}

    def _handle(self) -> Optional[int]:
        from ...ops import flexsn as K
        key = self._signature()
        if key not in self._kernels:
            def core(x, *states):
                return self._step(x, *states)
            core.__name__ = self._name
            try:
                kernel = K.build_kernel(core, 1, self._ns, 1)
                self._kernels[key] = K.register_kernel_handle(kernel)
            except (K.UnsupportedCore, K.CompileError, RuntimeError, TypeError, ValueError) as e:
                logger.warning("%s: the step rule does not compile (%s: %s); using the eager loop.", self._name, type(e).__name__, e)
                self._kernels[key] = None
        return self._kernels[key]

    def run(self, x_seq: torch.Tensor, states: Sequence[torch.Tensor], want_state_seqs: bool = False):
        if not x_seq.is_cuda or x_seq.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            return None
        handle = self._handle()
        if handle is None:
            return None
        from ...ops import flexsn as K
        flat = [x_seq.contiguous(), *[s.to(x_seq.dtype).contiguous() for s in states]]
        if torch.is_grad_enabled() and any(t.requires_grad for t in flat):
            outs, seqs, last = K.flexsn_training(handle, flat)
        else:
            outs, seqs, last = K.flexsn_forward(handle, flat, want_state_seqs)
        return outs[0], list(last), (list(seqs) if seqs is not None else None)


_REGISTRY: "weakref.WeakKeyDictionary" = weakref.WeakKeyDictionary()


def compiled_for(module, make: Callable[[], CompiledSequence]) -> CompiledSequence:
    """One :class:`CompiledSequence` per module object, kept outside the module (so that ``deepcopy`` / pickling of the
    module never drags a closure over the original along)."""
    seq = _REGISTRY.get(module)
    if seq is None:
        seq = _REGISTRY[module] = make()
    return seq


def scalar_signature(module, extra: Tuple = ()) -> tuple:
    """Every int / float / bool / None attribute of ``module``, its surrogate's description and the training flag."""
    items = tuple(sorted((k, v) for k, v in vars(module).items() if isinstance(v, (int, float, bool)) or v is None))
    sg = getattr(module, "surrogate_function", None)
    sg_items = tuple(sorted((k, v) for k, v in vars(sg).items() if isinstance(v, (int, float, bool, str)))) if hasattr(sg, "__dict__") else ()
    return (type(module).__name__, items, type(sg).__name__, sg_items, bool(module.training), *extra)
