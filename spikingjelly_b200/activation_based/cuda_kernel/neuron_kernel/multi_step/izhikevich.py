"""Izhikevich neuron (membrane potential + adaptation variable) as one generated kernel per direction
(``cuda_kernel/neuron_kernel/multi_step/izhikevich.py`` of the reference): the step rule ``functional.izhikevich_step`` is compiled
by the FlexSN generator, one compiled object per parameter set."""
from __future__ import annotations

from typing import Callable, Dict, Optional, Tuple

import torch

from .... import functional

__all__ = ["izhikevich_multi_step", "cupy_multistep_izhikevich_forward"]

_COMPILED: Dict[tuple, object] = {}


def izhikevich_multi_step(x_seq: torch.Tensor, v_init: torch.Tensor, w_init: torch.Tensor, tau: float, v_threshold: float,
                          v_reset: Optional[float], v_rest: float, a: float, b: float, tau_w: float, v_c: float, a0: float,
                          detach_reset: bool, surrogate_function: Callable) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``(spike_seq, v_seq, w_seq)``."""
    from ....neuron._compiled import CompiledSequence
    key = (tau, v_threshold, v_reset, v_rest, a, b, tau_w, v_c, a0, bool(detach_reset), type(surrogate_function).__name__,
           tuple(sorted((k, v) for k, v in vars(surrogate_function).items() if isinstance(v, (int, float, bool)))))

    def step(x, v, w):
        return functional.neuron.izhikevich_step(x, v, w, tau, a0, v_rest, v_c, tau_w, a, b, v_threshold, v_reset, surrogate_function, detach_reset)
    if x_seq.is_cuda:
        seq = _COMPILED.get(key)
        if seq is None:
            seq = _COMPILED[key] = CompiledSequence(step, 2, lambda: key, "izhikevich")
        res = seq.run(x_seq, (v_init, w_init), want_state_seqs=True)
        if res is not None and res[2] is not None:
            return res[0], res[2][0], res[2][1]
    s, _, _, v_seq, w_seq = functional.neuron.izhikevich_multi_step_eager(x_seq, v_init, w_init, tau, v_threshold, v_reset, v_rest, v_c, a0, tau_w, a,
                                                                         b, surrogate_function, detach_reset, store_v_seq=True)
    return s, v_seq, w_seq


def cupy_multistep_izhikevich_forward(x_seq, v_init, w_init, tau, v_threshold, v_reset, v_rest, a, b, tau_w, v_c, a0, detach_reset,
                                      surrogate_function, capture_context=False):
    s, v_seq, w_seq = izhikevich_multi_step(x_seq, v_init, w_init, tau, v_threshold, v_reset, v_rest, a, b, tau_w, v_c, a0, detach_reset,
                                            surrogate_function)
    return s, v_seq, w_seq, None
