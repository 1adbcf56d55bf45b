"""Which surrogate gradients the kernel back end evaluates on the device, under the reference's names
(``triton_kernel/surrogate_kernel.py:17-160``).  ``SG_TRITON_IDS`` keeps the reference's numbering of the seven surrogates
its Triton kernels know; ``resolve_sg_triton_id_and_alpha`` answers with that id and the slope.  The CUDA kernels of this
package are driven by ``surrogate.surrogate_spec`` instead, which covers every table-driven surrogate (``kernel_id_and_params``
returns that descriptor); ``sg_triton`` evaluates the same derivative on tensors."""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from .. import surrogate

__all__ = ["sg_triton", "SG_TRITON_IDS", "resolve_sg_triton_id_and_alpha", "kernel_id_and_params"]

SG_TRITON_IDS: Dict[type, int] = {surrogate.Sigmoid: 0, surrogate.ATan: 1, surrogate.PiecewiseQuadratic: 2, surrogate.PiecewiseExp: 3,
                                  surrogate.SoftSign: 4, surrogate.SuperSpike: 5, surrogate.Erf: 6}


def resolve_sg_triton_id_and_alpha(surrogate_function) -> Tuple[int, float]:
    for cls, sid in SG_TRITON_IDS.items():
        if isinstance(surrogate_function, cls):
            break
    else:
        raise NotImplementedError(f"Triton backend only supports surrogate functions {tuple(c.__name__ for c in SG_TRITON_IDS)}, "
                                  f"but got {type(surrogate_function).__name__}. Use backend='torch' for other surrogate functions.")
    if not hasattr(surrogate_function, "alpha"):
        raise TypeError(f"Triton backend requires surrogate_function.alpha, but got {type(surrogate_function).__name__} without 'alpha'.")
    alpha = surrogate_function.alpha
    if isinstance(alpha, torch.Tensor):
        if alpha.numel() != 1:
            raise TypeError(f"surrogate_function.alpha must be a scalar for Triton backend, but got tensor with shape={tuple(alpha.shape)}.")
        alpha = alpha.item()
    if isinstance(alpha, bool) or not isinstance(alpha, (int, float)):
        raise TypeError(f"surrogate_function.alpha must be a real scalar for Triton backend, but got {type(alpha).__name__}.")
    return sid, float(alpha)


def kernel_id_and_params(surrogate_function) -> Tuple[int, float, float]:
    """``(id, p0, p1)`` as the CUDA scan kernels and the FlexSN generator take it."""
    spec = surrogate.surrogate_spec(surrogate_function)
    if spec is None:
        raise NotImplementedError(f"{type(surrogate_function).__name__} has no kernel descriptor; it runs through PyTorch.")
    return spec


_BY_ID = {sid: cls for cls, sid in SG_TRITON_IDS.items()}


def sg_triton(h: torch.Tensor, alpha: float, sg_triton_id: int) -> torch.Tensor:
    """Derivative of surrogate number ``sg_triton_id`` (reference numbering) with slope ``alpha`` at ``h``."""
    if sg_triton_id not in _BY_ID:
        raise ValueError(f"unknown surrogate id {sg_triton_id}")
    sg = _BY_ID[sg_triton_id](alpha=float(alpha))
    x = h.detach().clone().requires_grad_(True)
    with torch.enable_grad():
        (g,) = torch.autograd.grad(sg(x).sum(), x)
    return g
