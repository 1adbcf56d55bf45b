"""``import_from_nir``: ``nir.NIRGraph`` (or a path to one) -> ``torch.fx.GraphModule`` of this framework's layers and
neurons (``spikingjelly/activation_based/nir_exchange/from_nir.py:151-237``)."""
from __future__ import annotations

from typing import Union

import torch

from ...logger import logger
from .. import functional
from ._spec import spec_to_module

__all__ = ["import_from_nir"]

_KINDS = ("Affine", "Linear", "Conv2d", "AvgPool2d", "Flatten", "IF", "LIF")
_FIELDS = {"Affine": ("weight", "bias"), "Linear": ("weight",), "Conv2d": ("weight", "bias", "stride", "padding", "dilation", "groups"),
           "AvgPool2d": ("kernel_size", "stride", "padding"), "Flatten": ("start_dim", "end_dim"), "IF": ("r", "v_threshold", "v_reset"),
           "LIF": ("tau", "r", "v_leak", "v_threshold", "v_reset")}


def import_from_nir(graph, dt: float = 1e-4, device: str = "cpu", dtype: torch.dtype = torch.float32, step_mode: str = "s"):
    try:
        import nir
        import nirtorch
    except ImportError as e:
        raise ImportError("NIR import needs the `nir` and `nirtorch` packages") from e

    def make(kind):
        return lambda node: spec_to_module(kind, {f: getattr(node, f) for f in _FIELDS[kind]}, dt)

    gm = nirtorch.nir_to_torch(graph, {getattr(nir, k): make(k) for k in _KINDS}, device=device, dtype=dtype)
    functional.set_step_mode(gm, step_mode)
    logger.info("nir_import_summary source=%s device=%s dtype=%s step_mode=%s", "path" if isinstance(graph, str) else type(graph).__name__,
                device, dtype, step_mode)
    return gm
