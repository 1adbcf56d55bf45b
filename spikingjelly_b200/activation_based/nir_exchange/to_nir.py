"""``export_to_nir``: trace the network (``nirtorch``), record every supported module's input/output shape with FX shape
propagation and emit a ``nir.NIRGraph`` (``spikingjelly/activation_based/nir_exchange/to_nir.py:225-307``)."""
from __future__ import annotations

from pathlib import Path
from typing import Optional, Union

import torch
import torch.nn as nn

from ...logger import logger
from ._spec import SUPPORTED_MODULES, module_to_spec

__all__ = ["export_to_nir"]


def _require():
    try:
        import nir
        import nirtorch
    except ImportError as e:
        raise ImportError("NIR export needs the `nir` and `nirtorch` packages") from e
    return nir, nirtorch


def _module_io_shapes(net: nn.Module, example_input: torch.Tensor, nirtorch) -> dict:
    from torch import fx
    from torch.fx.passes.shape_prop import ShapeProp
    tracer = nirtorch.torch_tracer.NIRTorchTracer(SUPPORTED_MODULES)
    gm = fx.GraphModule(tracer.root if hasattr(tracer, "root") else net, tracer.trace(net))
    ShapeProp(gm).propagate(example_input)
    shapes = {}
    for node in gm.graph.nodes:
        if node.op != "call_module" or "tensor_meta" not in node.meta:
            continue
        ins = [n.meta["tensor_meta"].shape for n in node.all_input_nodes if "tensor_meta" in n.meta]
        shapes[gm.get_submodule(node.target)] = (ins[0], node.meta["tensor_meta"].shape)
    return shapes


def export_to_nir(net: nn.Module, example_input: torch.Tensor, save_path: Optional[Union[str, Path]] = None, dt: float = 1e-4):
    nir, nirtorch = _require()
    shapes = _module_io_shapes(net, example_input, nirtorch)

    def convert(module):
        kind, params = module_to_spec(module, *shapes[module], dt)
        return getattr(nir, kind)(**params)

    graph = nirtorch.torch_to_nir(net, {cls: convert for cls in SUPPORTED_MODULES}, type_check=True)
    if save_path is not None:
        nir.write(save_path, graph)
    logger.info("nir_export_summary model=%s dt=%s save_path=%s", type(net).__name__, dt, save_path)
    return graph
