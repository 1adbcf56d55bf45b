"""ATen-level FX graphs of a step function (``triton_kernel/torch2triton/torch2graph.py:17-260`` of the reference).

``generate_inference_graph(fn, example_inputs)`` returns the forward graph; ``generate_forward_and_backward_graph`` returns the
forward graph and the *joint* backward graph ``(*inputs, *cotangents) -> gradients`` that recomputes the forward inside (the
reference partitions into a forward graph with saved intermediates and a backward graph that consumes them; the kernels
generated here keep no intermediates).  Graphs are cleaned of no-op ``aten.detach`` / ``alias`` nodes (``GraphOptimizer``)."""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.fx as fx
from torch.fx.experimental.proxy_tensor import make_fx

__all__ = ["GraphCollector", "GraphOptimizer", "generate_inference_graph", "generate_forward_and_backward_graph"]

_NOOPS = ("detach", "alias", "lift_fresh", "lift_fresh_copy")


class GraphOptimizer(fx.Transformer):
    """Drops operators that only re-label a tensor."""

    def call_function(self, target, args, kwargs):
        packet = getattr(getattr(target, "overloadpacket", None), "__name__", None)
        if packet in _NOOPS and args:
            return args[0]
        return super().call_function(target, args, kwargs)


def _optimize(gm) -> fx.Graph:
    if isinstance(gm, fx.Graph):
        gm = fx.GraphModule(torch.nn.Module(), gm)
    out = GraphOptimizer(gm).transform()
    out.graph.eliminate_dead_code()
    return out.graph


class GraphCollector:
    """Collects the graphs handed to ``get_forward_compiler()`` / ``get_backward_compiler()`` (the callbacks have the
    signature AOT-autograd expects: ``(graph_module, example_inputs) -> callable``)."""

    def __init__(self):
        self.fwd_graph: Optional[fx.Graph] = None
        self.bwd_graph: Optional[fx.Graph] = None
        self.fwd_graphs: List[fx.Graph] = []
        self.bwd_graphs: List[fx.Graph] = []

    def _compiler(self, which: str):
        def compiler(gm: fx.GraphModule, example_inputs):
            getattr(self, which + "_graphs").append(gm.graph)
            setattr(self, which + "_graph", gm.graph)
            return gm.forward
        return compiler

    def get_forward_compiler(self):
        return self._compiler("fwd")

    def get_backward_compiler(self):
        return self._compiler("bwd")


def _as_tuple(res):
    return tuple(res) if isinstance(res, (tuple, list)) else (res,)


def generate_inference_graph(fn: Callable, example_inputs: tuple) -> fx.Graph:
    with torch.no_grad():
        gm = make_fx(lambda *a: _as_tuple(fn(*a)), tracing_mode="real")(*[e.detach() for e in example_inputs])
    return _optimize(gm)


def generate_forward_and_backward_graph(fn: Callable, example_inputs: tuple,
                                        requires_grad: Optional[Sequence[bool]] = None) -> Tuple[fx.Graph, fx.Graph]:
    n = len(example_inputs)
    needs = tuple(bool(r) for r in requires_grad) if requires_grad is not None else (True,) * n
    if len(needs) != n:
        raise ValueError(f"requires_grad must hold {n} flags")
    fwd = generate_inference_graph(fn, example_inputs)
    with torch.no_grad():
        outs = _as_tuple(fn(*example_inputs))

    def joint(*flat):
        args = [a.detach().requires_grad_(needs[i]) for i, a in enumerate(flat[:n])]
        with torch.enable_grad():
            res = _as_tuple(fn(*args))
            pairs = [(r, c) for r, c in zip(res, flat[n:]) if r.requires_grad]
            wanted = [a for a, k in zip(args, needs) if k]
            grads = torch.autograd.grad([r for r, _ in pairs], wanted, [c for _, c in pairs], allow_unused=True) if pairs and wanted else ()
        it = iter(grads)
        return tuple((lambda g, a: torch.zeros_like(a) if g is None else g)(next(it, None) if k else None, a) for a, k in zip(args, needs))
    cot = [torch.ones_like(o, dtype=o.dtype if o.is_floating_point() else torch.float32) for o in outs]
    bwd = make_fx(joint, tracing_mode="real")(*[e.detach() for e in example_inputs], *cot)
    return fwd, _optimize(bwd)
