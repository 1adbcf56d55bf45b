"""CUDA kernels for a neuron whose charge rule is an arithmetic Python function
(``cuda_kernel/auto_cuda/generator.py:11-953`` of the reference).

``custom_fun(x, v_last, *extra) -> h`` is traced with ``torch.fx``; only ``+ - * /`` and negation between its arguments
and Python numbers are understood.  From the trace come

* :func:`analyse_graph`       - the variables (inputs, intermediates, output) and the list of three-address commands;
* :func:`gen_forward_codes`   - a :class:`~.base.CKernel2D` that walks time forward: charge by the traced rule, fire at
  ``v_th``, hard or soft reset; it stores the spikes, the charged potentials ``h_seq`` (needed by backward) and the
  potentials ``v_v_seq``;
* :func:`gen_backward_codes`  - a reverse-time :class:`~.base.CKernel2D`: the derivatives of the traced rule with respect
  to ``x``, ``v_last`` and every extra tensor input are produced by differentiating the command list backwards
  (reverse-mode on the straight-line program), the surrogate gradient and the reset path follow the usual BPTT recurrence.

Both generators return kernel objects, not just text: ``kernel.full_codes`` is the source, ``kernel.simple_call(...)``
runs it.  Extra arguments: a ``torch.Tensor`` annotation makes a per-neuron ``[N]`` input, ``float`` a scalar.
"""
from __future__ import annotations

import hashlib
import inspect
import operator
from typing import Callable, Dict, List, Tuple

import torch
from torch import fx

from .base import CKernel2D

__all__ = ["hash_str", "VarNode", "analyse_graph", "gen_forward_codes", "gen_backward_codes"]

_BINARY = {operator.add: "+", operator.sub: "-", operator.mul: "*", operator.truediv: "/", torch.add: "+", torch.sub: "-", torch.mul: "*",
           torch.div: "/", torch.true_divide: "/"}
_METHODS = {"add": "+", "sub": "-", "mul": "*", "div": "/", "true_divide": "/", "__add__": "+", "__sub__": "-", "__mul__": "*", "__truediv__": "/"}


def hash_str(x: object) -> str:
    """Short stable hexadecimal digest of ``str(x)`` (kernel names must not depend on the process)."""
    return hashlib.sha1(str(x).encode()).hexdigest()[:16]


class VarNode:
    """One variable of the traced program.  ``kind``: ``"seq"`` (``[T, N]`` input read at ``t``), ``"state"`` (the
    potential carried over time), ``"tensor"`` (``[N]`` per-neuron input), ``"scalar"`` (kernel argument by value) or
    ``"tmp"`` (register)."""

    def __init__(self, name: str, kind: str, requires_grad: bool = False):
        self.name, self.kind, self.requires_grad = name, kind, requires_grad

    @property
    def cu_var(self) -> str:
        return {"seq": f"{self.name}_seq[t]", "state": "v", "tensor": f"{self.name}[index]", "scalar": self.name}.get(self.kind, f"r_{self.name}")

    @property
    def cu_grad(self) -> str:
        return f"g_{self.name}"

    @property
    def name_bp(self) -> str:
        """Name of the gradient tensor that goes with this variable in a backward kernel's argument list."""
        return "grad_" + self.name

    @property
    def cu_var_bp(self) -> str:
        """The register holding this variable's gradient inside the generated backward code (the reference's name for
        :attr:`cu_grad`)."""
        return self.cu_grad

    def __repr__(self) -> str:
        return f"VarNode({self.name}, {self.kind}, requires_grad={self.requires_grad})"


def analyse_graph(custom_fun: Callable, requires_grad: tuple):
    """``(input_nodes, inter_nodes, output_nodes, cmds)``.  ``cmds`` is a list of ``(dst, op, a, b)`` with ``op`` one of
    ``+ - * /`` and operands that are variable names or Python numbers."""
    params = list(inspect.signature(custom_fun).parameters.values())
    if len(params) < 2:
        raise ValueError("custom_fun must take at least (x, v_last)")
    if len(requires_grad) != len(params):
        raise ValueError("requires_grad needs one flag per argument of custom_fun")
    graph = fx.symbolic_trace(custom_fun).graph
    inputs: Dict[str, VarNode] = {}
    for i, (p, rg) in enumerate(zip(params, requires_grad)):
        if i == 0:
            kind = "seq"
        elif i == 1:
            kind = "state"
        elif p.annotation in (float, int):
            kind = "scalar"
        elif p.annotation is torch.Tensor or p.annotation is inspect.Parameter.empty:
            kind = "tensor"
        else:
            raise TypeError(f"argument {p.name}: annotate extra arguments as torch.Tensor, float or int")
        inputs[p.name] = VarNode(p.name, kind, bool(rg) and kind != "scalar")
    inter: Dict[str, VarNode] = {}
    cmds: List[Tuple[str, str, object, object]] = []
    out_name = None

    def operand(a):
        if isinstance(a, fx.Node):
            return a.name
        if isinstance(a, (int, float)):
            return float(a)
        raise TypeError(f"unsupported operand {a!r}")

    placeholders = [n for n in graph.nodes if n.op == "placeholder"]
    if [n.name for n in placeholders] != list(inputs):      # fx renames arguments that clash with its own names
        inputs = {n.name: VarNode(n.name, v.kind, v.requires_grad) for n, v in zip(placeholders, inputs.values())}
    for node in graph.nodes:
        if node.op == "placeholder":
            continue
        elif node.op == "call_function" and node.target in _BINARY:
            inter[node.name] = VarNode(node.name, "tmp")
            cmds.append((node.name, _BINARY[node.target], operand(node.args[0]), operand(node.args[1])))
        elif node.op == "call_function" and node.target in (operator.neg, torch.neg):
            inter[node.name] = VarNode(node.name, "tmp")
            cmds.append((node.name, "-", 0.0, operand(node.args[0])))
        elif node.op == "call_method" and node.target in _METHODS:
            inter[node.name] = VarNode(node.name, "tmp")
            cmds.append((node.name, _METHODS[node.target], operand(node.args[0]), operand(node.args[1])))
        elif node.op == "output":
            res = node.args[0]
            if not isinstance(res, fx.Node):
                raise ValueError("custom_fun must return one tensor")
            out_name = res.name
        else:
            raise NotImplementedError(f"only + - * / are supported in custom_fun, found {node.op} {node.target}")
    if out_name is None or out_name not in inter:
        raise ValueError("custom_fun must return the result of an arithmetic expression")
    outputs = {out_name: inter.pop(out_name)}
    return inputs, inter, outputs, cmds


def _ref(name, nodes: Dict[str, VarNode]) -> str:
    if isinstance(name, float):
        return repr(name) + "f"
    return nodes[name].cu_var


def _declare_params(kernel: CKernel2D, inputs: Dict[str, VarNode], const: bool = True) -> None:
    for node in inputs.values():
        if node.kind == "seq":
            kernel.add_param("const float *", f"{node.name}_seq")
        elif node.kind == "tensor":
            kernel.add_param("const float *", node.name)
        elif node.kind == "scalar":
            kernel.add_param("const float &", node.name)


def _threshold_params(kernel: CKernel2D, hard_reset: bool) -> None:
    """``v_th`` and (hard reset) ``v_reset``; a charge rule that already takes one of them as a scalar shares it."""
    for name in ("v_th",) + (("v_reset",) if hard_reset else ()):
        if name not in kernel.cparams:
            kernel.add_param("const float &", name)


def gen_forward_codes(input_nodes: dict, inter_nodes: dict, output_nodes: dict, cmds: list, hard_reset: bool):
    """``(kernel, kernel_name, cuda_cmds)``: the forward kernel, its name and the generated charge statements.
    Kernel arguments besides the traced inputs: ``v_init [N]``, ``spike_seq``, ``h_seq``, ``v_v_seq`` (``[T, N]``),
    ``v_th`` and, for a hard reset, ``v_reset``."""
    nodes = {**input_nodes, **inter_nodes, **output_nodes}
    cuda_cmds = [f"const float {nodes[dst].cu_var} = {_ref(a, nodes)} {op} {_ref(b, nodes)};" for dst, op, a, b in cmds]
    name = f"auto_neuron_fwd_{'hard' if hard_reset else 'soft'}_{hash_str((cmds, sorted(input_nodes)))}"
    k = CKernel2D(name)
    _declare_params(k, input_nodes)
    k.add_param("const float *", "v_init")
    for out in ("spike_seq", "h_seq", "v_v_seq"):
        k.add_param("float *", out)
    _threshold_params(k, hard_reset)
    h = next(iter(output_nodes.values())).cu_var
    k.pre_core = "        float v = v_init[index];"
    reset = f"v = spike * v_reset + (1.0f - spike) * {h};" if hard_reset else f"v = {h} - spike * v_th;"
    k.core = "\n".join("            " + c for c in cuda_cmds + [f"h_seq[t] = {h};", f"const float spike = {h} >= v_th ? 1.0f : 0.0f;", "spike_seq[t] = spike;",
                                                               reset, "v_v_seq[t] = v;"])
    return k, name, cuda_cmds


def gen_backward_codes(cuda_cmds: list, input_nodes: dict, output_nodes: dict, cmds: list, hard_reset: bool, detach_reset: bool,
                       surrogate_fuction):
    """``(kernel, kernel_name, input_bp_vars)``.  The kernel walks time backwards over ``grad_spike_seq``, ``grad_v_seq``
    and the saved ``h_seq`` / ``v_v_seq`` (with ``v_init`` for the first step), writes ``grad_<x>_seq``, ``grad_v_init`` and
    one ``grad_<name>`` ``[N]`` per extra tensor input that requires a gradient.  ``surrogate_fuction`` provides the
    surrogate derivative as C code through ``cuda_codes(y, x, dtype)`` (``y = g'(x)``)."""
    inter = {dst: VarNode(dst, "tmp") for dst, _, _, _ in cmds}
    nodes = {**input_nodes, **inter}
    state = next(n for n in input_nodes.values() if n.kind == "state")
    seq = next(n for n in input_nodes.values() if n.kind == "seq")
    out = next(iter(output_nodes))
    tensors = [n for n in input_nodes.values() if n.kind == "tensor" and n.requires_grad]
    name = (f"auto_neuron_bwd_{'hard' if hard_reset else 'soft'}_{'detach' if detach_reset else 'full'}_"
            f"{hash_str((cmds, sorted(input_nodes), type(surrogate_fuction).__name__, sorted(vars(surrogate_fuction).items(), key=str)))}")
    k = CKernel2D(name, reverse=True)
    from pathlib import Path
    from .... import ops
    k.extra_headers = (Path(ops.__file__).parent / "csrc" / "surrogate.cuh").read_text()      # sjb200::surrogate_grad<ID>
    _declare_params(k, input_nodes)
    for arg in ("v_init", "grad_spike_seq", "grad_v_seq", "h_seq", "v_v_seq"):
        k.add_param("const float *", arg)
    k.add_param("float *", f"grad_{seq.name}_seq")
    k.add_param("float *", "grad_v_init")
    for n in tensors:
        k.add_param("float *", f"grad_{n.name}")
    _threshold_params(k, hard_reset)
    pre = ["        float grad_h = 0.0f;   // dL/dh of the step after this one, already multiplied by dh/dv"] + \
          [f"        float acc_{n.name} = 0.0f;" for n in tensors]
    k.pre_core = "\n".join(pre)
    lines = ["const float h = h_seq[t];", "const float over_th = h - v_th;", "const float spike = over_th >= 0.0f ? 1.0f : 0.0f;"]
    lines.append(surrogate_fuction.cuda_codes(y="grad_s_to_h", x="over_th", dtype="float") if hasattr(surrogate_fuction, "cuda_codes")
                 else "const float grad_s_to_h = 0.0f;")
    if hard_reset:
        lines.append("float grad_v_to_h = 1.0f - spike;" if detach_reset else "float grad_v_to_h = 1.0f - spike + (v_reset - h) * grad_s_to_h;")
    else:
        lines.append("float grad_v_to_h = 1.0f;" if detach_reset else "float grad_v_to_h = 1.0f - v_th * grad_s_to_h;")
    # grad_h currently holds dL/dv_t coming from step t + 1 (through h_{t+1}); add the direct gradient on v_t
    lines.append("const float g_h = grad_spike_seq[t] * grad_s_to_h + (grad_v_seq[t] + grad_h) * grad_v_to_h;")
    # the charge rule needs its inputs of step t: v_{t-1} is the stored potential of the previous step
    lines.append("const float v = (t - dt >= 0) ? v_v_seq[t - dt] : v_init[index];")
    lines += list(cuda_cmds)
    # reverse-mode differentiation of the straight-line program
    lines += [f"float {VarNode(d, 'tmp').cu_grad} = 0.0f;" for d, _, _, _ in cmds] + [f"float {n.cu_grad} = 0.0f;" for n in input_nodes.values() if n.kind != "scalar"]
    lines.append(f"{VarNode(out, 'tmp').cu_grad} = g_h;")
    for dst, op, a, b in reversed(cmds):
        g = VarNode(dst, "tmp").cu_grad
        ra, rb = _ref(a, nodes), _ref(b, nodes)
        contrib = {"+": ("{g}", "{g}"), "-": ("{g}", "-{g}"), "*": ("{g} * {rb}", "{g} * {ra}"), "/": ("{g} / {rb}", "-{g} * {ra} / ({rb} * {rb})")}[op]
        for operand, expr in ((a, contrib[0]), (b, contrib[1])):
            if isinstance(operand, str) and nodes[operand].kind != "scalar":
                lines.append(f"{nodes[operand].cu_grad} += {expr.format(g=g, ra=ra, rb=rb)};")
    lines.append(f"grad_{seq.name}_seq[t] = {seq.cu_grad};")
    lines.append(f"grad_h = {state.cu_grad};")
    lines += [f"acc_{n.name} += {n.cu_grad};" for n in tensors]
    k.core = "\n".join("            " + ln for ln in lines)
    k.post_core = "\n".join(["        grad_v_init[index] = grad_h;"] + [f"        grad_{n.name}[index] = acc_{n.name};" for n in tensors])
    return k, name, [n.name for n in tensors]
