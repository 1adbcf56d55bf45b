"""ATen FX graph -> CUDA C++ for user-defined neuron dynamics.

``trace_step`` captures the single-step function of a custom neuron twice with ``make_fx``: the forward
step ``(inputs, states) -> (outputs, new states)`` and the *joint* step, which recomputes the forward step
and back-propagates ``(grad outputs, grad new states)`` to ``(grad inputs, grad states)`` — custom
``autograd.Function`` s (surrogate gradients) are traced through their own ``backward``.  Both graphs hold
elementwise ATen nodes only; ``emit_device_function`` turns each into one ``__device__`` function in which
every value is an fp32 register (booleans are 0.0f / 1.0f), and ``emit_module`` wraps the two functions in
the time-loop kernels:

* forward: states live in registers across ``T``; writes the outputs and, if asked, the state after every
  step (what ``store_state_seqs`` returns and, at the same time, everything backward needs);
* backward: walks ``t = T-1 .. 0``, reloads the inputs and the state before step ``t``, calls the joint
  function, stores the input gradients and carries the state gradients in registers.

Role of ``torch2triton/graph2triton.py:135-389`` and ``flexsn/template.py:36-597`` in the reference, which
emit Triton source and save min-cut-chosen intermediates instead of recomputing inside the step.
"""
from __future__ import annotations

import hashlib
import math
import operator
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
from torch.fx.experimental.proxy_tensor import make_fx

__all__ = ["UnsupportedCore", "StepGraphs", "trace_step", "emit_device_function", "emit_module", "SUPPORTED_OPS"]

aten = torch.ops.aten


class UnsupportedCore(RuntimeError):
    """The step function cannot be expressed as a per-element register program."""


def _lit(v) -> str:
    if isinstance(v, bool):
        return "1.0f" if v else "0.0f"
    v = float(v)
    if math.isnan(v):
        return "__int_as_float(0x7fc00000)"
    if math.isinf(v):
        return "__int_as_float(0x7f800000)" if v > 0 else "__int_as_float(0xff800000)"
    # fp32 value of the python scalar, spelled exactly
    f = torch.tensor(v, dtype=torch.float32).item()
    return f"{float(f).hex()}f" if f != int(f) or abs(f) > 1e9 else f"{int(f)}.0f"


def _b(x: str) -> str:
    return f"(({x}) != 0.0f)"


def _f(cond: str) -> str:
    return f"(({cond}) ? 1.0f : 0.0f)"


def _bin(op):
    return lambda a, b: f"({a} {op} {b})"


def _cmp(op):
    return lambda a, b: _f(f"{a} {op} {b}")


def _scaled(a, b, alpha, fn):
    # add/sub with alpha: a (+|-) alpha*b, non-contracted like the eager kernels
    if alpha is None or alpha == "1.0f":
        return f"__f{fn}_rn({a}, {b})"
    return f"__f{fn}_rn({a}, __fmul_rn({alpha}, {b}))"


def _div(a, b, rounding_mode=None):
    q = f"__fdiv_rn({a}, {b})"
    if rounding_mode is None:
        return q
    return f"truncf({q})" if rounding_mode == "trunc" else f"floorf({q})"


def _round_dtype(x: str, dtype) -> str:
    if dtype == torch.float16:
        return f"__half2float(__float2half_rn({x}))"
    if dtype == torch.bfloat16:
        return f"__bfloat162float(__float2bfloat16_rn({x}))"
    if dtype == torch.bool:
        return _f(f"{x} != 0.0f")
    if dtype in (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8):
        return f"truncf({x})"
    return x


#: ATen overload packet name -> emitter(args as C expressions / python scalars already literalised)
SUPPORTED_OPS: Dict[str, Callable[..., str]] = {
    "add": lambda a, b, alpha=None: _scaled(a, b, alpha, "add"),
    "sub": lambda a, b, alpha=None: _scaled(a, b, alpha, "sub"),
    "rsub": lambda a, b, alpha=None: _scaled(b, a, alpha, "sub"),
    "mul": lambda a, b: f"__fmul_rn({a}, {b})",
    "div": _div,
    "true_divide": _div,
    "neg": lambda a: f"(-{a})",
    "abs": lambda a: f"fabsf({a})",
    "reciprocal": lambda a: f"__frcp_rn({a})",
    "square": lambda a: f"__fmul_rn({a}, {a})",
    "ge": _cmp(">="), "gt": _cmp(">"), "le": _cmp("<="), "lt": _cmp("<"), "eq": _cmp("=="), "ne": _cmp("!="),
    "logical_and": lambda a, b: _f(f"{_b(a)} && {_b(b)}"),
    "logical_or": lambda a, b: _f(f"{_b(a)} || {_b(b)}"),
    "logical_xor": lambda a, b: _f(f"{_b(a)} != {_b(b)}"),
    "logical_not": lambda a: _f(f"!{_b(a)}"),
    "bitwise_and": lambda a, b: _f(f"{_b(a)} && {_b(b)}"),      # booleans only (checked by the tracer)
    "bitwise_or": lambda a, b: _f(f"{_b(a)} || {_b(b)}"),
    "bitwise_xor": lambda a, b: _f(f"{_b(a)} != {_b(b)}"),
    "bitwise_not": lambda a: _f(f"!{_b(a)}"),
    "where": lambda c, a, b: f"({_b(c)} ? {a} : {b})",
    "masked_fill": lambda a, m, v: f"({_b(m)} ? {v} : {a})",
    "sigmoid": lambda a: f"__frcp_rn(__fadd_rn(1.0f, expf(-{a})))",
    "sigmoid_backward": lambda g, y: f"__fmul_rn({g}, __fmul_rn(__fsub_rn(1.0f, {y}), {y}))",
    "tanh": lambda a: f"tanhf({a})",
    "tanh_backward": lambda g, y: f"__fmul_rn({g}, __fsub_rn(1.0f, __fmul_rn({y}, {y})))",
    "threshold_backward": lambda g, x, th: f"(({x} <= {th}) ? 0.0f : {g})",
    "relu": lambda a: f"fmaxf({a}, 0.0f)",
    "hardtanh": lambda a, lo="-1.0f", hi="1.0f": f"fminf(fmaxf({a}, {lo}), {hi})",
    "hardtanh_backward": lambda g, x, lo, hi: f"((({x}) <= {lo} || ({x}) >= {hi}) ? 0.0f : {g})",
    "leaky_relu": lambda a, s="0x1.47ae14p-7f": f"(({a}) > 0.0f ? {a} : __fmul_rn({a}, {s}))",
    "leaky_relu_backward": lambda g, x, s, _r=None: f"(({x}) > 0.0f ? {g} : __fmul_rn({g}, {s}))",
    "exp": lambda a: f"expf({a})", "expm1": lambda a: f"expm1f({a})", "exp2": lambda a: f"exp2f({a})",
    "log": lambda a: f"logf({a})", "log1p": lambda a: f"log1pf({a})", "log2": lambda a: f"log2f({a})",
    "sqrt": lambda a: f"__fsqrt_rn({a})", "rsqrt": lambda a: f"__frcp_rn(__fsqrt_rn({a}))",
    "sin": lambda a: f"sinf({a})", "cos": lambda a: f"cosf({a})", "tan": lambda a: f"tanf({a})",
    "atan": lambda a: f"atanf({a})", "erf": lambda a: f"erff({a})", "erfc": lambda a: f"erfcf({a})",
    "floor": lambda a: f"floorf({a})", "ceil": lambda a: f"ceilf({a})", "round": lambda a: f"nearbyintf({a})",
    "trunc": lambda a: f"truncf({a})", "frac": lambda a: f"__fsub_rn({a}, truncf({a}))",
    "sign": lambda a: f"(({a}) > 0.0f ? 1.0f : (({a}) < 0.0f ? -1.0f : 0.0f))",
    "sgn": lambda a: f"(({a}) > 0.0f ? 1.0f : (({a}) < 0.0f ? -1.0f : 0.0f))",
    "heaviside": lambda a, v: f"(({a}) == 0.0f ? {v} : (({a}) > 0.0f ? 1.0f : 0.0f))",
    "minimum": lambda a, b: f"fminf({a}, {b})", "maximum": lambda a, b: f"fmaxf({a}, {b})",
    "fmin": lambda a, b: f"fminf({a}, {b})", "fmax": lambda a, b: f"fmaxf({a}, {b})",
    "clamp_min": lambda a, lo: f"fmaxf({a}, {lo})", "clamp_max": lambda a, hi: f"fminf({a}, {hi})",
    "pow": lambda a, b: (f"__fmul_rn({a}, {a})" if b == "2.0f" else f"powf({a}, {b})"),
    "fmod": lambda a, b: f"fmodf({a}, {b})",
    "remainder": lambda a, b: f"__fsub_rn({a}, __fmul_rn(floorf(__fdiv_rn({a}, {b})), {b}))",
    "zeros_like": lambda a, **_: "0.0f", "ones_like": lambda a, **_: "1.0f",
    "full_like": lambda a, v, **_: f"{v}",
    "scalar_tensor": lambda v, **_: f"{v}",
    "detach": lambda a: a, "alias": lambda a: a, "clone": lambda a, **_: a, "lift_fresh_copy": lambda a: a,
    "contiguous": lambda a, **_: a, "view": lambda a, *_: a, "_unsafe_view": lambda a, *_: a,
    "reshape": lambda a, *_: a, "expand": lambda a, *_, **__: a, "positive": lambda a: a,
    "softplus": lambda a, beta="1.0f", th="20.0f": f"((__fmul_rn({a}, {beta}) > {th}) ? {a} : __fdiv_rn(log1pf(expf(__fmul_rn({a}, {beta}))), {beta}))",
}


def _clamp(a, lo=None, hi=None):
    x = a
    if lo is not None:
        x = f"fmaxf({x}, {lo})"
    if hi is not None:
        x = f"fminf({x}, {hi})"
    return x


SUPPORTED_OPS["clamp"] = _clamp
SUPPORTED_OPS["clip"] = _clamp


@dataclass
class StepGraphs:
    """The traced forward and joint graphs of one step function plus its calling convention."""
    num_inputs: int
    num_states: int
    num_outputs: int
    forward: torch.fx.GraphModule
    joint: Optional[torch.fx.GraphModule]
    needs_grad: Tuple[bool, ...]                 # per (input..., state...) argument
    signature: str = field(default="")


def _check_elementwise(gm: torch.fx.GraphModule, shape: torch.Size) -> None:
    for node in gm.graph.nodes:
        if node.op == "get_attr":
            raise UnsupportedCore(f"the step function captures tensor `{node.target}`; pass it as an input or a state")
        if node.op != "call_function":
            continue
        val = node.meta.get("val", None)
        if isinstance(val, torch.Tensor) and val.shape != shape and val.numel() != 1:
            raise UnsupportedCore(f"`{node.target}` produces shape {tuple(val.shape)}; only elementwise cores "
                                  f"over shape {tuple(shape)} compile")
        if node.target is operator.getitem:
            continue
        name = node.target.overloadpacket.__name__ if hasattr(node.target, "overloadpacket") else str(node.target)
        if name == "_to_copy":
            continue
        if name not in SUPPORTED_OPS:
            raise UnsupportedCore(f"ATen operator `{node.target}` has no CUDA translation")
        if name.startswith("bitwise_"):
            for a in node.args:
                v = a.meta.get("val") if isinstance(a, torch.fx.Node) else None
                if isinstance(v, torch.Tensor) and v.dtype != torch.bool:
                    raise UnsupportedCore("bitwise operators compile for boolean tensors only")


def trace_step(core: Callable, num_inputs: int, num_states: int, num_outputs: int,
               example_inputs: Optional[Sequence[torch.Tensor]] = None,
               requires_grad: Optional[Sequence[bool]] = None, training: bool = True) -> StepGraphs:
    """Captures ``core`` on one step's worth of example tensors (defaults: fp32 vectors of 8 elements)."""
    n_args = num_inputs + num_states
    if example_inputs is None:
        example = [torch.zeros(8) for _ in range(n_args)]
    else:
        example = [torch.zeros(e.shape, dtype=e.dtype if e.is_floating_point() else torch.float32) for e in example_inputs]
        if len(example) != n_args:
            raise ValueError(f"example_inputs must hold {n_args} tensors (inputs then states), got {len(example)}")
    shape = example[0].shape
    if any(e.shape != shape for e in example):
        raise UnsupportedCore("all inputs and states of a compiled core must have one shape")
    # values in (0, 1) keep log/sqrt/div finite while tracing
    example = [torch.rand_like(e, dtype=torch.float32).to(e.dtype) * 0.5 + 0.25 for e in example]
    needs = tuple(bool(r) for r in requires_grad) if requires_grad is not None else (True,) * n_args
    if len(needs) != n_args:
        raise ValueError(f"requires_grad must hold {n_args} flags")

    def fwd(*args):
        res = core(*args)
        res = tuple(res) if isinstance(res, (tuple, list)) else (res,)
        if len(res) != num_outputs + num_states:
            raise ValueError(f"core returned {len(res)} tensors, expected {num_outputs} outputs + {num_states} states")
        return res

    with torch.no_grad():
        g_fwd = make_fx(fwd, tracing_mode="real")(*example)
    _check_elementwise(g_fwd, shape)

    g_joint = None
    if training and any(needs):
        def joint(*flat):
            args, cot = flat[:n_args], flat[n_args:]
            args = [a.detach().requires_grad_(needs[i]) for i, a in enumerate(args)]
            with torch.enable_grad():
                res = fwd(*args)
                pairs = [(r, c) for r, c in zip(res, cot) if r.requires_grad]
                wanted = [a for a, n in zip(args, needs) if n]
                if pairs:
                    grads = torch.autograd.grad([r for r, _ in pairs], wanted, [c for _, c in pairs], allow_unused=True)
                else:
                    grads = [None] * len(wanted)
            it = iter(grads)
            out = []
            for a, n in zip(args, needs):
                g = next(it) if n else None
                out.append(torch.zeros_like(a) if g is None else g)
            return tuple(out)

        with torch.no_grad():
            out_ex = fwd(*example)
        cot = [torch.rand_like(o, dtype=torch.float32).to(o.dtype if o.is_floating_point() else torch.float32) for o in out_ex]
        g_joint = make_fx(joint, tracing_mode="real")(*example, *cot)
        _check_elementwise(g_joint, shape)
    sg = StepGraphs(num_inputs, num_states, num_outputs, g_fwd, g_joint, needs)
    body = emit_device_function(g_fwd, "step_fwd") + (emit_device_function(g_joint, "step_bwd") if g_joint is not None else "")
    sg.signature = hashlib.sha256(body.encode()).hexdigest()
    return sg


def emit_device_function(gm: torch.fx.GraphModule, name: str) -> str:
    """One ``__device__`` function: placeholders become ``float`` parameters, results ``float&`` ones."""
    names: Dict[torch.fx.Node, str] = {}
    params: List[str] = []
    lines: List[str] = []
    results: List[str] = []

    def ref(a):
        if isinstance(a, torch.fx.Node):
            return names[a]
        if isinstance(a, (bool, int, float)):
            return _lit(a)
        return a          # None, strings (rounding_mode), dtypes ... consumed by the emitter

    for node in gm.graph.nodes:
        if node.op == "placeholder":
            names[node] = f"a{len(params)}"
            params.append(f"const float a{len(params)}")
        elif node.op == "call_function":
            var = f"t{len(names)}"
            if node.target is operator.getitem:
                raise UnsupportedCore("multi-output ATen operators are not supported in a compiled core")
            pkt = node.target.overloadpacket.__name__
            if pkt == "_to_copy":
                expr = _round_dtype(ref(node.args[0]), node.kwargs.get("dtype"))
            else:
                kwargs = {k: ref(v) for k, v in node.kwargs.items()
                          if k not in ("dtype", "layout", "device", "pin_memory", "memory_format", "non_blocking")}
                args = [ref(a) for a in node.args]
                if pkt in ("div", "true_divide") and len(node.args) == 2 and not isinstance(node.args[1], torch.fx.Node):
                    # tensor / python scalar: the eager CUDA kernel multiplies by the fp32 reciprocal
                    inv = torch.tensor(1.0, dtype=torch.float32) / torch.tensor(float(node.args[1]), dtype=torch.float32)
                    expr = f"__fmul_rn({args[0]}, {_lit(inv.item())})" if not kwargs else SUPPORTED_OPS[pkt](*args, **kwargs)
                else:
                    expr = SUPPORTED_OPS[pkt](*args, **kwargs)
                val = node.meta.get("val")
                # an op computed in half precision by eager rounds its result; keep the rounding points
                if isinstance(val, torch.Tensor) and val.dtype in (torch.float16, torch.bfloat16):
                    expr = _round_dtype(expr, val.dtype)
            lines.append(f"    const float {var} = {expr};")
            names[node] = var
        elif node.op == "output":
            outs = node.args[0]
            outs = outs if isinstance(outs, (tuple, list)) else (outs,)
            for i, o in enumerate(outs):
                params.append(f"float& r{i}")
                results.append(f"    r{i} = {ref(o) if o is not None else '0.0f'};")
    return (f"__device__ __forceinline__ void {name}({', '.join(params)}) {{\n" + "\n".join(lines + results) + "\n}\n")


_PRELUDE = r"""// generated by spikingjelly_b200.ops.flexsn -- do not edit
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace {
template <typename T> struct Cvt;
template <> struct Cvt<float> { static __device__ __forceinline__ float ld(float v) { return v; } static __device__ __forceinline__ float st(float v) { return v; } };
template <> struct Cvt<__half> { static __device__ __forceinline__ float ld(__half v) { return __half2float(v); } static __device__ __forceinline__ __half st(float v) { return __float2half_rn(v); } };
template <> struct Cvt<__nv_bfloat16> { static __device__ __forceinline__ float ld(__nv_bfloat16 v) { return __bfloat162float(v); } static __device__ __forceinline__ __nv_bfloat16 st(float v) { return __float2bfloat16_rn(v); } };

template <typename T, int V> struct alignas(sizeof(T) * V) Vec { T e[V]; };

template <typename T, int V>
__device__ __forceinline__ void load(const void* base, long long idx, float (&r)[V]) {
    if (base == nullptr) {
#pragma unroll
        for (int i = 0; i < V; ++i) r[i] = 0.0f;
        return;
    }
    const Vec<T, V> v = *reinterpret_cast<const Vec<T, V>*>(reinterpret_cast<const T*>(base) + idx);
#pragma unroll
    for (int i = 0; i < V; ++i) r[i] = Cvt<T>::ld(v.e[i]);
}
template <typename T, int V>
__device__ __forceinline__ void store(void* base, long long idx, const float (&r)[V]) {
    if (base == nullptr) return;
    Vec<T, V> v;
#pragma unroll
    for (int i = 0; i < V; ++i) v.e[i] = Cvt<T>::st(r[i]);
    *reinterpret_cast<Vec<T, V>*>(reinterpret_cast<T*>(base) + idx) = v;
}
}  // namespace
"""


def emit_module(sg: StepGraphs) -> str:
    """Complete ``.cu`` translation unit with C launchers ``flexsn_forward`` / ``flexsn_backward``."""
    NI, NS, NO = sg.num_inputs, sg.num_states, sg.num_outputs
    nsd = max(NS, 1)
    src = [_PRELUDE, f"#define NI {NI}\n#define NS {NS}\n#define NO {NO}\n#define NSD {nsd}\n#define NOD {max(NO, 1)}\n"]
    src.append("""
struct FwdArgs { const void* in[NI]; const void* s0[NSD]; void* out[NOD]; void* s_seq[NSD]; void* s_last[NSD]; long long n; int T; };
struct BwdArgs { const void* in[NI]; const void* s0[NSD]; const void* s_seq[NSD]; const void* g_out[NOD]; const void* g_seq[NSD];
                 const void* g_last[NSD]; void* g_in[NI]; void* g_s0[NSD]; long long n; int T; };
""")
    src.append(emit_device_function(sg.forward, "step_fwd"))
    # ---- forward kernel
    # Time is walked in chunks of TC steps: every load of a chunk is issued before the first use, so a thread has
    # TC x (number of streams) requests in flight instead of waiting for each step's data in turn.
    in_decl = "\n".join(f"            float x{i}[TC][V];" for i in range(NI))
    in_load = "\n".join(f"                    load<T, V>(a.in[{i}], off, x{i}[c]);" for i in range(NI))
    st_decl = "\n".join(f"    float s{j}[V]; load<T, V>(a.s0[{j}], e, s{j});" for j in range(NS))
    call_args = ", ".join([f"x{i}[c][k]" for i in range(NI)] + [f"s{j}[k]" for j in range(NS)]
                          + [f"y{o}[k]" for o in range(NO)] + [f"n{j}" for j in range(NS)])
    new_states = "".join(f" float n{j};" for j in range(NS))
    commit = "".join(f" s{j}[k] = n{j};" for j in range(NS))
    out_decl = "\n".join(f"                float y{o}[V];" for o in range(NO))
    out_store = "\n".join(f"                store<T, V>(a.out[{o}], off, y{o});" for o in range(NO))
    seq_store = "\n".join(f"                store<T, V>(a.s_seq[{j}], off, s{j});" for j in range(NS))
    last_store = "\n".join(f"    store<T, V>(a.s_last[{j}], e, s{j});" for j in range(NS))
    src.append(f"""
constexpr int TC = 4;     // forward: steps whose loads are issued together
constexpr int TCB = 2;    // backward: four streams per step, so half the depth keeps two blocks per SM resident

template <typename T, int V>
__global__ void __launch_bounds__(256) forward_kernel(const FwdArgs a) {{
    const long long e = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * V;
    if (e >= a.n) return;
{st_decl}
    for (int t0 = 0; t0 < a.T; t0 += TC) {{
{in_decl}
#pragma unroll
            for (int c = 0; c < TC; ++c) {{
                if (t0 + c < a.T) {{
                    const long long off = static_cast<long long>(t0 + c) * a.n + e;
{in_load}
                }}
            }}
#pragma unroll
            for (int c = 0; c < TC; ++c) {{
                if (t0 + c >= a.T) break;
                const long long off = static_cast<long long>(t0 + c) * a.n + e;
{out_decl}
#pragma unroll
                for (int k = 0; k < V; ++k) {{{new_states}
                    step_fwd({call_args});{commit}
                }}
{out_store}
{seq_store}
            }}
    }}
{last_store}
}}
""")
    if sg.joint is not None:
        src.append(emit_device_function(sg.joint, "step_bwd"))
        chunk_decl = "\n".join([f"            float x{i}[TCB][V];" for i in range(NI)] + [f"            float p{j}[TCB][V];" for j in range(NS)]
                               + [f"            float go{o}[TCB][V];" for o in range(NO)] + [f"            float q{j}[TCB][V];" for j in range(NS)])
        chunk_load = "\n".join(
            [f"                    load<T, V>(a.in[{i}], off, x{i}[c]);" for i in range(NI)]
            + [f"                    if (t > 0) load<T, V>(a.s_seq[{j}], off - a.n, p{j}[c]); else load<T, V>(a.s0[{j}], e, p{j}[c]);" for j in range(NS)]
            + [f"                    load<T, V>(a.g_out[{o}], off, go{o}[c]);" for o in range(NO)]
            + [f"                    load<T, V>(a.g_seq[{j}], off, q{j}[c]);" for j in range(NS)])
        gseq_add = "\n".join(
            f"                if (a.g_seq[{j}] != nullptr) {{\n#pragma unroll\n                    for (int k = 0; k < V; ++k) gs{j}[k] = __fadd_rn(gs{j}[k], q{j}[c][k]); }}"
            for j in range(NS))
        gs_decl = "\n".join(f"    float gs{j}[V]; load<T, V>(a.g_last[{j}], e, gs{j});" for j in range(NS))
        gx_decl = "\n".join(f"                float gx{i}[V];" for i in range(NI))
        bcall = ", ".join([f"x{i}[c][k]" for i in range(NI)] + [f"p{j}[c][k]" for j in range(NS)]
                          + [f"go{o}[c][k]" for o in range(NO)] + [f"gs{j}[k]" for j in range(NS)]
                          + [f"gx{i}[k]" for i in range(NI)] + [f"m{j}" for j in range(NS)])
        m_decl = "".join(f" float m{j};" for j in range(NS))
        m_commit = "".join(f" gs{j}[k] = m{j};" for j in range(NS))
        gx_store = "\n".join(f"                store<T, V>(a.g_in[{i}], off, gx{i});" for i in range(NI))
        gs0_store = "\n".join(f"    store<T, V>(a.g_s0[{j}], e, gs{j});" for j in range(NS))
        src.append(f"""
template <typename T, int V>
__global__ void __launch_bounds__(256) backward_kernel(const BwdArgs a) {{
    const long long e = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * V;
    if (e >= a.n) return;
{gs_decl}
    const int chunks = (a.T + TCB - 1) / TCB;
    for (int ck = chunks - 1; ck >= 0; --ck) {{
            const int t0 = ck * TCB;
{chunk_decl}
#pragma unroll
            for (int c = 0; c < TCB; ++c) {{
                const int t = t0 + c;
                if (t < a.T) {{
                    const long long off = static_cast<long long>(t) * a.n + e;
{chunk_load}
                }}
            }}
#pragma unroll
            for (int c = TCB - 1; c >= 0; --c) {{
                const int t = t0 + c;
                if (t >= a.T) continue;
                const long long off = static_cast<long long>(t) * a.n + e;
{gseq_add}
{gx_decl}
#pragma unroll
                for (int k = 0; k < V; ++k) {{{m_decl}
                    step_bwd({bcall});{m_commit}
                }}
{gx_store}
            }}
    }}
{gs0_store}
}}
""")
    src.append("""
template <typename T>
static int launch_fwd(const FwdArgs& a, int vec, cudaStream_t s) {
    // Four elements per thread for every type (16-byte accesses in fp32, 8-byte in fp16 / bf16): measured on B200, eight
    // 16-bit elements per thread halve the thread count and run the backward kernel 1.4x slower (T 16, 1 M and 8 M neurons).
    constexpr int V = 4;
    if (a.n <= 0 || a.T < 0) return 0;
    if (vec) { const long long th = a.n / V; forward_kernel<T, V><<<static_cast<unsigned>((th + 255) / 256), 256, 0, s>>>(a); }
    else forward_kernel<T, 1><<<static_cast<unsigned>((a.n + 255) / 256), 256, 0, s>>>(a);
    return static_cast<int>(cudaGetLastError());
}
extern "C" __attribute__((visibility("default"))) int flexsn_forward(const FwdArgs* a, int dtype, int vec, void* stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
    case 0: return launch_fwd<float>(*a, vec, s);
    case 1: return launch_fwd<__half>(*a, vec, s);
    case 2: return launch_fwd<__nv_bfloat16>(*a, vec, s);
    default: return -1;
    }
}
""")
    if sg.joint is not None:
        src.append("""
template <typename T>
static int launch_bwd(const BwdArgs& a, int vec, cudaStream_t s) {
    // Four elements per thread for every type (16-byte accesses in fp32, 8-byte in fp16 / bf16): measured on B200, eight
    // 16-bit elements per thread halve the thread count and run the backward kernel 1.4x slower (T 16, 1 M and 8 M neurons).
    constexpr int V = 4;
    if (a.n <= 0 || a.T < 0) return 0;
    if (vec) { const long long th = a.n / V; backward_kernel<T, V><<<static_cast<unsigned>((th + 255) / 256), 256, 0, s>>>(a); }
    else backward_kernel<T, 1><<<static_cast<unsigned>((a.n + 255) / 256), 256, 0, s>>>(a);
    return static_cast<int>(cudaGetLastError());
}
extern "C" __attribute__((visibility("default"))) int flexsn_backward(const BwdArgs* a, int dtype, int vec, void* stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
    case 0: return launch_bwd<float>(*a, vec, s);
    case 1: return launch_bwd<__half>(*a, vec, s);
    case 2: return launch_bwd<__nv_bfloat16>(*a, vec, s);
    default: return -1;
    }
}
""")
    return "".join(src)
