"""CUDA C code strings for scalar ``float`` and packed ``half2`` arithmetic, one function per operation
(``cuda_kernel/auto_cuda/cfunction.py:4-420`` of the reference: same names, argument order and conventions).

Every function takes the name of the result variable first; with ``None`` it returns the bare expression, otherwise the
statement ``result = expression;``.  Operands are C expressions given as strings.  ``dtype`` is ``"float"`` or ``"half2"``.
Multiplications by the literal one and additions of the literal zero are folded away.  The ``*_backward`` builders emit the
derivative of the surrogate of that name (the formulas of ``activation_based/surrogate.py``); for ``half2`` they evaluate both
halves in fp32 and pack the result, which keeps one formula per surrogate.
"""
from __future__ import annotations

from typing import Optional

__all__ = ["wrap_return_codes", "float2half2", "constant", "abs", "power", "if_else", "if_else_else", "greater_equal", "greater_than",
           "minimal", "maximum", "add", "sub", "mul", "div", "neg", "heaviside", "exp", "sigmoid", "sigmoid_backward", "atan_backward",
           "piecewise_leaky_relu_backward", "s2nn_backward", "q_pseudo_spike_backward", "leaky_k_relu_backward",
           "fake_numerical_gradient_backward", "log_tailed_relu_backward"]

_ONE = {"float": "1.0f", "half2": "__float2half2_rn(1.0f)"}
_ZERO = {"float": "0.0f", "half2": "__float2half2_rn(0.0f)"}


def _check(dtype: str) -> None:
    if dtype not in ("float", "half2"):
        raise NotImplementedError(dtype)


def wrap_return_codes(y: Optional[str], codes: str) -> str:
    return f"({codes})" if y is None else f"{y} = {codes};"


def float2half2(y: Optional[str], x: str) -> str:
    return wrap_return_codes(y, f"__float2half2_rn({x})")


def constant(y: Optional[str], x: float, dtype: str) -> str:
    _check(dtype)
    lit = f"{float(x)!r}f"
    return wrap_return_codes(y, lit if dtype == "float" else f"__float2half2_rn({lit})")


def _unary(float_fn: str, half_fn: str):
    def build(y: Optional[str], x: str, dtype: str) -> str:
        _check(dtype)
        return wrap_return_codes(y, f"{float_fn}({x})" if dtype == "float" else f"{half_fn}({x})")
    return build


abs = _unary("fabsf", "__habs2")
exp = _unary("expf", "h2exp")
neg = _unary("-", "__hneg2")


def _binary(float_op: str, half_fn: str, identity: Optional[dict] = None, left_identity: bool = True):
    def build(z: Optional[str], x: str, y: str, dtype: str) -> str:
        _check(dtype)
        if identity is not None:
            if left_identity and x == identity[dtype]:
                return wrap_return_codes(z, y)
            if y == identity[dtype]:
                return wrap_return_codes(z, x)
        return wrap_return_codes(z, f"{x} {float_op} {y}" if dtype == "float" else f"{half_fn}({x}, {y})")
    return build


add = _binary("+", "__hadd2", _ZERO)
sub = _binary("-", "__hsub2", _ZERO, left_identity=False)
mul = _binary("*", "__hmul2", _ONE)
div = _binary("/", "__h2div", _ONE, left_identity=False)


def power(z: Optional[str], x: str, y: str, dtype: str) -> str:
    _check(dtype)
    return wrap_return_codes(z, f"__powf({x}, {y})" if dtype == "float" else f"h2exp(__hmul2(h2log2({x}), __hmul2(__float2half2_rn(0.6931471806f), {y})))")


def _compare(float_op: str, half_fn: str):
    def build(z: Optional[str], x: str, y: str, dtype: str) -> str:
        _check(dtype)
        return wrap_return_codes(z, f"(float) ({x} {float_op} {y})" if dtype == "float" else f"{half_fn}({x}, {y})")
    return build


greater_equal = _compare(">=", "__hgeu2")
greater_than = _compare(">", "__hgtu2")


def minimal(z: Optional[str], x: str, y: str, dtype: str) -> str:
    _check(dtype)
    return wrap_return_codes(z, f"fminf({x}, {y})" if dtype == "float" else f"__hmin2({x}, {y})")


def maximum(z: Optional[str], x: str, y: str, dtype: str) -> str:
    _check(dtype)
    return wrap_return_codes(z, f"fmaxf({x}, {y})" if dtype == "float" else f"__hmax2({x}, {y})")


def if_else(z: Optional[str], x: str, y: str, mask: str, dtype: str) -> str:
    """``mask`` holds 1 where ``x`` is taken and 0 where ``y`` is."""
    _check(dtype)
    if dtype == "float":
        return wrap_return_codes(z, f"{x} * {mask} + {y} * (1.0f - {mask})")
    return wrap_return_codes(z, f"__hfma2({x}, {mask}, __hmul2({y}, __hsub2(__float2half2_rn(1.0f), {mask})))")


def if_else_else(w: Optional[str], x: str, y: str, z: str, mask_x: str, mask_y: str, dtype: str) -> str:
    """``x`` where ``mask_x``, else ``y`` where ``mask_y``, else ``z``."""
    return if_else(w, x, if_else(None, y, z, mask_y, dtype), mask_x, dtype)


def heaviside(y: Optional[str], x: str, dtype: str) -> str:
    _check(dtype)
    return wrap_return_codes(y, f"(float) ({x} >= 0.0f)" if dtype == "float" else f"__hgeu2({x}, __float2half2_rn(0.0f))")


def sigmoid(y: Optional[str], x: str, alpha: float, dtype: str) -> str:
    _check(dtype)
    a = f"{float(alpha)!r}f"
    if dtype == "float":
        return wrap_return_codes(y, f"1.0f / (1.0f + expf(- {a} * {x}))")
    return wrap_return_codes(y, f"__h2div(__float2half2_rn(1.0f), __hadd2(__float2half2_rn(1.0f), h2exp(__hneg2(__hmul2(__float2half2_rn({a}), {x})))))")


def _surrogate_backward(formula):
    """``formula(v, params...)`` gives the fp32 C expression of g'(v); the builder adapts it to the two dtypes.  The built
    function is ``f(y, x, <params...>, dtype)``; parameters and ``dtype`` may also be given by keyword (their names are the
    formula's argument names)."""
    import inspect
    names = list(inspect.signature(formula).parameters)[1:]

    def build(y: str, x: str, *args, **kwargs) -> str:
        bound = dict(zip(names + ["dtype"], args))
        for k, v in kwargs.items():
            if k not in names + ["dtype"] or k in bound:
                raise TypeError(f"unexpected or repeated argument {k!r}; expected {names + ['dtype']}")
            bound[k] = v
        missing = [n for n in names + ["dtype"] if n not in bound]
        if missing or len(args) > len(names) + 1:
            raise TypeError(f"expected (y, x, {', '.join(names)}, dtype); missing {missing}")
        dtype = bound["dtype"]
        _check(dtype)
        lits = [f"{float(bound[n])!r}f" for n in names]
        if dtype == "float":
            return f"const float {y} = {formula(x, *lits)};"
        lo, hi = f"{y}_lo", f"{y}_hi"
        return (f"const float2 {y}_f = __half22float2({x}); "
                f"const float {lo} = {formula(y + '_f.x', *lits)}; const float {hi} = {formula(y + '_f.y', *lits)}; "
                f"const half2 {y} = __floats2half2_rn({lo}, {hi});")
    return build


sigmoid_backward = _surrogate_backward(
    lambda v, alpha: f"(1.0f - 1.0f / (1.0f + expf(-{alpha} * {v}))) * (1.0f / (1.0f + expf(-{alpha} * {v}))) * {alpha}")
atan_backward = _surrogate_backward(
    lambda v, alpha: f"{alpha} * 0.5f / (1.0f + (1.5707963267948966f * {alpha} * {v}) * (1.5707963267948966f * {alpha} * {v}))")
piecewise_leaky_relu_backward = _surrogate_backward(
    lambda v, w, c: f"(fabsf({v}) > {w} ? {c} : 1.0f / {w})")
s2nn_backward = _surrogate_backward(
    lambda v, alpha, beta: f"({v} < 0.0f ? {alpha} * (1.0f / (1.0f + expf(-{alpha} * {v}))) * (1.0f - 1.0f / (1.0f + expf(-{alpha} * {v}))) : {beta} / ({v} + 1.0f))")
q_pseudo_spike_backward = _surrogate_backward(
    lambda v, alpha: f"__powf(1.0f + 2.0f / ({alpha} - 1.0f) * fabsf({v}), -{alpha})")
leaky_k_relu_backward = _surrogate_backward(
    lambda v, leak, k: f"({v} >= 0.0f ? {k} : {leak})")
fake_numerical_gradient_backward = _surrogate_backward(
    lambda v, alpha: f"fminf(({v} >= 0.0f ? 1.0f : -1.0f) / {v}, {alpha})")
log_tailed_relu_backward = _surrogate_backward(
    lambda v, alpha: f"({v} > 1.0f ? 1.0f / {v} : ({v} > 0.0f ? 1.0f : {alpha}))")
