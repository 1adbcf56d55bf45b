"""Surrogate gradient functions.

Every surrogate is one row of ``SURROGATES``: an integer id (shared with the
CUDA scan kernels, see ``ops/csrc/surrogate.cuh``), the names of up to two float
parameters, the derivative ``g'(x)`` used in backward and the smooth primitive
``g(x)``.  The ``nn.Module`` classes (``ATan``, ``Sigmoid`` …) are thin views of
a row; a single autograd function does Heaviside forward / table-driven backward.

Parity: ``spikingjelly/activation_based/surrogate.py`` — base class :291-398 and
the 19 classes at :401-3429 (derivatives listed there are reproduced exactly).
"""
from __future__ import annotations

import math
import numbers
from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

__all__ = [
    "heaviside", "SurrogateFunctionBase", "SURROGATES", "surrogate_spec",
    "PiecewiseQuadratic", "PiecewiseExp", "Sigmoid", "SoftSign", "SuperSpike", "ATan",
    "NonzeroSignLogAbs", "Erf", "PiecewiseLeakyReLU", "SquarewaveFourierSeries", "S2NN",
    "QPseudoSpike", "LeakyKReLU", "FakeNumericalGradient", "LogTailedReLU",
    "DeterministicPass", "PoissonPass", "MultiLevelSpikeCount", "Rect",
    "check_manual_grad", "check_cuda_grad", "plot_surrogate_function",
]


def heaviside(x: torch.Tensor) -> torch.Tensor:
    """``1`` where ``x >= 0`` else ``0``, in ``x``'s dtype (``surrogate.py:12-60``)."""
    return (x >= 0).to(x)


# ------------------------------------------------------------------- the table
@dataclass(frozen=True)
class _Spec:
    sid: int
    name: str
    params: Tuple[str, ...]
    grad: Callable[..., torch.Tensor]            # g'(x, *params)
    primitive: Optional[Callable[..., torch.Tensor]]


def _g_sigmoid(x, alpha):
    s = torch.sigmoid(x * alpha)
    return (1.0 - s) * s * alpha


def _g_atan(x, alpha):
    a = alpha / 2
    ax = math.pi * a * x
    return a / (1 + ax * ax)


def _g_pq(x, alpha):
    xa = x.abs()
    return (-(alpha ** 2) * xa + alpha).masked_fill(xa > (1 / alpha), 0)


def _g_squarewave(x, n, T_period):
    w = math.pi * 2.0 / T_period
    g = torch.zeros_like(x)
    for i in range(1, int(n)):
        g = g + torch.cos((2 * i - 1.0) * w * x)
    return g * (4.0 / T_period)


def _g_s2nn(x, alpha, beta):
    s = torch.sigmoid(alpha * x)
    return torch.where(x < 0.0, alpha * s * (1.0 - s), beta / (x + 1.0))


def _g_logtail(x, alpha):
    g = torch.ones_like(x)
    g = torch.where(x > 1.0, 1.0 / x, g)
    return torch.where(x <= 0.0, torch.full_like(x, alpha), g)


def _p_pq(x, alpha):
    m0 = (x > (1.0 / alpha)).to(x)
    m1 = (x.abs() <= (1.0 / alpha)).to(x)
    return m0 + m1 * (-(alpha ** 2) / 2 * x.square() * x.sign() + alpha * x + 0.5)


def _p_pexp(x, alpha):
    pos = heaviside(x)
    sgn = pos * 2.0 - 1.0
    return pos - torch.exp(sgn * x * -alpha) / 2.0 * sgn


def _p_nsla(x, alpha):
    sgn = heaviside(x) * 2.0 - 1.0
    return sgn * (alpha * sgn * x + 1).log()


def _p_plr(x, w, c):
    lo, hi = (x < -w).to(x), (x > w).to(x)
    mid = torch.ones_like(x) - lo - hi
    if c == 0:
        return mid * (x / (2 * w) + 0.5) + hi
    cw = c * w
    return lo * (c * x + cw) + hi * (c * x + (1 - cw)) + mid * (x / (2 * w) + 0.5)


def _p_squarewave(x, n, T_period):
    w = math.pi * 2.0 / T_period
    acc = torch.zeros_like(x)
    for i in range(1, int(n)):
        c = 2 * i - 1.0
        acc = acc + torch.sin(c * w * x) / c
    return 0.5 + 2.0 / math.pi * acc


def _p_qps(x, alpha):
    pos = heaviside(x)
    sgn = pos * 2.0 - 1.0
    return pos - sgn * (0.5 * (1.0 + 2.0 / (alpha - 1.0) * x * sgn).pow(1.0 - alpha))


def _p_lkr(x, leak, k):
    m = (x >= 0.0).to(x)
    return (leak * (1.0 - m) + k * m) * x


_ROWS = [
    _Spec(0, "sigmoid", ("alpha",), _g_sigmoid, lambda x, alpha: torch.sigmoid(x * alpha)),
    _Spec(1, "atan", ("alpha",), _g_atan, lambda x, alpha: torch.atan(math.pi / 2 * alpha * x) / math.pi + 0.5),
    _Spec(2, "piecewise_quadratic", ("alpha",), _g_pq, _p_pq),
    _Spec(3, "piecewise_exp", ("alpha",), lambda x, alpha: alpha / 2 * torch.exp(-alpha * x.abs()), _p_pexp),
    _Spec(4, "soft_sign", ("alpha",), lambda x, alpha: 1.0 / (2 * alpha * (1 / alpha + x.abs()).pow(2)),
          lambda x, alpha: (F.softsign(x * alpha) + 1.0) / 2.0),
    _Spec(5, "super_spike", ("alpha",), lambda x, alpha: alpha / (x.abs() + 1.0).pow(2), None),
    _Spec(6, "erf", ("alpha",), lambda x, alpha: torch.exp(-(x * alpha).pow(2)) * (alpha / math.sqrt(math.pi)),
          lambda x, alpha: torch.erfc(-alpha * x) / 2.0),
    _Spec(7, "nonzero_sign_log_abs", ("alpha",), lambda x, alpha: 1.0 / (1 / alpha + x.abs()), _p_nsla),
    _Spec(8, "piecewise_leaky_relu", ("w", "c"),
          lambda x, w, c: torch.where(x.abs() < w, torch.full_like(x, 1 / (2 * w)), torch.full_like(x, c)), _p_plr),
    _Spec(9, "squarewave_fourier_series", ("n", "T_period"), _g_squarewave, _p_squarewave),
    _Spec(10, "s2nn", ("alpha", "beta"), _g_s2nn,
          lambda x, alpha, beta: torch.where(x < 0.0, torch.sigmoid(x * alpha),
                                             beta * torch.log((x + 1.0).abs() + 1e-5) + 0.5)),
    _Spec(11, "q_pseudo_spike", ("alpha",), lambda x, alpha: (1 + 2 / (alpha - 1) * x.abs()).pow(-alpha), _p_qps),
    _Spec(12, "leaky_k_relu", ("leak", "k"),
          lambda x, leak, k: torch.where(x >= 0.0, torch.full_like(x, k), torch.full_like(x, leak)), _p_lkr),
    _Spec(13, "fake_numerical_gradient", ("alpha",),
          lambda x, alpha: torch.clamp_max(((x >= 0.0) * 2.0 - 1.0) / x, alpha), None),
    _Spec(14, "log_tailed_relu", ("alpha",), _g_logtail,
          lambda x, alpha: torch.where(x > 1.0, torch.log(torch.clamp_min(x, 1.0)) + 1.0, F.leaky_relu(x, alpha))),
    _Spec(15, "deterministic_pass", (), lambda x: torch.ones_like(x), lambda x: x),
    _Spec(16, "rect", ("alpha",), lambda x, alpha: alpha * (x.abs() < 0.5 / alpha).to(x),
          lambda x, alpha: torch.clamp(alpha * x + 0.5, min=0.0, max=1.0)),
]
SURROGATES: Dict[str, _Spec] = {r.name: r for r in _ROWS}
_BY_ID = {r.sid: r for r in _ROWS}


class _SpikeFn(torch.autograd.Function):
    """Heaviside forward; backward multiplies by row ``sid``'s derivative."""

    @staticmethod
    def forward(x, sid, p0, p1):
        return heaviside(x)

    @staticmethod
    def setup_context(ctx, inputs, output):
        x, ctx.sid, ctx.p0, ctx.p1 = inputs
        ctx.save_for_backward(x)

    @staticmethod
    def backward(ctx, grad_output):
        (x,) = ctx.saved_tensors
        spec = _BY_ID[ctx.sid]
        args = (ctx.p0, ctx.p1)[: len(spec.params)]
        return grad_output * spec.grad(x, *args), None, None, None


def _spike(name: str, x: torch.Tensor, *params) -> torch.Tensor:
    spec = SURROGATES[name]
    p = tuple(params) + (0.0,) * (2 - len(params))
    return _SpikeFn.apply(x, spec.sid, p[0], p[1])


class SurrogateFunctionBase(nn.Module):
    """``forward(x)`` = Heaviside with a surrogate derivative (``spiking=True``) or
    the smooth primitive (``spiking=False``).  Keyword arguments become attributes
    and are listed in ``_sg_param_names`` (``surrogate.py:327-358``)."""

    _row: Optional[str] = None  # key into SURROGATES for table-driven subclasses

    def __init__(self, spiking: bool = True, **kwargs):
        super().__init__()
        self.spiking = spiking
        self._sg_param_names = tuple(kwargs.keys())
        for k, v in kwargs.items():
            setattr(self, k, v)

    def set_spiking_mode(self, spiking: bool):
        self.spiking = spiking

    @property
    def _sg_params(self) -> dict:
        return {k: getattr(self, k) for k in self._sg_param_names}

    def extra_repr(self):
        return ", ".join([f"{k}={v}" for k, v in self._sg_params.items()] + [f"spiking={self.spiking}"])

    @classmethod
    def spiking_function(cls, x, *args, **kwargs):
        if cls._row is None:
            raise NotImplementedError
        spec = SURROGATES[cls._row]
        vals = list(args) + [kwargs[k] for k in spec.params[len(args):]]
        return _spike(cls._row, x, *vals)

    @classmethod
    def primitive_function(cls, x, *args, **kwargs):
        if cls._row is None or SURROGATES[cls._row].primitive is None:
            raise NotImplementedError
        spec = SURROGATES[cls._row]
        vals = list(args) + [kwargs[k] for k in spec.params[len(args):]]
        return spec.primitive(x, *vals)

    @classmethod
    def backward(cls, grad_output, x, *args, **kwargs):
        """``grad_output * g'(x)`` without autograd (used by hand-written BPTT)."""
        spec = SURROGATES[cls._row]
        vals = list(args) + [kwargs[k] for k in spec.params[len(args):]]
        return grad_output * spec.grad(x, *vals)

    def forward(self, x: torch.Tensor):
        fn = self.spiking_function if self.spiking else self.primitive_function
        return fn(x, **self._sg_params)

    # ---- native-kernel descriptor -------------------------------------------
    def kernel_spec(self) -> Tuple[int, float, float]:
        """``(id, p0, p1)`` understood by the CUDA scan kernels."""
        if self._row is None:
            raise NotImplementedError(f"{type(self).__name__} has no native kernel form")
        spec = SURROGATES[self._row]
        vals = [float(getattr(self, k)) for k in spec.params] + [0.0, 0.0]
        return spec.sid, vals[0], vals[1]

    def cuda_codes(self, y: str, x: str, dtype: str) -> str:
        """CUDA C expression ``y = g'(x)`` for the FlexSN code generator."""
        sid, p0, p1 = self.kernel_spec()
        return f"const float {y} = sjb200::surrogate_grad<{sid}>({x}, {p0!r}f, {p1!r}f);"


def surrogate_spec(sg) -> Optional[Tuple[int, float, float]]:
    """Kernel descriptor of ``sg`` or ``None`` if it must run through PyTorch."""
    if isinstance(sg, SurrogateFunctionBase) and sg.spiking:
        try:
            return sg.kernel_spec()
        except NotImplementedError:
            return None
    return None


def _table_class(name: str, row: str, defaults: Tuple[Tuple[str, float], ...], doc: str, check=None):
    def __init__(self, *args, spiking=True, **kwargs):
        vals = dict(defaults)
        keys = [k for k, _ in defaults]
        if len(args) > len(keys) + 1:
            raise TypeError(f"{name} takes at most {len(keys) + 1} positional arguments")
        for k, a in zip(keys + ["spiking"], args):
            if k == "spiking":
                spiking = a
            else:
                vals[k] = a
        for k, v in kwargs.items():
            if k not in vals:
                raise TypeError(f"{name} got an unexpected keyword argument {k!r}")
            vals[k] = v
        if check is not None:
            check(**vals)
        SurrogateFunctionBase.__init__(self, spiking=spiking, **vals)

    return type(name, (SurrogateFunctionBase,), {"__init__": __init__, "_row": row, "__doc__": doc})


def _pos_alpha(alpha, **_):
    assert alpha > 0, "alpha must be larger than 0"


def _plr_check(w, c):
    assert w > 0.0


def _sq_check(n, T_period):
    assert isinstance(n, int) and T_period > 0.0


PiecewiseQuadratic = _table_class("PiecewiseQuadratic", "piecewise_quadratic", (("alpha", 1.0),),
                                  "g'(x) = max(0, alpha - alpha^2 |x|)  (surrogate.py:401-593)")
PiecewiseExp = _table_class("PiecewiseExp", "piecewise_exp", (("alpha", 1.0),),
                            "g'(x) = alpha/2 * exp(-alpha |x|)  (surrogate.py:595-767)")
Sigmoid = _table_class("Sigmoid", "sigmoid", (("alpha", 4.0),),
                       "g'(x) = alpha * s(alpha x)(1 - s(alpha x))  (surrogate.py:769-934)")
SoftSign = _table_class("SoftSign", "soft_sign", (("alpha", 2.0),),
                        "g'(x) = 1 / (2 alpha (1/alpha + |x|)^2)  (surrogate.py:936-1099)", _pos_alpha)
SuperSpike = _table_class("SuperSpike", "super_spike", (("alpha", 1.0),),
                          "g'(x) = alpha / (|x| + 1)^2  (surrogate.py:1101-1245)")
ATan = _table_class("ATan", "atan", (("alpha", 2.0),),
                    "g'(x) = (alpha/2) / (1 + (pi/2 alpha x)^2)  (surrogate.py:1247-1412)")
NonzeroSignLogAbs = _table_class("NonzeroSignLogAbs", "nonzero_sign_log_abs", (("alpha", 1.0),),
                                 "g'(x) = 1 / (1/alpha + |x|)  (surrogate.py:1415-1608)")
Erf = _table_class("Erf", "erf", (("alpha", 2.0),),
                   "g'(x) = alpha/sqrt(pi) * exp(-(alpha x)^2)  (surrogate.py:1610-1784)")
PiecewiseLeakyReLU = _table_class("PiecewiseLeakyReLU", "piecewise_leaky_relu", (("w", 1.0), ("c", 0.01)),
                                  "g'(x) = 1/(2w) if |x| < w else c  (surrogate.py:1786-2002)", _plr_check)
SquarewaveFourierSeries = _table_class("SquarewaveFourierSeries", "squarewave_fourier_series",
                                       (("n", 2), ("T_period", 8)),
                                       "Fourier-series square wave  (surrogate.py:2004-2131)", _sq_check)
S2NN = _table_class("S2NN", "s2nn", (("alpha", 4.0), ("beta", 1.0)),
                    "sigmoid derivative for x<0, beta/(x+1) otherwise  (surrogate.py:2134-2287)")
QPseudoSpike = _table_class("QPseudoSpike", "q_pseudo_spike", (("alpha", 2.0),),
                            "g'(x) = (1 + 2|x|/(alpha-1))^(-alpha)  (surrogate.py:2289-2428)")
LeakyKReLU = _table_class("LeakyKReLU", "leaky_k_relu", (("leak", 0.0), ("k", 1.0)),
                          "g'(x) = k if x>=0 else leak  (surrogate.py:2430-2650)")
LogTailedReLU = _table_class("LogTailedReLU", "log_tailed_relu", (("alpha", 0.0),),
                             "g'(x) = alpha (x<=0), 1 (0<x<=1), 1/x (x>1)  (surrogate.py:2804-3012)")
Rect = _table_class("Rect", "rect", (("alpha", 1.0),),
                    "g'(x) = alpha * [|x| < 0.5/alpha]  (surrogate.py:3257-3429)")


class FakeNumericalGradient(SurrogateFunctionBase):
    """g'(x) = min(sign(x)/x, alpha); always spiking (``surrogate.py:2652-2801``)."""
    _row = "fake_numerical_gradient"

    def __init__(self, alpha=0.3):
        super().__init__(spiking=True, alpha=alpha)


class DeterministicPass(SurrogateFunctionBase):
    """Heaviside forward, identity backward (``surrogate.py:3015-3104``)."""
    _row = "deterministic_pass"

    def __init__(self, spiking=True):
        super().__init__(spiking=spiking)

    def forward(self, x):
        return _spike("deterministic_pass", x) if self.spiking else x


class _PoissonPassFn(torch.autograd.Function):
    @staticmethod
    def forward(x):
        return torch.bernoulli(x).float()

    @staticmethod
    def setup_context(ctx, inputs, output):
        pass

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output


class PoissonPass(SurrogateFunctionBase):
    """Bernoulli(x) forward, identity backward (``surrogate.py:3164-3254``)."""

    def __init__(self, spiking=True):
        super().__init__(spiking=spiking)

    def forward(self, x):
        return _PoissonPassFn.apply(x) if self.spiking else x

    @staticmethod
    def backward(grad_output, x, alpha=None):
        return grad_output


class MultiLevelSpikeCount(SurrogateFunctionBase):
    """Integer spike counts ``round(clamp(x, 0, D))`` with a pass-through gradient
    inside ``grad_window`` (default ``[0, D]``).  ``surrogate.py:3107-3161``."""

    def __init__(self, max_spike_count: int, spiking: bool = True, grad_window=None):
        if not isinstance(max_spike_count, numbers.Integral) or isinstance(max_spike_count, bool):
            raise TypeError("max_spike_count must be an integer.")
        max_spike_count = int(max_spike_count)
        if max_spike_count < 1:
            raise ValueError("max_spike_count must be >= 1.")
        if grad_window is None:
            lo, hi = 0.0, float(max_spike_count)
        else:
            lo, hi = grad_window
            if lo > hi:
                raise ValueError("grad_window must satisfy grad_min <= grad_max.")
        super().__init__(spiking=spiking, max_spike_count=max_spike_count, grad_min=lo, grad_max=hi)

    @staticmethod
    def spiking_function(x, max_spike_count, grad_min, grad_max):
        from . import quantize
        return quantize.multi_level_spike_count(x, max_spike_count, (grad_min, grad_max))

    @staticmethod
    def primitive_function(x, max_spike_count, grad_min=None, grad_max=None):
        return torch.clamp(x, 0, max_spike_count)


# ---- function-style aliases (``surrogate.atan.apply(x, alpha)`` etc.) ---------
def _fn_alias(row: str):
    """An autograd function per table row: ``forward(x, *params)`` is the Heaviside step, ``backward`` multiplies by the
    row's derivative; one ``None`` comes back for every parameter."""
    spec = SURROGATES[row]

    def forward(x, *params):
        return heaviside(x)

    def setup_context(ctx, inputs, output):
        ctx.save_for_backward(inputs[0])
        ctx.params = tuple(inputs[1:])

    def backward(ctx, grad_output):
        (x,) = ctx.saved_tensors
        return (grad_output * spec.grad(x, *ctx.params[: len(spec.params)]),) + (None,) * len(ctx.params)

    return type(row, (torch.autograd.Function,), {"forward": staticmethod(forward), "setup_context": staticmethod(setup_context),
                                                  "backward": staticmethod(backward), "__doc__": _fn_alias.__doc__})


def _backward_fn(row: _Spec):
    """``<name>_backward(grad_output, x, <params...>) -> (grad_x, None, ...)``; the parameters may be given by position or by the
    row's parameter names (``alpha=...``)."""
    def backward(grad_output, x, *args, **kwargs):
        unknown = set(kwargs) - set(row.params)
        if unknown or len(args) + len(kwargs) > len(row.params):
            raise TypeError(f"{row.name}_backward takes (grad_output, x, {', '.join(row.params)}); got unexpected {sorted(unknown) or 'extra positional arguments'}")
        values = list(args) + [kwargs[n] for n in row.params[len(args):] if n in kwargs]
        if len(values) != len(row.params):
            raise TypeError(f"{row.name}_backward is missing {row.params[len(values):]}")
        return (grad_output * row.grad(x, *values),) + (None,) * len(values)
    backward.__name__ = backward.__qualname__ = row.name + "_backward"
    return backward


for _r in _ROWS:
    globals()[_r.name] = _fn_alias(_r.name)
    globals()[_r.name + "_backward"] = _backward_fn(_r)
poisson_pass = _PoissonPassFn


# ------------------------------------------------------------------ diagnostics
def check_manual_grad(primitive_function, spiking_function, *args, **kwargs) -> float:
    """Largest absolute gap between autograd of the primitive and the hand-written
    derivative on ``x in [-2, 2)``.  Returns the gap (``surrogate.py:63-133``)."""
    x = torch.arange(-2, 2, 32 / 8192).requires_grad_(True)
    primitive_function(x, *args, **kwargs).sum().backward()
    auto = x.grad.clone()
    x.grad.zero_()
    spiking_function(x, *args, **kwargs).sum().backward()
    return float((x.grad - auto).abs().max())


def check_cuda_grad(neu, surrogate_function, device, *args, **kwargs) -> float:
    """Largest gap between the eager and the native-kernel gradient of ``neu`` with
    this surrogate, over fp32 and fp16 (``surrogate.py:136-227``)."""
    worst = 0.0
    for dtype in (torch.float, torch.half):
        net = neu(surrogate_function=surrogate_function(*args, **kwargs), step_mode="m").to(device)
        x = torch.arange(-2, 2, 32 / 8192, device=device, dtype=dtype).requires_grad_(True)
        grads = []
        for backend in ("torch", "cuda"):
            net.backend = backend
            if x.grad is not None:
                x.grad = None
            net(x.unsqueeze(0)).sum().backward()
            grads.append(x.grad.float().clone())
            net.reset()
        worst = max(worst, float((grads[0] - grads[1]).abs().max()))
    return worst


def plot_surrogate_function(surrogate_function, path: Optional[str] = None):
    """Plot Heaviside, primitive and gradient (needs matplotlib; Agg-safe)."""
    import matplotlib
    matplotlib.use("Agg", force=False)
    import matplotlib.pyplot as plt
    fig = plt.figure(dpi=200)
    x = torch.arange(-2.5, 2.5, 0.001)
    plt.plot(x, heaviside(x), label="Heaviside", linestyle="-.")
    was = surrogate_function.spiking
    surrogate_function.set_spiking_mode(False)
    try:
        plt.plot(x, surrogate_function(x).detach(), label="Primitive")
    except NotImplementedError:
        pass
    surrogate_function.set_spiking_mode(True)
    xg = x.clone().requires_grad_(True)
    surrogate_function(xg).sum().backward()
    plt.plot(x, xg.grad, label="Gradient")
    surrogate_function.set_spiking_mode(was)
    plt.xlim(-2, 2)
    plt.legend()
    plt.title(f"{type(surrogate_function).__name__} surrogate function")
    plt.grid(linestyle="--")
    if path is not None:
        fig.savefig(path, bbox_inches="tight")
    return fig
