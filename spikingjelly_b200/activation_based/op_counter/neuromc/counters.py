"""Primitive-operation counters of the NeuroMC model: additions, multiplications, comparisons, multiplexer selections and
square roots executed by the ATen operators of a run, per stage (forward / backward / optimizer) and per operator
(``op_counter/neuromc/{base,add,mul,cmp,mux,sqrt}_counter.py`` of the reference).

Conventions.  A product with a binary (0 / 1) operand needs no multiplier: its multiplications count as zero and its
additions are the accumulations that really happen (``max(nnz - 1, 0)`` per output, obtained by running the same
contraction on the 0 / 1 pattern).  A dense contraction of depth ``k`` costs ``k`` multiplications and ``k - 1``
additions per output (+ 1 with a bias / ``beta`` term).  Batch norm in training mode: mean, variance, normalisation, the
affine map and the running-statistics update are counted separately so that disabling one of them shows."""
from __future__ import annotations

from collections import defaultdict
from math import prod
from typing import Any, Callable, Dict, Optional

import torch
from torch.overrides import resolve_name

from ..base import BaseCounter, _infer_stage

aten = torch.ops.aten

__all__ = ["NeuroMCBaseCounter", "NeuroMCAddCounter", "NeuroMCMulCounter", "NeuroMCCmpCounter", "NeuroMCMuxCounter", "NeuroMCSqrtCounter",
           "is_spike", "spike_nnz"]


def is_spike(x) -> bool:
    if not torch.is_tensor(x):
        return False
    if x.dtype == torch.bool:
        return True
    return x.numel() > 0 and bool(((x == 0) | (x == 1)).all())


def spike_nnz(x) -> Optional[int]:
    return int(x.count_nonzero()) if is_spike(x) else None


def _plain(fn, *tensors, **kw):
    """Run an ATen function outside the counting dispatch mode, in float64."""
    with torch.no_grad(), torch._C._ExcludeDispatchKeyGuard(torch._C.DispatchKeySet(torch._C.DispatchKey.Python)):
        return fn(*[t.double() if torch.is_tensor(t) else t for t in tensors], **kw)


def _accumulations(counts: torch.Tensor) -> int:
    return int((counts - 1.0).clamp_min(0.0).sum())


class NeuroMCBaseCounter(BaseCounter):
    """Books every counted value three ways: per stage, per operator name, and per (stage, operator)."""

    def __init__(self, extra_rules: Optional[Dict[Any, Callable]] = None, extra_ignore_modules: Optional[list] = None):
        super().__init__()
        self.rules.update(extra_rules or {})
        self.ignore_modules.extend(extra_ignore_modules or [])
        self.stage_records: Dict[str, int] = defaultdict(int)
        self.op_records: Dict[str, int] = defaultdict(int)
        self.stage_op_records: Dict[str, Dict[str, int]] = defaultdict(lambda: defaultdict(int))

    def count(self, func, args: tuple, kwargs: dict, out, active_modules=None, parent_names=None) -> int:
        rule = self.rules.get(func)
        if rule is None:
            return 0
        value, name, stage = int(rule(args, kwargs, out)), resolve_name(func), _infer_stage(func, args, kwargs, out)
        self.stage_records[stage] += value
        self.op_records[name] += value
        self.stage_op_records[stage][name] += value
        return value

    def get_stage_counts(self) -> Dict[str, int]:
        return dict(self.stage_records)

    def get_op_counts(self) -> Dict[str, int]:
        return dict(self.op_records)

    def get_stage_op_counts(self) -> Dict[str, Dict[str, int]]:
        return {k: dict(v) for k, v in self.stage_op_records.items()}

    def reset(self) -> None:
        super().reset()
        self.stage_records.clear()
        self.op_records.clear()
        self.stage_op_records.clear()


# ---------------------------------------------------------------------------------------------------------------------
# contractions
# ---------------------------------------------------------------------------------------------------------------------
def _matmul_adds(x, y, batched: bool) -> int:
    op = aten.bmm.default if batched else aten.mm.default
    sx, sy = is_spike(x), is_spike(y)
    if sx and sy:
        return _accumulations(_plain(op, x, y))
    if sx:
        return _accumulations(_plain(lambda t: t.sum(-1), x)) * y.shape[-1]
    if sy:
        return _accumulations(_plain(lambda t: t.sum(-2), y)) * x.shape[-2]
    return int(prod(x.shape[:-1]) * y.shape[-1] * max(x.shape[-1] - 1, 0))


def _matmul_muls(x, y) -> int:
    return 0 if is_spike(x) or is_spike(y) else int(prod(x.shape[:-1]) * y.shape[-1] * x.shape[-1])


def _conv_depth(x, w, groups) -> int:
    return x.shape[1] // groups * prod(w.shape[2:])


def _conv_adds(args, kwargs, out) -> int:
    x, w, bias, stride, padding, dilation, transposed, output_padding, groups = args[:9]
    if is_spike(x):
        pattern = w if is_spike(w) else torch.ones_like(w)
        hits = _plain(aten.convolution.default, x, pattern, None, stride, padding, dilation, transposed, output_padding, groups)
        return _accumulations(hits) + (out.numel() if bias is not None else 0)
    if is_spike(w):
        ref = x if transposed else out
        return int(w.count_nonzero()) * ref.shape[0] * prod(ref.shape[2:])
    return out.numel() * max(_conv_depth(x, w, groups) - 1, 0) + (out.numel() if bias is not None else 0)


def _conv_muls(args, kwargs, out) -> int:
    x, w, groups = args[0], args[1], args[8]
    return 0 if is_spike(x) or is_spike(w) else out.numel() * _conv_depth(x, w, groups)


def _conv_backward(adds: bool):
    def rule(args, kwargs, out):
        grad_out, x, w = args[:3]
        groups, mask = args[9], args[10]
        total = 0
        if mask[0]:                                   # data gradient: every input element gathers C_out/groups x taps products
            depth = w.shape[0] // groups * prod(w.shape[2:])
            total += out[0].numel() * (max(depth - 1, 0) if adds else depth)
        if mask[1]:                                   # weight gradient: every weight gathers batch x output positions products
            depth = grad_out.shape[0] * prod(grad_out.shape[2:])
            if is_spike(x):
                total += 0 if not adds else out[1].numel() * max(depth - 1, 0)
            else:
                total += out[1].numel() * (max(depth - 1, 0) if adds else depth)
        if adds and mask[2] and len(out) > 2 and torch.is_tensor(out[2]):
            total += grad_out.shape[1] * (grad_out.shape[0] * prod(grad_out.shape[2:]) - 1)
        return int(total)
    return rule


def _numel(args, kwargs, out) -> int:
    return int(out.numel()) if torch.is_tensor(out) else 0


def _scaled_add(adds: bool):
    def rule(args, kwargs, out):
        if adds:
            return int(out.numel())
        return 0 if kwargs.get("alpha", 1) == 1 else int(out.numel())
    return rule


def _reduction_adds(args, kwargs, out) -> int:
    x = args[0]
    groups = out.numel() if torch.is_tensor(out) else 1
    return int(max(x.numel() - groups, 0))


def _bn(adds: bool):
    def rule(args, kwargs, out):
        x, weight, running, train = args[0], args[1], args[3], args[5]
        n, c = x.numel(), x.shape[1]
        if not train:
            return int(n + (n if weight is not None else 0))         # (x - mean) * invstd [* w + b]
        if adds:          # mean, centring, variance, eps, shift; running statistics 2 per channel
            return int((n - c) + n + (n - c) + c + (n if weight is not None else 0) + (2 * c if running is not None else 0))
        return int(n + c + n + (n if weight is not None else 0) + (2 * c if running is not None else 0))   # squares, 1/n, scale, affine, momentum
    return rule


def _bn_backward(adds: bool):
    def rule(args, kwargs, out):
        n, train, mask = args[0].numel(), args[-3], args[-1]
        per_input = (4 if adds else 5) if train else (0 if adds else 2)
        return int((per_input * n if mask[0] else 0) + (n if mask[1] else 0) + (n if adds and mask[2] else 0))
    return rule


def _max_pool_cmps(args, kwargs, out) -> int:
    kernel = args[1]
    k = prod(kernel) if isinstance(kernel, (tuple, list)) else int(kernel) ** 2
    return int(out[0].numel() * max(k - 1, 0))


_ELEMENT_WISE_ADD = (aten.add.Tensor, aten.add_.Tensor, aten.add.Scalar, aten.add_.Scalar, aten.sub.Tensor, aten.sub_.Tensor, aten.sub.Scalar,
                     aten.sub_.Scalar, aten.rsub.Tensor, aten.rsub.Scalar)
_ELEMENT_WISE_MUL = (aten.mul.Tensor, aten.mul_.Tensor, aten.mul.Scalar, aten.mul_.Scalar, aten.div.Tensor, aten.div_.Tensor, aten.div.Scalar,
                     aten.div_.Scalar)
_COMPARISONS = (aten.eq.Tensor, aten.eq.Scalar, aten.ne.Tensor, aten.ne.Scalar, aten.lt.Tensor, aten.lt.Scalar, aten.le.Tensor, aten.le.Scalar,
                aten.gt.Tensor, aten.gt.Scalar, aten.ge.Tensor, aten.ge.Scalar, aten.logical_and.default, aten.logical_or.default,
                aten.logical_xor.default, aten.logical_not.default)


def _with_beta(rule, adds: bool):
    def wrapped(args, kwargs, out):
        value = rule(args[1:3], kwargs, out)
        if adds:
            return value + (out.numel() if kwargs.get("beta", 1) != 0 else 0)
        return value + (out.numel() if kwargs.get("alpha", 1) != 1 else 0) + (out.numel() if kwargs.get("beta", 1) not in (0, 1) else 0)
    return wrapped


class NeuroMCAddCounter(NeuroMCBaseCounter):
    def default_rules(self):
        mm = lambda a, k, o: _matmul_adds(a[0], a[1], False)
        bmm = lambda a, k, o: _matmul_adds(a[0], a[1], True)
        rules = {aten.mm.default: mm, aten.bmm.default: bmm, aten.addmm.default: _with_beta(mm, True), aten.baddbmm.default: _with_beta(bmm, True),
                 aten.convolution.default: _conv_adds, aten.convolution_backward.default: _conv_backward(True),
                 aten.native_batch_norm.default: _bn(True), aten.native_batch_norm_backward.default: _bn_backward(True),
                 aten.sum.default: _reduction_adds, aten.sum.dim_IntList: _reduction_adds, aten.mean.dim: _reduction_adds}
        rules.update({op: _scaled_add(True) for op in _ELEMENT_WISE_ADD})
        return rules


class NeuroMCMulCounter(NeuroMCBaseCounter):
    def default_rules(self):
        mm = lambda a, k, o: _matmul_muls(a[0], a[1])
        rules = {aten.mm.default: mm, aten.bmm.default: mm, aten.addmm.default: _with_beta(mm, False), aten.baddbmm.default: _with_beta(mm, False),
                 aten.convolution.default: _conv_muls, aten.convolution_backward.default: _conv_backward(False),
                 aten.native_batch_norm.default: _bn(False), aten.native_batch_norm_backward.default: _bn_backward(False)}
        rules.update({op: _numel for op in _ELEMENT_WISE_MUL})
        rules.update({op: _scaled_add(False) for op in _ELEMENT_WISE_ADD})
        return rules


class NeuroMCCmpCounter(NeuroMCBaseCounter):
    def default_rules(self):
        rules = {op: _numel for op in _COMPARISONS}
        rules[aten.max_pool2d_with_indices.default] = _max_pool_cmps
        return rules


class NeuroMCMuxCounter(NeuroMCBaseCounter):
    def default_rules(self):
        return {aten.where.self: _numel, aten.where.ScalarOther: _numel, aten.where.ScalarSelf: _numel}


class NeuroMCSqrtCounter(NeuroMCBaseCounter):
    def default_rules(self):
        bn = lambda a, k, o: int(a[0].shape[1]) if a[5] else 0          # one inverse standard deviation per channel
        return {aten.sqrt.default: _numel, aten.sqrt_.default: _numel, aten.rsqrt.default: _numel, aten.native_batch_norm.default: bn}
