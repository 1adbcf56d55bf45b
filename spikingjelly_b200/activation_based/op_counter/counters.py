"""The counters: FLOPs, multiply-accumulates, accumulates, synaptic operations, memory traffic.

Conventions (as in ``spikingjelly/activation_based/op_counter/{flop,mac,ac,synop,memory_access}.py``):

* ``FlopCounter``: adds and multiplies separately, a length-k dot product is ``2k - 1`` FLOPs.
* ``MACCounter``: dense multiply-accumulates; a product with a *spike* operand (all 0/1) costs none.
* ``ACCounter``: accumulates; a product with a spike operand costs one accumulate per (spike, fan-out)
  pair — computed exactly by running the operator on the spike tensor against ones.
* ``SynOpCounter``: only those spike-driven accumulates (synaptic operations).
* ``MemoryAccessCounter``: bytes read + written by each operator, assuming no reuse across operators.
"""
from __future__ import annotations

from math import prod
from typing import Any, Callable, Dict, Optional

import torch

from .base import BaseCounter

aten = torch.ops.aten
__all__ = ["FlopCounter", "MACCounter", "ACCounter", "SynOpCounter", "MemoryAccessCounter"]


def _zero(args, kwargs, out):
    return 0


def _no_python_dispatch():
    return torch._C._ExcludeDispatchKeyGuard(torch._C.DispatchKeySet(torch._C.DispatchKey.Python))


def _spike_nnz(x) -> Optional[int]:
    """number of non-zeros if ``x`` is binary, else None"""
    if x is None or not torch.is_tensor(x):
        return None
    if x.dtype == torch.bool:
        return int(x.count_nonzero())
    if not bool(x.eq(0).logical_or_(x.eq(1)).all()):
        return None
    return int(x.count_nonzero())


# ------------------------------------------------------------------------------------- FLOPs
def _mm_dims(x, y, batched):
    if batched:
        b, m, k = x.shape
        bb, kk, n = y.shape
        if b != bb or k != kk:
            raise AssertionError(f"bmm: batch or inner dimensions mismatch [{x.shape} and {y.shape}]")
        return b, m, k, n
    m, k = x.shape
    kk, n = y.shape
    if k != kk:
        raise AssertionError(f"mm: inner dimensions mismatch [{x.shape} and {y.shape}]")
    return 1, m, k, n


def _flop_matmul(batched: bool, has_bias: bool):
    def rule(args, kwargs, out):
        bias, x, y = (args[0], args[1], args[2]) if has_bias else (None, args[0], args[1])
        b, m, k, n = _mm_dims(x, y, batched)
        flops = b * m * n * (2 * k - 1)
        if has_bias:
            alpha, beta = kwargs.get("alpha", 1), kwargs.get("beta", 1)
            if alpha != 1:
                flops += b * m * n
            if beta == 1:
                flops += b * m * n
            elif beta != 0:
                flops += bias.numel() + b * m * n
        return flops
    return rule


def _flop_convolution(args, kwargs, out):
    x, w, bias = args[:3]
    transposed = kwargs.get("transposed", args[6] if len(args) > 6 else False)
    c_out, c_in, *kernel = w.shape
    spatial = x.shape[2:] if transposed else out.shape[2:]
    flops = 2 * c_in * prod(kernel) * prod(spatial) * c_out * x.shape[0] - out.numel()
    return flops + (out.numel() if bias is not None else 0)


def _flop_convolution_backward(args, kwargs, out):
    grad_out, x, w, bias, _s, _p, _d, transposed, _op, _g, mask = args
    flops = 0
    if mask[0]:
        flops += _flop_convolution([grad_out, w, None], {"transposed": not transposed}, out[0])
    if mask[1]:
        px, pw = (grad_out, x) if transposed else (x, grad_out)
        flops += _flop_convolution([px.transpose(0, 1), pw.transpose(0, 1), None], {"transposed": False}, out[1])
    if mask[2] and bias is not None:
        flops += grad_out.shape[1] * (grad_out.shape[0] * prod(grad_out.shape[2:]) - 1)
    return flops


def _flop_add(args, kwargs, out):
    if kwargs.get("alpha", 1.0) == 1.0:
        return out.numel()
    return (args[1].numel() if torch.is_tensor(args[1]) else 1) + out.numel()


def _numel(args, kwargs, out):
    return out.numel()


def _flop_bn(args, kwargs, out):
    x, train = args[0], args[5]
    n, c = x.numel(), x.shape[1]
    affine, running = args[1] is not None, args[3] is not None
    if train:
        return n + (2 * n + 2 * c) + 2 * c + 2 * n + (2 * n if affine else 0) + (6 * c if running else 0)
    return 2 * c + 2 * n + (2 * n if affine else 0)


def _flop_bn_backward(args, kwargs, out):
    g, gamma, train, mask = args[0], args[2], args[-3], args[-1]
    n, c = g.numel(), gamma.numel()
    flops = 0
    if train:
        if mask[0]:
            flops += 2 * n + (n - c) + (2 * n - c) + (5 * n + 2 * c)
        if mask[1] and not mask[0]:
            flops += 2 * n + 2 * n - c
        if mask[2] and not mask[0]:
            flops += n - c
    else:
        flops += (2 * n if mask[0] else 0) + (4 * n - c if mask[1] else 0) + (n - c if mask[2] else 0)
    return flops


def _native_gemm_dims(args):
    a, b, a_mn, b_mn = args[0], args[1], args[2], args[3]
    m, k = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    n = b.shape[1] if b_mn else b.shape[0]
    return m, n, k


def _flop_native_gemm(args, kwargs, out):
    m, n, k = _native_gemm_dims(args)
    return m * n * (2 * k - 1)


def _flop_native_gemm_fp8(args, kwargs, out):
    (m, k), n = args[0].shape, args[1].shape[0]
    return m * n * (2 * k - 1)


def _native(name):
    ns = getattr(torch.ops, "sjb200", None)
    try:
        return getattr(ns, name).default if ns is not None else None
    except (AttributeError, RuntimeError):
        return None


_ELEMENTWISE = [aten.neg.default, aten.neg_.default, aten.mul.Tensor, aten.mul_.Tensor, aten.mul.Scalar, aten.mul_.Scalar,
                aten.div.Tensor, aten.div_.Tensor, aten.div.Scalar, aten.div_.Scalar, aten.eq.Tensor, aten.eq.Scalar, aten.ne.Tensor,
                aten.ne.Scalar, aten.lt.Tensor, aten.lt.Scalar, aten.le.Tensor, aten.le.Scalar, aten.gt.Tensor, aten.gt.Scalar,
                aten.ge.Tensor, aten.ge.Scalar, aten.logical_and.default, aten.logical_or.default, aten.logical_xor.default,
                aten.logical_not.default]
_ADD_LIKE = [aten.add.Tensor, aten.add_.Tensor, aten.add.Scalar, aten.add_.Scalar, aten.sub.Tensor, aten.sub_.Tensor, aten.sub.Scalar,
             aten.sub_.Scalar, aten.rsub.Tensor, aten.rsub.Scalar]
_FREE = [aten.stack.default, aten.clone.default, aten._to_copy.default, aten.full_like.default, aten.ones_like.default,
         aten.view.default, aten.empty.memory_format, aten.select.int, aten.select_backward.default, aten.detach.default,
         aten.t.default, aten.expand.default, aten.max_pool2d_with_indices_backward.default]


class FlopCounter(BaseCounter):
    def default_rules(self):
        rules = {aten.mm.default: _flop_matmul(False, False), aten.addmm.default: _flop_matmul(False, True),
                 aten.bmm.default: _flop_matmul(True, False), aten.baddbmm.default: _flop_matmul(True, True),
                 aten.convolution.default: _flop_convolution, aten.convolution_backward.default: _flop_convolution_backward,
                 aten.native_batch_norm.default: _flop_bn, aten.native_batch_norm_backward.default: _flop_bn_backward,
                 aten.max_pool2d_with_indices.default: lambda a, k, o: o[0].numel() * (prod(a[1]) - 1),
                 aten.avg_pool2d.default: lambda a, k, o: o.numel() * prod(a[1]),
                 aten.sum.default: lambda a, k, o: a[0].numel() - o.numel(), aten.sum.dim_IntList: lambda a, k, o: a[0].numel() - o.numel(),
                 aten.mean.dim: lambda a, k, o: a[0].numel(), aten.sigmoid_.default: lambda a, k, o: 4 * o.numel()}
        rules.update({op: _flop_add for op in _ADD_LIKE})
        rules.update({op: _numel for op in _ELEMENTWISE})
        rules.update({op: _zero for op in _FREE})
        for name, rule in (("gemm_16bit", _flop_native_gemm), ("gemm_fp8", _flop_native_gemm_fp8)):
            op = _native(name)
            if op is not None:
                rules[op] = rule
        return rules


# -------------------------------------------------------------------------------------- MACs
def _mac_matmul(batched: bool, has_bias: bool):
    def rule(args, kwargs, out):
        x, y = (args[1], args[2]) if has_bias else (args[0], args[1])
        if _spike_nnz(x) is not None or _spike_nnz(y) is not None:
            return 0
        b, m, k, n = _mm_dims(x, y, batched)
        return b * m * n * k
    return rule


def _mac_convolution(args, kwargs, out):
    x, w, transposed = args[0], args[1], args[6]
    if _spike_nnz(x) is not None or _spike_nnz(w) is not None:
        return 0
    c_out, c_in, *kernel = w.shape
    return c_in * prod(kernel) * prod(x.shape[2:] if transposed else out.shape[2:]) * c_out * x.shape[0]


def _mac_bn(args, kwargs, out):
    x, train = args[0], args[5]
    return (x.numel() if args[1] is not None else 0) + (2 * x.shape[1] if train and args[3] is not None else 0)


def _mac_native_gemm(args, kwargs, out):
    if _spike_nnz(args[0]) is not None or _spike_nnz(args[1]) is not None:
        return 0
    m, n, k = _native_gemm_dims(args)
    return m * n * k


class MACCounter(BaseCounter):
    def default_rules(self):
        rules = {aten.mm.default: _mac_matmul(False, False), aten.addmm.default: _mac_matmul(False, True),
                 aten.bmm.default: _mac_matmul(True, False), aten.baddbmm.default: _mac_matmul(True, True),
                 aten.convolution.default: _mac_convolution, aten.native_batch_norm.default: _mac_bn}
        op = _native("gemm_16bit")
        if op is not None:
            rules[op] = _mac_native_gemm
        return rules


# ------------------------------------------------------------------------------- ACs and SynOps
def _spike_matmul(batched: bool, has_bias: bool):
    mm = aten.bmm.default if batched else aten.mm.default

    def rule(args, kwargs, out):
        x, y = (args[1], args[2]) if has_bias else (args[0], args[1])
        nx, ny = _spike_nnz(x), _spike_nnz(y)
        if nx is not None and ny is not None:
            with torch.no_grad(), _no_python_dispatch():
                return int(mm(x.double(), y.double()).sum())
        if has_bias and kwargs.get("alpha", 1) != 1:
            return 0
        if nx is not None:
            return nx * y.shape[-1]
        if ny is not None:
            return ny * x.shape[-2]
        return 0
    return rule


def _spike_convolution(args, kwargs, out):
    x, w, _, stride, padding, dilation, transposed, output_padding, groups = args[:9]
    nx, nw = _spike_nnz(x), _spike_nnz(w)
    if nx is not None:
        other = w.double() if nw is not None else torch.ones(w.shape, dtype=torch.float64, device=x.device)
        with torch.no_grad(), _no_python_dispatch():
            return int(aten.convolution.default(x.double(), other, None, stride, padding, dilation, transposed, output_padding, groups).sum())
    if nw is not None:
        ref = x if transposed else out
        return nw * ref.shape[0] * prod(ref.shape[2:])
    return 0


def _spike_native_gemm(args, kwargs, out):
    a, b, a_mn, b_mn = args[:4]
    A = a.t() if a_mn else a
    B = b if b_mn else b.t()
    return _spike_matmul(False, False)((A, B), {}, out)


def _ac_element_wise(args, kwargs, out):
    nx = _spike_nnz(args[0])
    ny = _spike_nnz(args[1]) if len(args) > 1 and torch.is_tensor(args[1]) else None
    return nx + ny if nx is not None and ny is not None else out.numel()


def _ac_bn(args, kwargs, out):
    x, train = args[0], args[5]
    n, c = x.numel(), x.shape[1]
    return (n - c) + n + c + n + (2 * c if args[3] is not None else 0) if train else c + n


def _synop_rules():
    rules = {aten.mm.default: _spike_matmul(False, False), aten.addmm.default: _spike_matmul(False, True),
             aten.bmm.default: _spike_matmul(True, False), aten.baddbmm.default: _spike_matmul(True, True),
             aten.convolution.default: _spike_convolution}
    op = _native("gemm_16bit")
    if op is not None:
        rules[op] = _spike_native_gemm
    return rules


class SynOpCounter(BaseCounter):
    def default_rules(self):
        return _synop_rules()


class ACCounter(BaseCounter):
    def default_rules(self):
        rules = _synop_rules()
        rules.update({aten.native_batch_norm.default: _ac_bn, aten.avg_pool2d.default: lambda a, k, o: o.numel() * (prod(a[1]) - 1),
                      aten.sum.default: lambda a, k, o: a[0].numel() - o.numel(), aten.sum.dim_IntList: lambda a, k, o: a[0].numel() - o.numel(),
                      aten.mean.dim: lambda a, k, o: a[0].numel() - o.numel(), aten.sigmoid_.default: _numel})
        rules.update({op: _ac_element_wise for op in _ADD_LIKE})
        return rules


# ------------------------------------------------------------------------------- memory traffic
def _bytes(x) -> int:
    return int(x.numel() * x.element_size()) if torch.is_tensor(x) else 0


def _io_bytes(args, kwargs, out):
    flat_in = [a for a in args if torch.is_tensor(a)]
    outs = out if isinstance(out, (tuple, list)) else (out,)
    return sum(_bytes(t) for t in flat_in) + sum(_bytes(t) for t in outs)


def _first_and_out(args, kwargs, out):
    return _bytes(args[0]) + _bytes(out)


def _two_and_out(args, kwargs, out):
    return _bytes(args[0]) + _bytes(args[1] if len(args) > 1 else None) + _bytes(out)


def _biased_product_bytes(args, kwargs, out):
    """``beta * bias + a @ b``: the bias is read only when ``beta`` is not zero."""
    return sum(_bytes(t) for t in args[1:3]) + _bytes(out) + (_bytes(args[0]) if kwargs.get("beta", 1.0) != 0 else 0)


def _convolution_bytes(args, kwargs, out):
    return sum(_bytes(t) for t in args[:3]) + _bytes(out)


def _convolution_backward_bytes(args, kwargs, out):
    """The gradient of the output is read once; each requested gradient reads its other operand and writes itself."""
    grad_out, x, w, want = args[0], args[1], args[2], args[10]
    total = _bytes(grad_out)
    if want[0]:
        total += _bytes(w) + _bytes(out[0])
    if want[1]:
        total += _bytes(x) + _bytes(out[1])
    if want[2]:
        total += _bytes(out[2])
    return total


def _batch_norm_bytes(args, kwargs, out):
    """Input, affine pair and running pair are read; training writes the output and the two saved statistics, inference the
    output alone."""
    return sum(_bytes(t) for t in args[:5]) + (sum(_bytes(t) for t in out[:3]) if args[5] else _bytes(out[0]))


def _batch_norm_backward_bytes(args, kwargs, out):
    """Reads only (the rule set counts no writes for this operator).  Training: the first requested gradient decides what is
    read (the input gradient needs everything, the scale gradient everything but the scale, the shift gradient the output
    gradient alone).  Inference: each requested gradient adds the operands the ones before it have not read yet."""
    grad_out, x, gamma, mean, invstd = args[0], args[1], args[2], args[5], args[6]
    train, want = args[-3], args[-1]
    stats = _bytes(x) + _bytes(mean) + _bytes(invstd)
    if train:
        if want[0]:
            return _bytes(grad_out) + stats + _bytes(gamma)
        return _bytes(grad_out) + stats if want[1] else _bytes(grad_out) if want[2] else 0
    total = _bytes(grad_out) + _bytes(invstd) + _bytes(gamma) if want[0] else 0
    if want[1]:
        total += _bytes(x) + _bytes(mean) + (0 if want[0] else _bytes(invstd) + _bytes(grad_out))
    if want[2] and not want[0] and not want[1]:
        total += _bytes(grad_out)
    return total


class MemoryAccessCounter(BaseCounter):
    """Lower bound of the bytes an operator moves: the operands it has to read plus the results it has to write, per operator
    (views and metadata-only operators move nothing; ``full_like`` / ``ones_like`` only write; ``stack`` reads every listed
    tensor).  Same rule set as ``spikingjelly/activation_based/op_counter/memory_access.py:15-411``."""

    def default_rules(self):
        rules = {op: _two_and_out for op in _ADD_LIKE + _ELEMENTWISE + [aten.mm.default, aten.bmm.default]}
        rules.update({op: _first_and_out for op in (aten.neg.default, aten.neg_.default, aten.avg_pool2d.default, aten.sum.default,
                                                    aten.sum.dim_IntList, aten.mean.dim, aten.sigmoid_.default, aten.clone.default,
                                                    aten._to_copy.default, aten.select_backward.default)})
        rules.update({
            aten.addmm.default: _biased_product_bytes, aten.baddbmm.default: _biased_product_bytes,
            aten.convolution.default: _convolution_bytes, aten.convolution_backward.default: _convolution_backward_bytes,
            aten.native_batch_norm.default: _batch_norm_bytes, aten.native_batch_norm_backward.default: _batch_norm_backward_bytes,
            aten.max_pool2d_with_indices.default: lambda a, k, o: _bytes(a[0]) + _bytes(o[0]) + _bytes(o[1]),
            aten.max_pool2d_with_indices_backward.default: _two_and_out,
            aten.stack.default: lambda a, k, o: sum(_bytes(t) for t in a[0]) + _bytes(o),
            aten.full_like.default: lambda a, k, o: _bytes(o), aten.ones_like.default: lambda a, k, o: _bytes(o)})
        rules.update({op: _zero for op in (aten.view.default, aten.empty.memory_format, aten.select.int, aten.detach.default,
                                           aten.t.default, aten.expand.default)})
        for name in ("gemm_16bit", "gemm_fp8", "scan_forward", "scan_backward", "bn_lif_forward", "bn_lif_backward", "ssa_forward",
                     "ssa_backward", "bit_pack", "bit_unpack"):
            op = _native(name)
            if op is not None:
                rules[op] = _io_bytes
        return rules
