"""Stateless plasticity rules (STDP family).

Traces: ``tr <- tr - tr/tau + spike`` (STDP) or ``tr <- tr*exp(-1/tau) + spike``
(reward-modulated variants).  Weight update of pair-based STDP:
``dw = -f_pre(w) * sum_b(tr_post (x) s_in) + f_post(w) * sum_b(tr_pre (x) s_out)``.
Parity: ``functional/learning.py:23-602``.
"""
from __future__ import annotations

import math
from typing import Callable, Tuple

import torch
import torch.nn.functional as F

__all__ = ["stdp_linear_step", "mstdp_linear_step", "mstdpet_linear_step", "stdp_conv1d_step",
           "stdp_conv2d_step", "mstdpet_reward_step"]


def _identity(x):
    return x


def _decay_add(trace, tau, spike):
    return trace - trace / tau + spike


def stdp_linear_step(in_spike, out_spike, trace, weight, *, tau_pre, tau_post, f_pre=_identity, f_post=_identity):
    """``in_spike [B, Nin]``, ``out_spike [B, Nout]``, ``weight [Nout, Nin]``."""
    tr_pre = _decay_add(trace[0], tau_pre, in_spike)
    tr_post = _decay_add(trace[1], tau_post, out_spike)
    dw_pre = -f_pre(weight) * torch.einsum("bo,bi->oi", tr_post, in_spike)
    dw_post = f_post(weight) * torch.einsum("bo,bi->oi", out_spike, tr_pre)
    return dw_pre + dw_post, (tr_pre, tr_post)


def mstdp_linear_step(in_spike, out_spike, trace, weight, *, tau_pre, tau_post, f_pre=_identity, f_post=_identity):
    """Per-sample eligibility ``[B, Nout, Nin]`` (not summed over the batch)."""
    tr_pre = trace[0] * math.exp(-1 / tau_pre) + in_spike
    tr_post = trace[1] * math.exp(-1 / tau_post) + out_spike
    elig = (f_post(weight) * (tr_pre.unsqueeze(1) * out_spike.unsqueeze(2))
            - f_pre(weight) * (tr_post.unsqueeze(2) * in_spike.unsqueeze(1)))
    return elig, (tr_pre, tr_post)


def mstdpet_linear_step(in_spike, out_spike, trace, weight, *, tau_pre, tau_post, f_pre=_identity, f_post=_identity):
    """Unbatched eligibility ``[Nout, Nin]`` (``in_spike [Nin]``, ``out_spike [Nout]``)."""
    tr_pre = trace[0] * math.exp(-1 / tau_pre) + in_spike
    tr_post = trace[1] * math.exp(-1 / tau_post) + out_spike
    elig = f_post(weight) * torch.outer(out_spike, tr_pre) - f_pre(weight) * torch.outer(tr_post, in_spike)
    return elig, (tr_pre, tr_post)


def _conv_corr(pre, post, ksize, stride):
    """``sum_{b, out positions} post[b, o, p] * pre[b, i, p*stride + k]`` for every tap ``k``:
    returns ``[O, I, *ksize]``.  ``pre`` is the (already padded) input-side signal."""
    nd = len(ksize)
    if nd == 1:
        pre, post, ksize, stride = pre.unsqueeze(2), post.unsqueeze(2), (1, ksize[0]), (1, stride[0])
    B, I = pre.shape[:2]
    O = post.shape[1]
    cols = F.unfold(pre, kernel_size=ksize, stride=stride)          # [B, I*kh*kw, P]
    P = post.shape[2] * post.shape[3]
    cols = cols[:, :, :P]
    out = torch.einsum("bop,bkp->ok", post.reshape(B, O, P), cols).reshape(O, I, *ksize)
    return out.squeeze(2) if nd == 1 else out


def _stdp_conv(in_spike, out_spike, trace, weight, stride, tau_pre, tau_post, f_pre, f_post):
    tr_pre = _decay_add(trace[0], tau_pre, in_spike)
    tr_post = _decay_add(trace[1], tau_post, out_spike)
    ks = tuple(weight.shape[2:])
    dw = (-f_pre(weight) * _conv_corr(in_spike, tr_post, ks, stride)
          + f_post(weight) * _conv_corr(tr_pre, out_spike, ks, stride))
    return dw, (tr_pre, tr_post)


def stdp_conv2d_step(in_spike, out_spike, trace, weight, *, stride, tau_pre, tau_post, f_pre=_identity,
                     f_post=_identity):
    """``in_spike`` is the padded input ``[B, Cin, H, W]``; ``weight [Cout, Cin, kh, kw]``."""
    return _stdp_conv(in_spike, out_spike, trace, weight, tuple(stride), tau_pre, tau_post, f_pre, f_post)


def stdp_conv1d_step(in_spike, out_spike, trace, weight, *, stride, tau_pre, tau_post, f_pre=_identity,
                     f_post=_identity):
    return _stdp_conv(in_spike, out_spike, trace, weight, tuple(stride), tau_pre, tau_post, f_pre, f_post)


def mstdpet_reward_step(reward, eligibility, trace_e, *, tau_trace):
    """Eligibility trace ``e <- e*exp(-1/tau) + elig/tau``; update is ``reward * e``."""
    trace_e = trace_e * math.exp(-1 / tau_trace) + eligibility / tau_trace
    return reward * trace_e, trace_e
