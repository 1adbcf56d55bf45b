"""Functional forms of the SpikeZIP ternary IF neuron under the reference's names (``triton_kernel/neuron_kernel/stbif.py:196-440``):
gradient-free state transitions ``(x, q, acc_q) -> (out, q, acc_q, cur_output, work_flag)``.  The multi-step form runs the
kernel the FlexSN generator makes from ``functional.stbif_step`` (one launch for the whole sequence, the work flag kept as a
register state); CPU tensors take the eager loop."""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ... import functional

__all__ = ["single_step_stbif", "multi_step_stbif"]

_NODES: Dict[tuple, object] = {}


def _scalar(t) -> float:
    return float(t.reshape(-1)[0]) if torch.is_tensor(t) else float(t)


def _check(x, q, acc_q):
    if not (x.shape[-q.dim():] == q.shape == acc_q.shape) or not (x.dtype == q.dtype == acc_q.dtype) or not (x.device == q.device == acc_q.device):
        raise ValueError("x, q and acc_q must share shape (per step), dtype and device.")


def single_step_stbif(x, q, acc_q, q_threshold, pos_max, neg_min) -> Tuple[torch.Tensor, ...]:
    _check(x, q, acc_q)
    with torch.no_grad():
        out, q, acc, cur = functional.stbif_step(x, q, acc_q, q_threshold, pos_max, neg_min)
        return out, q, acc, cur, ((x != 0).any() | (out != 0).any()).reshape(1)


def multi_step_stbif(x_seq, q, acc_q, q_threshold, pos_max, neg_min) -> Tuple[torch.Tensor, ...]:
    _check(x_seq, q, acc_q)
    with torch.no_grad():
        if x_seq.is_cuda and x_seq.shape[0] > 0:
            from ...neuron.conversion import STBIFNeuron
            key = (_scalar(q_threshold), _scalar(pos_max), _scalar(neg_min))
            node = _NODES.get(key)
            if node is None:                        # one module per parameter set keeps its compiled kernel alive
                node = _NODES[key] = STBIFNeuron(key[0], level=2, pos_max=key[1], neg_min=key[2], step_mode="m").to(x_seq.device)
            res = node._compiled_run(x_seq.contiguous(), q.contiguous(), acc_q.contiguous(), torch.zeros_like(q))
            if res is not None:
                out_seq, (q, acc, cur), flag = res
                return out_seq, q, acc, cur, flag.reshape(1)
        outs, cur = [], torch.zeros_like(q)
        acc = acc_q
        for x in x_seq:
            o, q, acc, cur = functional.stbif_step(x, q, acc, q_threshold, pos_max, neg_min)
            outs.append(o)
        out_seq = torch.stack(outs) if outs else x_seq.clone()
        return out_seq, q, acc, cur, ((x_seq != 0).any() | (out_seq != 0).any()).reshape(1)
