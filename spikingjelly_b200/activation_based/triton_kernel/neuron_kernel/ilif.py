"""Functional forms of the integer LIF neuron under the reference's names (``triton_kernel/neuron_kernel/ilif.py:556-700``).
``decay`` is the factor the membrane potential keeps per step (``1 - 1 / tau``); a step emits
``round(clamp(h / v_threshold, 0, max_spike_count))`` spikes and subtracts ``spikes * v_threshold``.  On a CUDA tensor the
sequence runs as the kernel generated from ``functional.ilif_step``; the intermediate ``h_seq`` of the reference's training
form is not materialised (backward recomputes from the stored state sequence), so ``None`` stands in its place."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ... import surrogate

__all__ = ["multistep_ilif_forward_no_grad", "multistep_ilif_forward"]

_NODES: Dict[tuple, object] = {}


def _node(decay: float, v_threshold: float, max_spike_count: int, window, detach_reset: bool, store_v_seq: bool, device):
    from ...neuron import ILIFNode
    if not 0.0 <= decay < 1.0:
        raise ValueError(f"decay must lie in [0, 1), got {decay}")
    key = (float(decay), float(v_threshold), int(max_spike_count), window, bool(detach_reset), bool(store_v_seq), str(device))
    node = _NODES.get(key)
    if node is None:
        sg = surrogate.MultiLevelSpikeCount(int(max_spike_count), grad_window=window)
        node = _NODES[key] = ILIFNode(tau=1.0 / (1.0 - float(decay)), v_threshold=float(v_threshold), surrogate_function=sg,
                                      detach_reset=detach_reset, step_mode="m", backend="cuda" if device.type == "cuda" else "torch",
                                      store_v_seq=store_v_seq)
    return node


def _run(node, x_seq, v_init, store_v_seq: bool):
    node.reset()
    node.v = v_init
    spikes = node(x_seq)
    v_out = node.v_seq if store_v_seq else node.v
    node.reset()
    return spikes, v_out


def multistep_ilif_forward_no_grad(x_seq, v_init, decay: float, v_threshold: float, max_spike_count: int,
                                   store_v_seq: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    with torch.no_grad():
        return _run(_node(decay, v_threshold, max_spike_count, None, False, store_v_seq, x_seq.device), x_seq, v_init, store_v_seq)


def multistep_ilif_forward(x_seq, v_init, decay: float, v_threshold: float, max_spike_count: int, grad_min: float, grad_max: float,
                           detach_reset: bool, store_v_seq: bool) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """Differentiable: the spike count has a pass-through gradient for ``h / v_threshold`` inside ``[grad_min, grad_max]``."""
    node = _node(decay, v_threshold, max_spike_count, (float(grad_min), float(grad_max)), detach_reset, store_v_seq, x_seq.device)
    spikes, v_out = _run(node, x_seq, v_init, store_v_seq)
    return spikes, v_out, None
