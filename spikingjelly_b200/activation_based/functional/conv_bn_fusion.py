"""Graph rewrites of ``Conv -> BatchNorm`` pairs.

* :func:`fuse_conv_bn_eval_modules` folds a frozen BatchNorm into the preceding convolution's
  weights (inference).
* :func:`pack_conv_bn_train_modules` replaces the pair by one module that folds time into the
  batch once, runs conv and BN in single-step mode and unfolds once (training, multi-step).

Both trace the network with ``torch.fx`` (stateful modules, neurons and the step-mode layers are
leaves) and only rewrite a pair when *every* call of the convolution feeds that same BatchNorm and
nothing else reads the convolution's output.

Parity: ``spikingjelly/activation_based/functional/conv_bn_fusion.py:11-330``.
Not imported by ``functional/__init__`` (it depends on ``layer`` and ``neuron``).
"""
from __future__ import annotations

from collections import Counter, defaultdict
from typing import Callable, Dict, List, Tuple

import torch
import torch.nn as nn
from torch import Tensor, fx
from torch.nn.utils.fusion import fuse_conv_bn_eval

from ...logger import logger
from .. import base, layer, neuron

__all__ = ["fuse_conv_bn_eval_modules", "pack_conv_bn_train_modules"]

_PAIRS = [(layer.Conv1d, layer.BatchNorm1d), (layer.Conv2d, layer.BatchNorm2d), (layer.Conv3d, layer.BatchNorm3d),
          (nn.Conv1d, nn.BatchNorm1d), (nn.Conv2d, nn.BatchNorm2d), (nn.Conv3d, nn.BatchNorm3d)]
_STEP_LAYERS = (layer.Conv1d, layer.Conv2d, layer.Conv3d, layer.BatchNorm1d, layer.BatchNorm2d, layer.BatchNorm3d)
_CONV_NDIM = {nn.Conv1d: 3, nn.Conv2d: 4, nn.Conv3d: 5}     # dims of a single-step input


class _TrainConvBnWrapper(nn.Module):
    """conv + bn applied to ``[T, N, ...]`` with ONE fold / unfold of the time dimension."""

    def __init__(self, conv: nn.Module, bn: nn.Module):
        super().__init__()
        self.conv, self.bn = conv, bn

    def _is_sequence(self, x: Tensor) -> bool:
        for cls, nd in _CONV_NDIM.items():
            if isinstance(self.conv, cls):
                return x.dim() == nd + 1
        return False

    def forward(self, x: Tensor) -> Tensor:
        multi = getattr(self.conv, "step_mode", "m") == "m" and getattr(self.bn, "step_mode", "m") == "m"
        if not (multi and self._is_sequence(x)):
            return self.bn(self.conv(x))
        t, n = x.shape[:2]
        saved = [(m, m.step_mode) for m in (self.conv, self.bn) if isinstance(m, base.StepModule)]
        try:
            for m, _ in saved:
                m.step_mode = "s"
            y = self.bn(self.conv(x.flatten(0, 1)))
        finally:
            for m, mode in saved:
                m.step_mode = mode
        return y.reshape(t, n, *y.shape[1:])


class _Tracer(fx.Tracer):
    def is_leaf_module(self, m: nn.Module, qualname: str) -> bool:
        if isinstance(m, (_TrainConvBnWrapper, base.MemoryModule, neuron.BaseNode) + _STEP_LAYERS):
            return True
        return super().is_leaf_module(m, qualname)


def _trace(net: nn.Module) -> Tuple[fx.GraphModule, Dict[str, nn.Module]]:
    tracer = _Tracer()
    gm = fx.GraphModule(tracer.root if hasattr(tracer, "root") else net, tracer.trace(net))
    return gm, dict(gm.named_modules())


def _find_pairs(gm: fx.GraphModule, modules) -> Dict[Tuple[str, str], List[fx.Node]]:
    """(conv target, bn target) -> the bn call nodes, for unambiguous pairs only."""
    calls = Counter(n.target for n in gm.graph.nodes if n.op == "call_module")
    found: Dict[Tuple[str, str], List[fx.Node]] = defaultdict(list)
    partners = defaultdict(set)
    for node in gm.graph.nodes:
        if node.op != "call_module" or not node.args or not isinstance(node.args[0], fx.Node):
            continue
        src = node.args[0]
        if src.op != "call_module" or len(src.users) > 1:
            continue
        conv, bn = modules.get(src.target), modules.get(node.target)
        if any(isinstance(conv, c) and isinstance(bn, b) for c, b in _PAIRS):
            found[(src.target, node.target)].append(node)
            partners[src.target].add(node.target)
    return {pair: nodes for pair, nodes in found.items()
            if len(partners[pair[0]]) == 1 and len(nodes) == calls[pair[0]]}


def _set_module(gm: fx.GraphModule, modules, target: str, new: nn.Module) -> None:
    parent, _, name = target.rpartition(".")
    modules[target] = new
    setattr(modules[parent], name, new)


def _rewrite(net: nn.Module, make: Callable[[str, nn.Module, str, nn.Module], nn.Module], mode: str) -> fx.GraphModule:
    gm, modules = _trace(net)
    pairs = _find_pairs(gm, modules)
    done = skipped = 0
    for (conv_t, bn_t), bn_nodes in pairs.items():
        replacement = make(conv_t, modules[conv_t], bn_t, modules[bn_t])
        if replacement is None:
            skipped += 1
            continue
        _set_module(gm, modules, conv_t, replacement)
        for node in bn_nodes:
            node.replace_all_uses_with(node.args[0])
            gm.graph.erase_node(node)
        done += 1
    gm.graph.lint()
    gm.delete_all_unused_submodules()
    gm.recompile()
    logger.info("conv_bn_transform_summary mode=%s matched_pairs=%s transformed_pairs=%s skipped_step_mode_pairs=%s",
                mode, len(pairs), done, skipped)
    return gm


def fuse_conv_bn_eval_modules(net: nn.Module) -> fx.GraphModule:
    """Fold every eligible BatchNorm into its convolution.  ``net`` must be in ``eval()`` mode and the
    BatchNorms must track running statistics.  Returns a ``GraphModule`` sharing the other submodules."""
    if net.training:
        raise ValueError("fuse_conv_bn_eval_modules only supports eval() models.")

    def make(conv_t, conv, bn_t, bn):
        if getattr(bn, "track_running_stats", True) is False or bn.running_mean is None or bn.running_var is None:
            raise ValueError(f"Cannot fuse {bn_t}: BatchNorm must track running stats.")
        return fuse_conv_bn_eval(conv, bn)

    return _rewrite(net, make, "eval_fuse")


def pack_conv_bn_train_modules(net: nn.Module) -> fx.GraphModule:
    """Pack every eligible pair so that time is folded into the batch once per pair instead of once
    per layer.  ``net`` must be in ``train()`` mode; pairs whose two layers disagree on the step mode
    are left alone."""
    if not net.training:
        raise ValueError("pack_conv_bn_train_modules only supports train() models.")

    def make(conv_t, conv, bn_t, bn):
        if isinstance(conv, _STEP_LAYERS) and isinstance(bn, _STEP_LAYERS) and \
                getattr(conv, "step_mode", None) != getattr(bn, "step_mode", None):
            return None
        return _TrainConvBnWrapper(conv, bn)

    return _rewrite(net, make, "train_pack")
