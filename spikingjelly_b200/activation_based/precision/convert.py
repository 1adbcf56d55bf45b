"""Inventory of the modules a precision policy may replace (``ConversionReport``) and the entry
point that lets a policy do it.  Parity: ``spikingjelly/activation_based/precision/convert.py:12-91``."""
from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import List, Tuple

import torch.nn as nn

from .. import layer
from ..neuron.base_node import BaseNode
from .float8_conv import is_supported_pointwise_conv1d

__all__ = ["ConversionReport", "analyze_convertible_modules", "convert_model_for_precision"]

try:
    from ..neuron.base_node import SimpleBaseNode
except ImportError:                              # the simplified base class is optional
    SimpleBaseNode = BaseNode


@dataclass
class ConversionReport:
    total_modules: int = 0
    convertible_linear: int = 0
    convertible_torch_linear: int = 0
    convertible_pointwise_conv1d: int = 0
    convertible_layer_norm: int = 0
    convertible_modules: List[str] = field(default_factory=list)
    converted_modules: List[str] = field(default_factory=list)
    converted_patterns: List[dict] = field(default_factory=list)
    skipped_modules: List[str] = field(default_factory=list)
    high_precision_modules: List[str] = field(default_factory=list)
    unsupported_modules: List[str] = field(default_factory=list)

    def to_dict(self) -> dict:
        return asdict(self)


_HIGH_PRECISION = (BaseNode, SimpleBaseNode, nn.BatchNorm1d, nn.BatchNorm2d, nn.BatchNorm3d, nn.LayerNorm)
_UNSUPPORTED = (nn.Conv1d, nn.Conv2d, nn.Conv3d, nn.MultiheadAttention)


def analyze_convertible_modules(model: nn.Module, *, include_layer_norm: bool = False) -> ConversionReport:
    """Classify every sub-module: convertible (step-mode Linear, torch Linear, 1x1 Conv1d, optionally
    LayerNorm), high-precision (neurons and normalisation stay in fp32 / bf16) or unsupported."""
    r = ConversionReport()
    for name, m in model.named_modules():
        name = name or "<root>"
        r.total_modules += 1
        if isinstance(m, layer.Linear):
            r.convertible_linear += 1
            r.convertible_modules.append(name)
        elif isinstance(m, nn.Linear):
            r.convertible_torch_linear += 1
            r.convertible_modules.append(name)
        elif is_supported_pointwise_conv1d(m):
            r.convertible_pointwise_conv1d += 1
            r.convertible_modules.append(name)
        elif include_layer_norm and isinstance(m, nn.LayerNorm):
            r.convertible_layer_norm += 1
            r.convertible_modules.append(name)
        elif isinstance(m, _HIGH_PRECISION):
            r.high_precision_modules.append(name)
        elif isinstance(m, _UNSUPPORTED):
            r.unsupported_modules.append(name)
    return r


def convert_model_for_precision(model: nn.Module, policy) -> Tuple[nn.Module, ConversionReport]:
    report = analyze_convertible_modules(model, include_layer_norm=getattr(policy, "supports_layer_norm_conversion", False))
    return policy._convert_modules(model, report), report
