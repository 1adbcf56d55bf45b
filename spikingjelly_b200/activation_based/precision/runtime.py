"""Mode name -> policy object.  Parity: ``spikingjelly/activation_based/precision/runtime.py:8-39``."""
from __future__ import annotations

from .capability import _resolve_device_type
from .config import PrecisionConfig
from .policy import BF16Policy, FP16Policy, FP32Policy

__all__ = ["normalize_precision_mode", "resolve_precision_policy"]


def normalize_precision_mode(config) -> str:
    return PrecisionConfig.from_any(config).mode.lower()


def resolve_precision_policy(config):
    cfg = PrecisionConfig.from_any(config)
    mode = cfg.mode.lower()
    device_type = _resolve_device_type(cfg.device or "cuda")
    if mode == "fp32":
        return FP32Policy()
    if mode == "fp16":
        return FP16Policy(device_type=device_type)
    if mode == "bf16":
        return BF16Policy(device_type=device_type)
    if mode in ("fp8", "fp8-torchao", "fp8-te"):
        from . import float8_native as f8
        cls = {"fp8": f8.Float8NativePolicy, "fp8-torchao": f8.Float8TorchAOPolicy, "fp8-te": f8.Float8TransformerEnginePolicy}[mode]
        return cls(device_type=device_type, fp8_recipe=cfg.fp8_recipe)
    raise ValueError(f"Unsupported precision mode {mode!r}. Supported modes in the current stage are: "
                     "fp32, fp16, bf16, fp8, fp8-torchao, fp8-te.")
