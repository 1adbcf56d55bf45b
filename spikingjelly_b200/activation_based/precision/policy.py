"""Precision policies: how a model is prepared, which autocast context and gradient scaler a
training step uses.  Parity: ``spikingjelly/activation_based/precision/policy.py:11-96``."""
from __future__ import annotations

from contextlib import nullcontext

import torch

from .capability import build_capability_report, validate_capability
from .convert import ConversionReport, convert_model_for_precision

__all__ = ["PrecisionPolicy", "FP32Policy", "FP16Policy", "BF16Policy"]


class PrecisionPolicy:
    name = "fp32"

    def __init__(self):
        self._capability_report = None
        self._conversion_report = None

    def set_capability_report(self, report) -> None:
        self._capability_report = report

    def check_capability(self, model, device) -> None:
        self._capability_report = build_capability_report(model, device, self.name)
        validate_capability(self._capability_report)

    def prepare_model(self, model):
        model, self._conversion_report = convert_model_for_precision(model, self)
        return model

    def _convert_modules(self, model, report):
        return model

    def autocast_context(self):
        return nullcontext()

    def create_grad_scaler(self):
        return None

    def describe(self) -> dict:
        return {"name": self.name, "autocast": False, "grad_scaler": False}

    def capability_report(self) -> dict:
        return self._capability_report or {"requested_mode": self.name}

    def conversion_report(self) -> dict:
        return (self._conversion_report or ConversionReport()).to_dict()


class FP32Policy(PrecisionPolicy):
    name = "fp32"


class _AutocastPolicy(PrecisionPolicy):
    amp_dtype: torch.dtype
    needs_scaler = False

    def __init__(self, device_type: str = "cuda"):
        super().__init__()
        self.device_type = device_type

    def autocast_context(self):
        return torch.amp.autocast(self.device_type, dtype=self.amp_dtype)

    def create_grad_scaler(self):
        return torch.amp.GradScaler("cuda") if self.device_type == "cuda" else None

    def describe(self) -> dict:
        return {"name": self.name, "autocast": True, "device_type": self.device_type, "dtype": str(self.amp_dtype),
                "grad_scaler": self.device_type == "cuda"}


class FP16Policy(_AutocastPolicy):
    name = "fp16"
    amp_dtype = torch.float16


class BF16Policy(_AutocastPolicy):
    name = "bf16"
    amp_dtype = torch.bfloat16
