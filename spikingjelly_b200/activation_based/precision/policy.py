"""Precision policies: how a model is prepared and which autocast context / gradient scaler a training step runs under
(``spikingjelly/activation_based/precision/policy.py:11-96``).

A policy is described by a :class:`PolicyTraits` record (name, autocast dtype, whether fp16-style loss scaling is needed);
the base class derives its context manager, scaler and description from the record, so the concrete fp32 / fp16 / bf16
policies only state their traits.  Policies that rewrite modules (fp8) override :meth:`PrecisionPolicy._convert_modules`."""
from __future__ import annotations

from contextlib import nullcontext
from dataclasses import dataclass
from typing import Optional

import torch

from .capability import build_capability_report, validate_capability
from .convert import ConversionReport, convert_model_for_precision

__all__ = ["PolicyTraits", "PrecisionPolicy", "FP32Policy", "FP16Policy", "BF16Policy"]


@dataclass(frozen=True)
class PolicyTraits:
    name: str
    autocast_dtype: Optional[torch.dtype] = None      # None: run in the parameters' own dtype
    loss_scaling: bool = False                        # a GradScaler guards against fp16 underflow (CUDA only)


class PrecisionPolicy:
    traits = PolicyTraits("fp32")

    def __init__(self, device_type: str = "cuda"):
        self.device_type = device_type
        self._capability: Optional[dict] = None
        self._conversion: Optional[ConversionReport] = None

    # the mode name, as reports and capability checks use it
    @property
    def name(self) -> str:
        return self.traits.name

    # ------------------------------------------------------------------ preparation
    def check_capability(self, model, device) -> None:
        """Record what ``device`` offers for this mode and raise ``RuntimeError`` if it cannot run it."""
        self._capability = build_capability_report(model, device, self.name)
        validate_capability(self._capability)

    def set_capability_report(self, report) -> None:
        """Adopt the findings of another policy (the fp32 fallback keeps the report that explains the fallback)."""
        self._capability = report

    def prepare_model(self, model):
        model, self._conversion = convert_model_for_precision(model, self)
        return model

    def _convert_modules(self, model, report):
        """Hook for module-rewriting policies; the autocast policies leave the model alone."""
        return model

    # ------------------------------------------------------------------ per step
    def autocast_context(self):
        dtype = self.traits.autocast_dtype
        return nullcontext() if dtype is None else torch.amp.autocast(self.device_type, dtype=dtype)

    def create_grad_scaler(self):
        wanted = self.traits.autocast_dtype is not None and self.device_type == "cuda"
        return torch.amp.GradScaler("cuda") if wanted else None

    # ------------------------------------------------------------------ reports
    def describe(self) -> dict:
        dtype = self.traits.autocast_dtype
        info = {"name": self.name, "autocast": dtype is not None, "grad_scaler": dtype is not None and self.device_type == "cuda"}
        if dtype is not None:
            info.update(device_type=self.device_type, dtype=str(dtype))
        return info

    def capability_report(self) -> dict:
        return self._capability if self._capability else {"requested_mode": self.name}

    def conversion_report(self) -> dict:
        return (self._conversion if self._conversion is not None else ConversionReport()).to_dict()


class FP32Policy(PrecisionPolicy):
    traits = PolicyTraits("fp32")

    def __init__(self, device_type: str = "cuda"):
        super().__init__(device_type)


class FP16Policy(PrecisionPolicy):
    traits = PolicyTraits("fp16", torch.float16, loss_scaling=True)


class BF16Policy(PrecisionPolicy):
    # bf16 has fp32's exponent range; the scaler is kept for API symmetry with the fp16 step (it is a no-op in practice)
    traits = PolicyTraits("bf16", torch.bfloat16)
