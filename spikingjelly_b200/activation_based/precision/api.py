"""``prepare_model_for_precision(model, device, config)`` -> ``PrecisionArtifacts`` (prepared model,
policy, optional gradient scaler, fallback information) and the JSON reports.
Parity: ``spikingjelly/activation_based/precision/api.py:23-167``."""
from __future__ import annotations

import json
import os
import time
import warnings
from contextlib import AbstractContextManager
from dataclasses import asdict, dataclass, replace
from typing import Iterable, Optional

import torch

from ...logger import logger
from .config import PrecisionConfig
from .policy import FP32Policy, PrecisionPolicy
from .runtime import resolve_precision_policy

__all__ = ["PrecisionArtifacts", "prepare_model_for_precision", "save_precision_reports"]


@dataclass
class PrecisionArtifacts:
    requested_config: PrecisionConfig
    effective_config: PrecisionConfig
    policy: PrecisionPolicy
    model: torch.nn.Module
    scaler: Optional[torch.amp.GradScaler] = None
    fallback_reason: Optional[str] = None

    def autocast_context(self) -> AbstractContextManager:
        return self.policy.autocast_context()

    def backward(self, loss: torch.Tensor, optimizer: torch.optim.Optimizer, clip_grad_norm: Optional[float] = None,
                 parameters: Optional[Iterable[torch.nn.Parameter]] = None, step_optimizer: bool = True) -> Optional[float]:
        """backward (+ unscale / clip) (+ optimizer step), with or without a gradient scaler.
        Returns the total gradient norm when clipping was requested."""
        if clip_grad_norm is not None and parameters is None:
            parameters = self.model.parameters()
        norm = None
        if self.scaler is None:
            loss.backward()
            if clip_grad_norm is not None:
                norm = torch.nn.utils.clip_grad_norm_(parameters, clip_grad_norm)
            if step_optimizer:
                optimizer.step()
        else:
            self.scaler.scale(loss).backward()
            if clip_grad_norm is not None:
                if not step_optimizer:
                    raise ValueError("clip_grad_norm with step_optimizer=False is not supported when a grad scaler is active.")
                self.scaler.unscale_(optimizer)
                norm = torch.nn.utils.clip_grad_norm_(parameters, clip_grad_norm)
            if step_optimizer:
                self.scaler.step(optimizer)
                self.scaler.update()
        return float(norm) if norm is not None else None

    def describe(self) -> dict:
        return {"requested_config": asdict(self.requested_config), "effective_config": asdict(self.effective_config),
                "policy": self.policy.describe(), "capability_report": self.policy.capability_report(),
                "conversion_report": self.policy.conversion_report(), "fallback_reason": self.fallback_reason}


def prepare_model_for_precision(model: torch.nn.Module, device, config) -> PrecisionArtifacts:
    """Resolve the policy for ``config``, check that ``device`` can run it (``strictness``: ``"strict"``
    raises, ``"warn"`` / ``"silent"`` fall back to fp32), convert the model and create the scaler."""
    t0 = time.perf_counter()
    device = torch.device(device)
    requested = PrecisionConfig.from_any(config, default_device=str(device))
    policy = resolve_precision_policy(requested)
    fallback = None
    try:
        policy.check_capability(model, device)
    except RuntimeError as exc:
        if requested.strictness == "strict":
            raise
        fallback = str(exc)
        if requested.strictness == "warn":
            warnings.warn(f"precision={requested.mode!r} is falling back to fp32: {fallback}", RuntimeWarning, stacklevel=2)
        fp32 = FP32Policy()
        fp32.set_capability_report(policy.capability_report())
        policy = fp32
    prepared = policy.prepare_model(model)
    effective = requested if fallback is None else replace(requested, mode="fp32")
    art = PrecisionArtifacts(requested, effective, policy, prepared, policy.create_grad_scaler(), fallback)
    conv = policy.conversion_report()
    logger.info("precision_prepare_summary requested_mode=%s effective_mode=%s device=%s fallback=%s fallback_reason=%s "
                "converted_modules=%s unsupported_modules=%s grad_scaler=%s elapsed_ms=%.3f", requested.mode, effective.mode,
                device, fallback is not None, fallback, len(conv.get("converted_modules", ())),
                len(conv.get("unsupported_modules", ())), art.scaler is not None, (time.perf_counter() - t0) * 1e3)
    return art


def save_precision_reports(artifacts: PrecisionArtifacts, output_dir: str) -> None:
    """Writes precision_policy.json, capability_report.json, conversion_report.json, precision_runtime.json."""
    os.makedirs(output_dir, exist_ok=True)
    payload = artifacts.describe()
    payload["runtime_summary"] = {k: payload[k] for k in ("requested_config", "effective_config", "fallback_reason")}
    files = (("precision_policy.json", "policy"), ("capability_report.json", "capability_report"),
             ("conversion_report.json", "conversion_report"), ("precision_runtime.json", "runtime_summary"))
    for filename, key in files:
        with open(os.path.join(output_dir, filename), "w", encoding="utf-8") as f:
            json.dump(payload[key], f, indent=2, sort_keys=True)
    logger.info("precision_reports_saved output_dir=%s files=%s", output_dir, tuple(n for n, _ in files))
