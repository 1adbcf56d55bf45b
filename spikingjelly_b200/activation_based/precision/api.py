"""``prepare_model_for_precision(model, device, config)`` -> :class:`PrecisionArtifacts`, and the JSON reports
(``spikingjelly/activation_based/precision/api.py:23-167``).

The artifacts object is what a training loop holds on to::

    art = prepare_model_for_precision(net, "cuda", "bf16")
    with art.autocast_context():
        loss = criterion(art.model(x), y)
    art.backward(loss, optimizer, clip_grad_norm=1.0)
"""
from __future__ import annotations

import json
import time
import warnings
from contextlib import AbstractContextManager
from dataclasses import asdict, dataclass, replace
from pathlib import Path
from typing import Iterable, Optional, Tuple

import torch

from ...logger import logger
from .config import PrecisionConfig
from .policy import FP32Policy, PrecisionPolicy
from .runtime import resolve_precision_policy

__all__ = ["PrecisionArtifacts", "prepare_model_for_precision", "save_precision_reports"]

#: report file -> key of ``PrecisionArtifacts.describe()`` (plus the derived ``runtime_summary``)
REPORT_FILES = {"precision_policy.json": "policy", "capability_report.json": "capability_report",
                "conversion_report.json": "conversion_report", "precision_runtime.json": "runtime_summary"}


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
        """Backward pass, optional gradient clipping and optional optimizer step, identical for scaled (fp16) and
        unscaled runs.  Returns the total gradient norm if clipping was asked for, else ``None``."""
        scaled = self.scaler is not None
        if scaled and clip_grad_norm is not None and not step_optimizer:
            # unscale_ may run only once per optimizer step; without the step the next call would unscale twice
            raise ValueError("clipping needs unscaled gradients, and with a gradient scaler those exist only inside an optimizer "
                             "step: pass step_optimizer=True or clip yourself")
        (self.scaler.scale(loss) if scaled else loss).backward()
        total_norm = None
        if clip_grad_norm is not None:
            if scaled:
                self.scaler.unscale_(optimizer)
            over = self.model.parameters() if parameters is None else parameters
            total_norm = float(torch.nn.utils.clip_grad_norm_(over, clip_grad_norm))
        if step_optimizer:
            if scaled:
                self.scaler.step(optimizer)
                self.scaler.update()
            else:
                optimizer.step()
        return total_norm

    def describe(self) -> dict:
        return {"requested_config": asdict(self.requested_config), "effective_config": asdict(self.effective_config),
                "policy": self.policy.describe(), "capability_report": self.policy.capability_report(),
                "conversion_report": self.policy.conversion_report(), "fallback_reason": self.fallback_reason}


def _usable_policy(requested: PrecisionConfig, model, device) -> Tuple[PrecisionPolicy, Optional[str]]:
    """The policy for ``requested`` if ``device`` can run it, else (unless strict) the fp32 policy and the reason."""
    policy = resolve_precision_policy(requested)
    try:
        policy.check_capability(model, device)
        return policy, None
    except RuntimeError as problem:
        if requested.strictness == "strict":
            raise
        reason = str(problem)
    if requested.strictness == "warn":
        warnings.warn(f"precision {requested.mode!r} cannot run here, falling back to fp32: {reason}", RuntimeWarning, stacklevel=3)
    plain = FP32Policy()
    plain.set_capability_report(policy.capability_report())
    return plain, reason


def prepare_model_for_precision(model: torch.nn.Module, device, config) -> PrecisionArtifacts:
    """Pick the policy for ``config`` (a mode string, a dict or a :class:`PrecisionConfig`), verify that ``device`` can run
    it — ``strictness="strict"`` raises otherwise, ``"warn"`` / ``"silent"`` continue in fp32 — convert the model's modules
    where the policy asks for it and create the gradient scaler."""
    started = time.perf_counter()
    device = torch.device(device)
    requested = PrecisionConfig.from_any(config, default_device=str(device))
    policy, reason = _usable_policy(requested, model, device)
    prepared = policy.prepare_model(model)
    effective = requested if reason is None else replace(requested, mode="fp32")
    artifacts = PrecisionArtifacts(requested, effective, policy, prepared, policy.create_grad_scaler(), reason)
    report = policy.conversion_report()
    logger.info("precision: asked for %s, running %s on %s (%d module(s) converted, %d left unsupported, scaler=%s, %.1f ms)%s",
                requested.mode, effective.mode, device, len(report.get("converted_modules", ())),
                len(report.get("unsupported_modules", ())), artifacts.scaler is not None, (time.perf_counter() - started) * 1e3,
                "" if reason is None else f"; fallback because: {reason}")
    return artifacts


def save_precision_reports(artifacts: PrecisionArtifacts, output_dir: str) -> None:
    """Write ``precision_policy.json``, ``capability_report.json``, ``conversion_report.json`` and
    ``precision_runtime.json`` into ``output_dir`` (created if missing)."""
    facts = artifacts.describe()
    facts["runtime_summary"] = {key: facts[key] for key in ("requested_config", "effective_config", "fallback_reason")}
    target = Path(output_dir)
    target.mkdir(parents=True, exist_ok=True)
    for filename, key in REPORT_FILES.items():
        (target / filename).write_text(json.dumps(facts[key], indent=2, sort_keys=True), encoding="utf-8")
    logger.info("precision reports written to %s: %s", target, ", ".join(REPORT_FILES))
