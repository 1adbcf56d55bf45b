"""``PrecisionConfig``: what a user asks for (mode, strictness, fp8 recipe, device).
Parity: ``spikingjelly/activation_based/precision/config.py:7-46``."""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Optional

__all__ = ["PrecisionConfig"]


@dataclass(frozen=True)
class PrecisionConfig:
    mode: str = "fp32"          # fp32 | fp16 | bf16 | fp8 (aliases: fp8-torchao, fp8-te)
    strictness: str = "warn"    # strict: raise if unavailable; warn / silent: fall back to fp32
    fp8_recipe: str = "auto"    # auto | current | delayed | block | mxfp8 (native backend: "delayed" and "current"; the other names resolve to "delayed")
    device: Optional[str] = None

    def __post_init__(self):
        object.__setattr__(self, "mode", "fp32" if self.mode is None else str(self.mode).lower())
        if self.device is not None and not isinstance(self.device, str):
            object.__setattr__(self, "device", str(self.device))

    @classmethod
    def from_any(cls, config, default_device: Optional[str] = None) -> "PrecisionConfig":
        if config is None:
            return cls(device=default_device)
        if isinstance(config, cls):
            return dataclasses.replace(config, device=default_device) if config.device is None and default_device is not None else config
        if isinstance(config, str):
            return cls(mode=config.lower(), device=default_device)
        if isinstance(config, dict):
            data = dict(config)
            data["device"] = default_device if "device" not in data else (None if data["device"] is None else str(data["device"]))
            return cls(**data)
        raise TypeError("PrecisionConfig.from_any() expects None, a PrecisionConfig, str, or dict.")
