"""What the machine can do for a requested precision mode, as a plain dict, and its validation.

fp8 here means the package's own tensor-core kernels (``ops/csrc/gemm_tcgen05.cu``, ``kind::f8f6f4``):
it needs a CUDA device of compute capability 10.x and the compiled library.  The torchao /
Transformer-Engine fields of the reference's report are kept (always reporting "not used") so that
tooling that reads the report keeps working.

Parity: ``spikingjelly/activation_based/precision/capability.py:120-373``.
"""
from __future__ import annotations

from typing import Any, Dict

import torch

__all__ = ["build_capability_report", "validate_capability"]

FP8_MODES = ("fp8", "fp8-torchao", "fp8-te")


def _resolve_device_type(device) -> str:
    s = str(device)
    return "cuda" if s.startswith("cuda") else ("mps" if s.startswith("mps") else "cpu")


def _module_available(name: str) -> bool:
    import importlib.util
    try:
        return importlib.util.find_spec(name) is not None
    except (ImportError, ValueError):
        return False


def _native_library_available() -> bool:
    try:
        from ... import ops
        return bool(ops.available())
    except Exception:
        return False


def build_capability_report(model, device, mode: str) -> Dict[str, Any]:
    device = torch.device(device)
    dtype_ = _resolve_device_type(device)
    cuda_ok = torch.cuda.is_available()
    capability = tuple(torch.cuda.get_device_capability(device)) if dtype_ == "cuda" and cuda_ok else None
    mps = getattr(torch.backends, "mps", None)
    mps_available = bool(mps is not None and mps.is_available())
    if dtype_ == "cuda":
        bf16 = cuda_ok and torch.cuda.is_bf16_supported()
    elif dtype_ == "mps":
        bf16 = mps_available and bool(getattr(mps, "is_bf16_supported", lambda: False)())
    else:
        bf16 = True
    native = _native_library_available()
    can_convert = can_execute = True
    note = None
    if mode in FP8_MODES:
        can_convert = True                      # module substitution itself needs nothing
        can_execute = dtype_ == "cuda" and cuda_ok and capability is not None and capability[0] == 10 and native
        if dtype_ != "cuda":
            note = "fp8 requires a CUDA device"
        elif not cuda_ok:
            note = "fp8 requires CUDA, but CUDA is not available"
        elif capability is None or capability[0] != 10:
            note = f"the fp8 tensor-core kernels are built for compute capability 10.x; got {capability}"
        elif not native:
            note = "the compiled kernel library is not available"
    return {
        "requested_mode": mode, "device": str(device), "device_type": dtype_, "cuda_available": cuda_ok,
        "cuda_device_count": torch.cuda.device_count() if cuda_ok else 0, "cuda_device_capability": capability,
        "native_fp8_available": bool(dtype_ == "cuda" and cuda_ok and capability is not None and capability[0] == 10 and native),
        "fp8_backend": "sjb200" if mode in FP8_MODES else None,
        "torchao_installed": _module_available("torchao"), "transformer_engine_installed": _module_available("transformer_engine"),
        "te_fp8_available": False, "te_fp8_unavailable_reason": "not used: fp8 runs on the package's own kernels",
        "te_autocast_api": None, "te_recipe_availability": {}, "te_recipe_requested": None, "te_recipe_resolved": None,
        "te_recipe_fallback_reason": None,
        "bf16_supported": bool(bf16), "cpu_bf16_autocast": dtype_ == "cpu", "mps_available": mps_available,
        "model_class": type(model).__name__, "can_convert": can_convert, "can_execute": can_execute,
        "runtime_validation_required": can_execute, "execution_note": note,
    }


def validate_capability(report: Dict[str, Any]) -> None:
    """Raise ``RuntimeError`` when the requested mode cannot run on the reported machine."""
    mode, dev = report["requested_mode"], report["device_type"]
    if mode == "fp32":
        return
    if mode == "fp16":
        if dev == "cpu":
            raise RuntimeError("precision='fp16' is not supported on cpu in the current stage.")
        if dev == "cuda" and not report["cuda_available"]:
            raise RuntimeError("precision='fp16' requires CUDA, but CUDA is not available.")
        return
    if mode == "bf16":
        if dev == "cpu":
            return
        if dev == "cuda" and not report["cuda_available"]:
            raise RuntimeError("precision='bf16' requires CUDA or CPU bf16 autocast support.")
        if not report["bf16_supported"]:
            raise RuntimeError(f"precision='bf16' was requested on {dev.upper()}, but this device does not report bf16 support.")
        return
    if mode in FP8_MODES:
        if not report.get("native_fp8_available", False):
            raise RuntimeError(f"precision={mode!r} is unavailable: {report.get('execution_note') or 'unknown reason'}")
        return
    raise RuntimeError(f"Unsupported precision mode {mode!r}. Supported: fp32, fp16, bf16, fp8 (aliases fp8-torchao, fp8-te).")
