"""What this device and build can do with 8-bit floats (the reference probes Triton for the same answers,
``triton_kernel/fp8_capability.py:29-330``)."""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

__all__ = ["fp8_dtypes", "fp8_capability", "is_fp8_dtype"]


def fp8_dtypes() -> Dict[str, Optional[torch.dtype]]:
    return {name: getattr(torch, name, None) for name in ("float8_e4m3fn", "float8_e5m2")}


def is_fp8_dtype(dtype) -> bool:
    return dtype is not None and dtype in tuple(d for d in fp8_dtypes().values() if d is not None)


def fp8_capability(device=None) -> Dict[str, Any]:
    """``available``: the native fp8 GEMM and the fp8-input neuron kernels can run on ``device``; ``reason`` otherwise."""
    if not torch.cuda.is_available():
        return {"available": False, "reason": "no CUDA device", "dtypes": fp8_dtypes()}
    major, minor = torch.cuda.get_device_capability(device)
    if major < 10:
        return {"available": False, "reason": f"compute capability {major}.{minor} < 10.0 (the kernels are built for sm_100a)", "dtypes": fp8_dtypes()}
    from ... import ops
    ok = ops.available()
    return {"available": bool(ok), "reason": None if ok else "native library not loaded", "dtypes": fp8_dtypes(),
            "gemm": "tcgen05 kind::f8f6f4 (e4m3 / e5m2, per-tensor scales)", "neuron_input": "float8_e4m3fn"}
