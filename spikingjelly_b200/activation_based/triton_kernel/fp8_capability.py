"""What this device and build can do with 8-bit floats (the reference probes Triton for the same answers,
``triton_kernel/fp8_capability.py:29-330``)."""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

__all__ = ["fp8_dtypes", "fp8_capability", "is_fp8_dtype", "supports_triton_fp8_e4m3fn", "supports_triton_fp8_e5m2",
           "supports_triton_fp8_neuron_forward", "supports_triton_fp8_neuron_backward", "triton_fp8_neuron_capability",
           "triton_fp8_neuron_backward_capability", "triton_fp8_neuron_capability_report"]


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
            "gemm": "tcgen05 kind::f8f6f4 (e4m3 / e5m2, per-tensor scales)", "neuron_input": "float8_e4m3fn / float8_e5m2"}


# ------------------------------------------------------------------ the reference's probe names
_COMPUTE = ("fp32", "fp16", "bf16", "fp8")


def _neuron_probe(dtype, device, compute_dtype="fp32") -> Dict[str, Any]:
    """Can the neuron kernels take ``dtype`` as input storage on ``device``?  Storage in either fp8 format is supported with
    fp32 arithmetic in registers; the other compute dtypes are reported as unavailable (the kernels never compute in fewer
    than 32 bits, so asking for them is accepted by the plan but changes nothing)."""
    if isinstance(dtype, str):
        dtype = {"fp8_e4m3fn": "float8_e4m3fn", "fp8_e5m2": "float8_e5m2"}.get(dtype, dtype)
        dtype = getattr(torch, dtype, None)
    if not is_fp8_dtype(dtype):
        raise ValueError(f"not an fp8 dtype: {dtype!r}")
    dev = torch.device(device) if not isinstance(device, torch.device) else device
    if dev.type != "cuda":
        return {"available": False, "reason": "fp8 neuron kernels need a CUDA device"}
    name = str(compute_dtype).replace("torch.", "")
    name = {"float32": "fp32", "float16": "fp16", "bfloat16": "bf16"}.get(name, name)
    if name.startswith("fp8") or name.startswith("float8"):
        name = "fp8"
    if name not in _COMPUTE:
        raise ValueError(f"unknown compute dtype {compute_dtype!r}")
    cap = fp8_capability(dev)
    if not cap["available"]:
        return {"available": False, "reason": cap["reason"]}
    if name != "fp32":
        return {"available": False, "reason": f"arithmetic is fp32 in registers; {name} compute is not a separate kernel"}
    return {"available": True, "reason": None}


def supports_triton_fp8_e4m3fn(device) -> bool:
    return bool(_neuron_probe(torch.float8_e4m3fn, device)["available"])


def supports_triton_fp8_e5m2(device) -> bool:
    return bool(_neuron_probe(torch.float8_e5m2, device)["available"])


def supports_triton_fp8_neuron_forward(dtype, device, compute_dtype="fp32") -> bool:
    return bool(_neuron_probe(dtype, device, compute_dtype)["available"])


supports_triton_fp8_neuron_backward = supports_triton_fp8_neuron_forward       # one kernel pair: what runs forward runs backward
triton_fp8_neuron_capability = triton_fp8_neuron_backward_capability = _neuron_probe


def triton_fp8_neuron_capability_report(device) -> Dict[str, Any]:
    """``dtypes``: per fp8 storage dtype, forward / backward availability with fp32 compute; ``compute_dtypes``: the same for
    every compute dtype name."""
    dev = torch.device(device) if not isinstance(device, torch.device) else device
    def cell(dt, comp):
        r = _neuron_probe(dt, dev, comp)
        return {"forward": r["available"], "backward": r["available"], "reason": r["reason"]}
    names = {n: d for n, d in fp8_dtypes().items() if d is not None}
    return {"device": str(dev), "torch": torch.__version__, "backend": "cuda scan kernels (sm_100a)",
            "dtypes": {n: cell(d, "fp32") for n, d in names.items()},
            "compute_dtypes": {c: {n: cell(d, c) for n, d in names.items()} for c in _COMPUTE}}
