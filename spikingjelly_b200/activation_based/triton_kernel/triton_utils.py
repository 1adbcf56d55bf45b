"""Names and small helpers that scripts written against the reference's ``triton_kernel/triton_utils.py`` use: dtype
spellings and numeric ids of the neuron kernels' storage / compute / spike types, device normalisation, the ``SJ_*``
environment switches and the contiguity-and-device guard.  There is no Triton here; the kernels behind these names are
the CUDA scan kernels of ``ops/csrc/neuron_scan.cuh``, which keep the recurrence in fp32 registers whatever the storage
type, so a "compute dtype" only selects how the reference would have rounded - it is validated and recorded, not obeyed."""
from __future__ import annotations

import functools
import os
from typing import Callable, Union

import torch

__all__ = ["triton_neuron_compute_dtype_id_to_tl_dtype", "torch_dtype_for_triton_neuron_compute_dtype_id", "convert_and_store",
           "register_op", "wrap_triton", "TRITON_NEURON_DTYPE_FP32", "TRITON_NEURON_DTYPE_FP16", "TRITON_NEURON_DTYPE_BF16", "TRITON_NEURON_DTYPE_FP8_E4M3FN",
           "TRITON_NEURON_DTYPE_FP8_E5M2", "normalize_triton_compute_dtype_name", "normalize_triton_storage_dtype", "is_fp8_dtype",
           "torch_dtype_to_triton_neuron_dtype_id", "triton_neuron_dtype_id_to_torch_dtype", "triton_compute_dtype_name_to_neuron_dtype_id",
           "resolve_triton_compute_dtype", "torch_dtype_for_triton_compute_dtype", "normalize_cuda_device", "contiguous_and_device_guard",
           "use_static_range_for_triton_neuron_kernel", "env_flag_enabled"]

TRITON_NEURON_DTYPE_FP32, TRITON_NEURON_DTYPE_FP16, TRITON_NEURON_DTYPE_BF16 = 0, 1, 2
TRITON_NEURON_DTYPE_FP8_E4M3FN, TRITON_NEURON_DTYPE_FP8_E5M2 = 3, 4

_IDS = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2, torch.float8_e4m3fn: 3, torch.float8_e5m2: 4}
_COMPUTE = {"fp32": ("float32", "torch.float32", "float", "fp32"), "fp16": ("float16", "torch.float16", "half", "fp16"),
            "bf16": ("bfloat16", "torch.bfloat16", "bf16"), "fp8": ("float8", "fp8")}
_STORAGE = {torch.float32: ("float32", "fp32", "float"), torch.float16: ("float16", "fp16", "half"), torch.bfloat16: ("bfloat16", "bf16"),
            torch.float8_e4m3fn: ("float8_e4m3fn", "fp8_e4m3fn", "e4m3fn"), torch.float8_e5m2: ("float8_e5m2", "fp8_e5m2", "e5m2")}


def normalize_triton_compute_dtype_name(compute_dtype: Union[str, torch.dtype]) -> str:
    """``"fp32" | "fp16" | "bf16" | "fp8"`` from any accepted spelling or a torch dtype."""
    key = str(compute_dtype).lower() if not isinstance(compute_dtype, str) else compute_dtype.lower()
    if isinstance(compute_dtype, torch.dtype) and is_fp8_dtype(compute_dtype):
        return "fp8"
    for name, spellings in _COMPUTE.items():
        if key in spellings:
            return name
    raise ValueError(f"Unsupported compute dtype {compute_dtype!r}; expected one of fp32, fp16, bf16, fp8.")


def normalize_triton_storage_dtype(storage_dtype: Union[str, torch.dtype]) -> torch.dtype:
    if isinstance(storage_dtype, torch.dtype):
        if storage_dtype in _STORAGE:
            return storage_dtype
        raise ValueError(f"Unsupported storage dtype {storage_dtype}.")
    key = str(storage_dtype).lower().removeprefix("torch.")
    for dtype, spellings in _STORAGE.items():
        if key in spellings:
            return dtype
    raise ValueError(f"Unsupported storage dtype {storage_dtype!r}.")


def is_fp8_dtype(dtype: torch.dtype) -> bool:
    return dtype in (torch.float8_e4m3fn, torch.float8_e5m2)


def torch_dtype_to_triton_neuron_dtype_id(dtype: torch.dtype) -> int:
    try:
        return _IDS[dtype]
    except KeyError:
        raise ValueError(f"Unsupported neuron dtype {dtype}.") from None


def triton_neuron_dtype_id_to_torch_dtype(dtype_id: int) -> torch.dtype:
    for dtype, i in _IDS.items():
        if i == dtype_id:
            return dtype
    raise ValueError(f"Unknown neuron dtype id {dtype_id}.")


def triton_compute_dtype_name_to_neuron_dtype_id(compute_dtype_name: str, storage_dtype: torch.dtype) -> int:
    """``"fp8"`` means "compute in the storage format", so its id is the storage dtype's."""
    name = normalize_triton_compute_dtype_name(compute_dtype_name)
    if name == "fp8":
        if not is_fp8_dtype(storage_dtype):
            raise ValueError("compute_dtype='fp8' requires an fp8 storage dtype.")
        return _IDS[storage_dtype]
    return {"fp32": 0, "fp16": 1, "bf16": 2}[name]


def resolve_triton_compute_dtype(compute_dtype, storage_dtype=None) -> str:
    return normalize_triton_compute_dtype_name(compute_dtype)


def torch_dtype_for_triton_compute_dtype(compute_dtype, storage_dtype: torch.dtype) -> torch.dtype:
    name = normalize_triton_compute_dtype_name(compute_dtype)
    return storage_dtype if name == "fp8" else {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}[name]


def normalize_cuda_device(device) -> torch.device:
    """A CUDA ``torch.device`` with an explicit index."""
    if isinstance(device, int):
        device = torch.device("cuda", device)
    device = torch.device(device)
    if device.type != "cuda":
        raise ValueError(f"expected a CUDA device, got {device}.")
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device() if torch.cuda.is_available() else 0)
    return device


def env_flag_enabled(var_name: str) -> bool:
    """``SJ_*`` switches: set and not one of ``0 / false / no / off``."""
    return os.environ.get(var_name, "").strip().lower() not in ("", "0", "false", "no", "off")


_env_flag_enabled = env_flag_enabled


def contiguous_and_device_guard(f: Callable) -> Callable:
    """Decorator: tensor arguments are made contiguous and the call runs with the first CUDA tensor's device current."""
    @functools.wraps(f)
    def wrapper(*args, **kwargs):
        device = next((a.device for a in list(args) + list(kwargs.values()) if isinstance(a, torch.Tensor) and a.is_cuda), None)
        args = [a.contiguous() if isinstance(a, torch.Tensor) else a for a in args]
        kwargs = {k: (v.contiguous() if isinstance(v, torch.Tensor) else v) for k, v in kwargs.items()}
        if device is None:
            return f(*args, **kwargs)
        with torch.cuda.device(device):
            return f(*args, **kwargs)
    return wrapper


def use_static_range_for_triton_neuron_kernel(T: int) -> bool:
    """Whether the reference would unroll the time loop at compile time; here: whether T fits one register chunk."""
    return T <= 8


def triton_neuron_compute_dtype_id_to_tl_dtype(dtype_id: int, storage_dtype_id: int):
    """The reference maps a compute dtype id to a Triton language dtype; the CUDA kernels compute in fp32 registers whatever is
    asked, so the answer here is the torch dtype the id names (after the same validity checks: fp8 compute needs the matching
    fp8 storage)."""
    dt = triton_neuron_dtype_id_to_torch_dtype(dtype_id)
    if is_fp8_dtype(dt) and dtype_id != storage_dtype_id:
        raise ValueError("FP8 compute requires the matching FP8 storage dtype.")
    return dt


def torch_dtype_for_triton_neuron_compute_dtype_id(dtype_id: int) -> torch.dtype:
    """Dtype of reduction buffers for a compute dtype id: fp32 for the fp8 ids (no useful reductions exist on fp8 tensors)."""
    dt = triton_neuron_dtype_id_to_torch_dtype(dtype_id)
    return torch.float32 if is_fp8_dtype(dt) else dt


def convert_and_store(pointer: torch.Tensor, value: torch.Tensor, boundary_check=None) -> None:
    """``pointer[...] = value`` with an explicit cast to the destination dtype (in a Triton kernel the reference needs this for
    block pointers; on tensors it is a converting copy)."""
    pointer.copy_(value.to(pointer.dtype))


def register_op(opname: str, mutates_args=()):
    """Decorator registering a custom operator (``torch.library.custom_op``; there is no Triton-op variant to choose)."""
    return torch.library.custom_op(opname, mutates_args=mutates_args)


def wrap_triton(kernel):
    """Identity: kernels here are CUDA launchers, which need no wrapping to be traced as opaque calls."""
    return kernel
