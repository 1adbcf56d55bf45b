"""Hand-assembled CUDA kernels from Python: a kernel is a parameter table plus code fragments (declaration, head, core,
tail) that the user fills in; calling it compiles the source once and launches it on PyTorch tensors
(``cuda_kernel/auto_cuda/base.py:18-1439`` of the reference, where the source goes to CuPy's NVRTC).

Here the assembled translation unit is compiled ahead of the first launch by ``nvcc`` for sm_100a into a cached shared
object (the same compile-and-cache path as the generated neuron kernels, ``ops/flexsn/compiler.py``); next to the
``__global__`` function it holds a small ``extern "C"`` launcher that takes the grid, the block, the CUDA stream of
PyTorch and the argument pointers.  Scalars are passed by value: a ``const int &`` parameter type, the convention of the
reference's kernels, is accepted and compiled as ``const int``.

* :class:`CKernel`    - free-form kernel; the caller gives grid and block.
* :class:`CKernel1D`  - element-wise: ``index`` runs over ``numel`` elements.
* :class:`CKernel2D`  - sequences ``[T, N]``: thread ``index`` owns column ``index`` and walks ``t = index, index + N,
  ...`` (or backwards with ``reverse=True``), with ``pre_core`` / ``post_core`` fragments around the time loop.
* :class:`CodeTyper`, :class:`CodeBlock` - indentation-aware assembly of code fragments.

``float16`` tensors bound to ``half2`` parameters are processed two elements per thread; odd lengths are padded by
repeating the last element (1-D) or the last column (``[T, N]``) for the call and cut back afterwards.
"""
from __future__ import annotations

import ctypes
import logging
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from ....logger import logger
from .... import configure

__all__ = ["wrap_with_comment", "startswiths", "CKernel", "CKernel1D", "CKernel2D", "CodeTyper", "CodeBlock"]

_PREAMBLE = "#include <cuda_fp16.h>\n#include <cuda_runtime.h>\n"
_SCALARS = {"int": (ctypes.c_int, int), "float": (ctypes.c_float, float), "double": (ctypes.c_double, float), "bool": (ctypes.c_bool, bool),
            "long long": (ctypes.c_longlong, int), "unsigned int": (ctypes.c_uint, int), "half": (ctypes.c_uint16, float)}
_POINTER_DTYPES = {"float": (torch.float32,), "double": (torch.float64,), "int": (torch.int32,), "half": (torch.float16,), "half2": (torch.float16,),
                   "bool": (torch.bool,), "long long": (torch.int64,), "unsigned char": (torch.uint8,), "char": (torch.int8,)}


def wrap_with_comment(code: str, comment: str) -> str:
    """``code`` between ``// ------ comment start`` / ``end`` markers; empty code stays empty."""
    if code == "":
        return ""
    return f"\n//------{comment} start------\n{code}\n//------{comment} end--------\n\n"


def startswiths(x: str, prefixes: tuple) -> bool:
    return any(x.startswith(p) for p in prefixes)


def _base_type(ctype: str) -> Tuple[str, bool]:
    """``'const float *'`` -> ``('float', True)``; ``'const int &'`` -> ``('int', False)``."""
    t = ctype.replace("const", " ").replace("&", " ").replace("__restrict__", " ")
    pointer = "*" in t
    return " ".join(t.replace("*", " ").split()), pointer


class CKernel:
    """``cparams``: ordered ``{name: C type}``; ``reserved_cnames``: names the code fragments use themselves.  Subclasses
    override :attr:`head` / :attr:`tail`; the user sets :attr:`core`."""

    def __init__(self, kernel_name: str):
        self.cparams: Dict[str, str] = {}
        self.reserved_cnames: list = []
        self.kernel_name = kernel_name
        self._core = ""
        self.extra_headers = ""             # source text placed before the kernel (device helpers the fragments call)
        self._lib = None
        self._built_source: Optional[str] = None

    def check_attributes(self, **kwargs) -> bool:
        """True when every given attribute of this kernel has the given value (used to decide whether a cached kernel
        object can be reused)."""
        return all(hasattr(self, k) and getattr(self, k) == v for k, v in kwargs.items())

    @property
    def core(self) -> str:
        return self._core

    @core.setter
    def core(self, value: str) -> None:
        self._core = value

    # -- source -------------------------------------------------------------------------------------------------------
    def add_param(self, ctype: str, cname: str) -> None:
        if cname in self.cparams:
            raise ValueError(f"{cname} has been added to cparams!")
        if cname in self.reserved_cnames:
            raise ValueError(f"{cname} is the reserved cname. You should change the name of your variable to avoid conflict.")
        self.cparams[cname] = ctype

    @property
    def declaration(self) -> str:
        params = ", ".join(f"{ctype.replace('&', '').rstrip()} {name}" for name, ctype in self.cparams.items())
        return f'extern "C" __global__\nvoid {self.kernel_name}({params})\n'

    @property
    def head(self) -> str:
        return "{"

    @property
    def tail(self) -> str:
        return "}"

    @property
    def full_codes(self) -> str:
        return self.declaration + self.head + wrap_with_comment(self.core, "core") + self.tail

    @property
    def translation_unit(self) -> str:
        """:attr:`full_codes` with the includes and the host launcher."""
        return (_PREAMBLE + self.extra_headers + "\n" + self.full_codes +
                f'\nextern "C" __attribute__((visibility("default"))) int launch_{self.kernel_name}(unsigned gx, unsigned gy, unsigned gz, '
                f"unsigned bx, unsigned by, unsigned bz, void* stream, void** args) {{\n"
                f"    return (int)cudaLaunchKernel((const void*){self.kernel_name}, dim3(gx, gy, gz), dim3(bx, by, bz), args, 0, (cudaStream_t)stream);\n}}\n")

    # -- argument checks ----------------------------------------------------------------------------------------------
    def set_contiguous(self, py_dict: dict) -> None:
        for key, value in py_dict.items():
            if isinstance(value, torch.Tensor):
                py_dict[key] = value.contiguous()
            elif not isinstance(value, (int, float, bool, np.generic)):
                raise TypeError(f"{key}: tensors and Python / NumPy scalars are supported, got {type(value)}")

    def get_device(self, py_dict: dict) -> int:
        for value in py_dict.values():
            if isinstance(value, torch.Tensor):
                if not value.is_cuda:
                    raise ValueError("CKernel arguments must live on a CUDA device.")
                return value.get_device()
        raise ValueError("No CUDA tensor among the kernel arguments: the device cannot be determined.")

    def check_device(self, device: int, py_dict: dict) -> None:
        for key, value in py_dict.items():
            if isinstance(value, torch.Tensor) and value.get_device() != device:
                raise ValueError(f"{key} is on device {value.get_device()}, expected {device}.")

    def check_keys(self, py_dict: dict) -> None:
        if set(py_dict) != set(self.cparams):
            missed, unexpected = set(self.cparams) - set(py_dict), set(py_dict) - set(self.cparams)
            raise ValueError(f"py_dict does not match cparams: missing {sorted(missed)}, unexpected {sorted(unexpected)}")

    def check_ctypes(self, py_dict: dict) -> None:
        for name, ctype in self.cparams.items():
            base, pointer = _base_type(ctype)
            value = py_dict[name]
            if pointer:
                if not isinstance(value, torch.Tensor):
                    raise TypeError(f"{name}: parameter type '{ctype}' needs a tensor, got {type(value)}")
                allowed = _POINTER_DTYPES.get(base)
                if allowed is not None and value.dtype not in allowed:
                    raise TypeError(f"{name}: parameter type '{ctype}' does not accept a tensor of {value.dtype}")
            elif isinstance(value, torch.Tensor):
                raise TypeError(f"{name}: parameter type '{ctype}' is a scalar, got a tensor")
            elif base not in _SCALARS:
                raise TypeError(f"{name}: unsupported scalar parameter type '{ctype}'")

    def check_half2(self, py_dict: dict) -> None:
        """Free-form kernels take ``half2`` buffers as they are (an even number of elements is the caller's business)."""
        for name, ctype in self.cparams.items():
            if _base_type(ctype)[0] == "half2" and isinstance(py_dict.get(name), torch.Tensor) and py_dict[name].numel() % 2:
                raise ValueError(f"{name}: a half2 parameter needs an even number of float16 elements")

    def get_ptrs(self, py_dict: dict):
        """ctypes values in parameter order (data pointers for tensors)."""
        out = []
        for name, ctype in self.cparams.items():
            base, pointer = _base_type(ctype)
            value = py_dict[name]
            if pointer:
                out.append(ctypes.c_void_p(value.data_ptr()))
            elif base == "half":
                out.append(ctypes.c_uint16(int(np.float16(value).view(np.uint16))))
            else:
                c_type, py_type = _SCALARS[base]
                out.append(c_type(py_type(value)))
        return out

    # -- build and launch ---------------------------------------------------------------------------------------------
    def _library(self):
        source = self.translation_unit
        if self._lib is None or self._built_source != source:
            from ....ops.flexsn import compiler
            if logger.isEnabledFor(logging.DEBUG):
                logger.debug("auto_cuda source of %s:\n%s", self.kernel_name, source)
            self._lib = compiler.compile_module(source, name=f"auto_cuda_{self.kernel_name}")
            self._built_source = source
        return self._lib

    def __call__(self, grid: tuple, block: tuple, py_dict: dict, *args_1, **kwargs) -> None:
        """Launch with ``py_dict = {parameter name: tensor or scalar}``.  Tensors may be replaced in ``py_dict`` by their
        contiguous versions; read results from ``py_dict`` after the call."""
        self.set_contiguous(py_dict)
        device = self.get_device(py_dict)
        self.check_device(device, py_dict)
        self.check_keys(py_dict)
        self.check_ctypes(py_dict)
        values = self.get_ptrs(py_dict)
        argv = (ctypes.c_void_p * len(values))(*[ctypes.cast(ctypes.pointer(v), ctypes.c_void_p) for v in values])
        g = tuple(grid) + (1,) * (3 - len(grid))
        b = tuple(block) + (1,) * (3 - len(block))
        fn = getattr(self._library(), f"launch_{self.kernel_name}")
        fn.restype = ctypes.c_int
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream().cuda_stream
            err = fn(*(ctypes.c_uint(int(v)) for v in g + b), ctypes.c_void_p(stream), argv)
        if err != 0:
            raise RuntimeError(f"launch of {self.kernel_name} failed with CUDA error {err}")


def _blocks(numel: int, threads: int) -> int:
    return (numel + threads - 1) // threads


class CKernel1D(CKernel):
    """Element-wise kernel: thread ``index`` handles element ``index`` of ``numel``."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.cparams["numel"] = "const int &"
        self.reserved_cnames.append("index")

    @property
    def head(self) -> str:
        return "\n{\n    const int index = blockIdx.x * blockDim.x + threadIdx.x;\n    if (index < numel)\n    {\n"

    @property
    def tail(self) -> str:
        return "\n    }\n}\n"

    def check_half2(self, py_dict: dict):
        """Pad odd float16 tensors bound to ``half2`` parameters by repeating their last element; returns the list of
        ``(name, original shape)`` to cut back."""
        padded = []
        for name, ctype in self.cparams.items():
            v = py_dict.get(name)
            if _base_type(ctype)[0] == "half2" and isinstance(v, torch.Tensor) and v.numel() % 2:
                flat = v.flatten()
                py_dict[name] = torch.cat((flat, flat[-1:]))
                padded.append((name, v.shape))
        return padded

    def __call__(self, grid: Optional[tuple], block: Optional[tuple], py_dict: dict, *args_1, **kwargs) -> None:
        padded = self.check_half2(py_dict)
        if block is None:
            block = (configure.cuda_threads,)
        if grid is None:
            grid = (_blocks(int(py_dict["numel"]), block[0]),)
        super().__call__(grid, block, py_dict, *args_1, **kwargs)
        for name, shape in padded:
            py_dict[name] = py_dict[name][:-1].view(shape)

    def simple_call(self, **kwargs) -> dict:
        """``kernel.simple_call(x=..., y=...)``: ``numel`` is taken from the first tensor (halved when the kernel works on
        ``half2``), the launch shape from ``configure.cuda_threads``.  Returns the argument dictionary after the call."""
        py_dict = dict(kwargs)
        if "numel" not in py_dict:
            name, first = next((k, v) for k, v in py_dict.items() if isinstance(v, torch.Tensor))
            n = first.numel()
            if _base_type(self.cparams[name])[0] == "half2":
                n = (n + 1) // 2
            py_dict["numel"] = n
        self(None, None, py_dict)
        return py_dict


class CKernel2D(CKernel):
    """Kernel over sequences ``[T, N]``: ``numel = T * N`` elements, thread ``index < N`` visits ``t = index + k * N``
    in time order (or from the last step back with ``reverse=True``).  ``pre_core`` runs before the time loop, ``core``
    inside it, ``post_core`` after it."""

    def __init__(self, kernel_name: str, reverse: bool = False):
        super().__init__(kernel_name)
        self.cparams["numel"] = "const int &"
        self.cparams["N"] = "const int &"
        self.reverse = reverse
        self.reserved_cnames += ["index", "dt", "t"]
        self._pre_core = self._post_core = ""

    @property
    def pre_core(self) -> str:
        return self._pre_core

    @pre_core.setter
    def pre_core(self, value: str) -> None:
        self._pre_core = value

    @property
    def post_core(self) -> str:
        return self._post_core

    @post_core.setter
    def post_core(self, value: str) -> None:
        self._post_core = value

    @property
    def head(self) -> str:
        loop = "for (int t = numel - N + index; t >= 0; t -= dt)" if self.reverse else "for (int t = index; t < numel; t += dt)"
        return ("\n{\n    const int index = blockIdx.x * blockDim.x + threadIdx.x;\n    if (index < N)\n    {\n        const int dt = N;\n"
                + wrap_with_comment(self.pre_core, "pre_core") + f"        {loop}\n        {{\n")

    @property
    def tail(self) -> str:
        return "\n        }\n" + wrap_with_comment(self.post_core, "post_core") + "    }\n}\n"

    def check_shape(self, py_dict: dict) -> None:
        """Every 2-D tensor is ``[T, N]`` with the same ``N``; every 1-D tensor has ``N`` elements.  One-element tensors are
        parameters (a learnable scalar and its gradient accumulator) and are not checked."""
        n = None
        for key, v in py_dict.items():
            if isinstance(v, torch.Tensor) and v.dim() >= 1 and v.numel() != 1:
                cols = v.shape[1] if v.dim() == 2 else (v.shape[0] if v.dim() == 1 else None)
                if cols is None:
                    raise ValueError(f"{key}: CKernel2D takes [T, N] and [N] tensors, got shape {tuple(v.shape)}")
                if n is None:
                    n = cols
                elif cols != n:
                    raise ValueError(f"{key}: expected {n} columns, got {cols}")

    def check_half2(self, py_dict: dict):
        padded = []
        for name, ctype in self.cparams.items():
            v = py_dict.get(name)
            if _base_type(ctype)[0] != "half2" or not isinstance(v, torch.Tensor):
                continue
            if v.dim() <= 1 and v.numel() % 2:
                flat = v.flatten()
                py_dict[name] = torch.cat((flat, flat[-1:]))
                padded.append((name, v.shape))
            elif v.dim() == 2 and v.shape[1] % 2:
                py_dict[name] = torch.cat((v, v[:, -1:]), dim=1)
                padded.append((name, v.shape))
        return padded

    def __call__(self, grid: Optional[tuple], block: Optional[tuple], py_dict: dict, *args_1, **kwargs) -> None:
        self.check_shape(py_dict)
        padded = self.check_half2(py_dict)
        if block is None:
            block = (configure.cuda_threads,)
        if grid is None:
            grid = (_blocks(int(py_dict["N"]), block[0]),)
        super().__call__(grid, block, py_dict, *args_1, **kwargs)
        for name, shape in padded:
            v = py_dict[name]
            py_dict[name] = v[:-1].view(shape) if len(shape) <= 1 else v[:, :-1]

    def simple_call(self, **kwargs) -> dict:
        """``numel`` and ``N`` come from the first ``[T, N]`` tensor (``N`` counted in ``half2`` pairs when the kernel
        works on ``half2``)."""
        py_dict = dict(kwargs)
        name, first = next((k, v) for k, v in py_dict.items() if isinstance(v, torch.Tensor) and v.dim() == 2)
        T, n = first.shape
        if _base_type(self.cparams[name])[0] == "half2":
            n = (n + 1) // 2
        py_dict.setdefault("N", n)
        py_dict.setdefault("numel", T * n)
        self(None, None, py_dict)
        return py_dict


class CodeTyper:
    """Accumulates statements with a base indentation: ``append("a = b; c = d;")`` writes one statement per line, adding
    the missing final semicolon; ``{`` and ``}`` lines are written as they are."""

    def __init__(self, indent_num: int):
        self.indent = " " * indent_num
        self.codes = "\n"

    def append(self, codes: str) -> None:
        for piece in codes.replace("\n", "").split(";"):
            piece = piece.strip()
            if not piece:
                continue
            if piece in ("{", "}") or piece.endswith("{") or piece.endswith("}"):
                self.codes += f"{self.indent}{piece}\n"
            else:
                self.codes += f"{self.indent}{piece};\n"


class CodeBlock:
    """``with CodeBlock(typer): typer.append(...)`` wraps what is appended in braces, indented one level deeper."""

    def __init__(self, env: CodeTyper):
        self.env = env

    def __enter__(self):
        self.env.append("{")
        self.env.indent += " "
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        self.env.indent = self.env.indent[:-1]
        self.env.append("}")
