"""Compile-and-cache for generated neuron kernels.

The translation unit is written atomically to ``<cache>/<name>_<sha16>.cu`` and compiled by ``nvcc`` for
sm_100a into a shared object next to it; the object is opened with ``ctypes`` and memoised per process.  The
cache directory is ``$SJB200_FLEXSN_CACHE``, else ``~/.cache/spikingjelly_b200/flexsn`` (mode 0700), else a
per-user directory under the system temp directory.  Same role as the source cache of
``triton_kernel/torch2triton/graph2triton.py:79-122,392-500`` in the reference.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import tempfile
import threading
from pathlib import Path
from typing import Dict, Optional

__all__ = ["cache_dir", "compile_module", "nvcc_path", "CompileError"]

_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}

NVCC_FLAGS = ["-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-fmad=false",
              "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo"]


class CompileError(RuntimeError):
    pass


def nvcc_path() -> Optional[str]:
    for cand in (os.environ.get("SJB200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def cache_dir() -> Path:
    choices = []
    if os.environ.get("SJB200_FLEXSN_CACHE"):
        choices.append(Path(os.environ["SJB200_FLEXSN_CACHE"]))
    choices.append(Path.home() / ".cache" / "spikingjelly_b200" / "flexsn")
    choices.append(Path(tempfile.gettempdir()) / f"spikingjelly_b200_flexsn_{os.getuid()}")
    for d in choices:
        try:
            d.mkdir(parents=True, exist_ok=True, mode=0o700)
            if os.access(d, os.W_OK):
                return d
        except OSError:
            continue
    raise CompileError("no writable cache directory for generated kernels")


def _atomic_write(path: Path, data: str) -> None:
    fd, tmp = tempfile.mkstemp(dir=str(path.parent), prefix=path.name + ".", suffix=".tmp")
    try:
        with os.fdopen(fd, "w") as f:
            f.write(data)
        os.replace(tmp, path)
    finally:
        if os.path.exists(tmp):
            os.remove(tmp)


def compile_module(source: str, name: str = "flexsn", load: bool = True):
    """Returns the loaded library (``load=True``) or the path of the shared object."""
    digest = hashlib.sha256((source + " ".join(NVCC_FLAGS)).encode()).hexdigest()[:16]
    key = f"{name}_{digest}"
    with _lock:
        if load and key in _loaded:
            return _loaded[key]
        d = cache_dir()
        cu, so = d / f"{key}.cu", d / f"{key}.so"
        if not so.exists():
            nvcc = nvcc_path()
            if nvcc is None:
                raise CompileError("nvcc was not found (set SJB200_NVCC); generated neuron kernels cannot be built")
            _atomic_write(cu, source)
            tmp_so = d / f"{key}.{os.getpid()}.so.tmp"
            proc = subprocess.run([nvcc, *NVCC_FLAGS, "-o", str(tmp_so), str(cu)], capture_output=True, text=True)
            if proc.returncode != 0:
                if tmp_so.exists():
                    tmp_so.unlink()
                raise CompileError(f"nvcc failed for {cu}:\n{proc.stderr[-4000:]}")
            os.replace(tmp_so, so)
        if not load:
            return so
        lib = ctypes.CDLL(str(so))
        _loaded[key] = lib
        return lib
