"""Native sm_100a operators.

``load()`` makes ``torch.ops.sjb200.*`` available (building the library first when
a compiler is present and the sources changed).  On a machine with a GPU a missing
library is an error, never a silent fallback: callers that asked for the native
backend get an exception that says how to build it.
"""
from __future__ import annotations

import threading

import torch

from ..logger import logger
from . import _build

_lock = threading.Lock()
_loaded = False
_error: Exception | None = None


def load(build_if_needed: bool = True) -> None:
    """Load ``libsjb200.so`` into this process (idempotent, thread-safe)."""
    global _loaded, _error
    if _loaded:
        return
    with _lock:
        if _loaded:
            return
        try:
            if build_if_needed and not _build.is_current():
                try:
                    _build.build()
                except Exception as exc:  # stale or missing library and no way to rebuild it
                    if not _build.LIB.exists():
                        raise
                    logger.warning("using an out-of-date %s: rebuild failed (%s)", _build.LIB.name, exc)
            if not _build.LIB.exists():
                raise RuntimeError(f"{_build.LIB} does not exist; run `python -m spikingjelly_b200.ops._build`")
            torch.ops.load_library(str(_build.LIB))
            _loaded = True
            _error = None
            from . import _fake
            _fake.register()
        except Exception as exc:
            _error = exc
            raise


def available() -> bool:
    """True if the native operators can run here (library loads and CUDA is up)."""
    if not torch.cuda.is_available():
        return False
    try:
        load()
        return True
    except Exception:
        return False


def require() -> None:
    """Load the library or raise a clear error (used by every native entry point)."""
    try:
        load()
    except Exception as exc:
        raise RuntimeError(
            "the sm_100a extension of spikingjelly_b200 is not usable: "
            f"{exc}.  Build it with `python -m spikingjelly_b200.ops._build`.") from exc


def library_path() -> str:
    return str(_build.LIB)
