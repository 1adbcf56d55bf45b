"""In-tree build of the sm_100a extension (``ops/build/libsjb200.so``).

Every ``csrc/*.cu`` is compiled by ``nvcc -gencode arch=compute_100a,code=sm_100a``
(cross-compiles without a GPU) and linked against libtorch.  Object files are
cached by a hash of the source, the headers and the flags.  Ops register
themselves with ``TORCH_LIBRARY`` so the library is loaded with
``torch.ops.load_library`` and needs no Python headers.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import List

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD = HERE / "build"
LIB = BUILD / "libsjb200.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "--expt-extended-lambda",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-diag-suppress", "177,550"]


#: ptxas resource reports (registers, spills, shared memory) of the translation units compiled by the last verbose build
LAST_PTXAS_LOG: List[str] = []


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; cannot build the sm_100a extension")
    return cand


def _torch_flags():
    import torch
    from torch.utils.cpp_extension import include_paths, library_paths
    inc = []
    for p in include_paths("cuda"):
        inc += ["-isystem", p]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    defs = [f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    libdirs = library_paths("cuda")
    return inc, defs, libdirs


def sources() -> List[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest(src: Path, flags: List[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    h.update(src.read_bytes())
    for hdr in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(hdr.read_bytes())
    return h.hexdigest()[:16]


def _compile_one(nvcc: str, src: Path, obj: Path, flags: List[str], verbose: bool) -> str:
    cmd = [nvcc, "-c", str(src), "-o", str(obj)] + flags
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return proc.stderr


def manifest() -> str:
    inc, defs, _ = _torch_flags()
    flags = ARCH_FLAGS + NVCC_FLAGS + defs
    return ",".join(f"{s.name}:{_digest(s, flags)}" for s in sources())


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile what changed and link ``libsjb200.so``.  Returns its path."""
    nvcc = _nvcc()
    inc, defs, libdirs = _torch_flags()
    flags = ARCH_FLAGS + NVCC_FLAGS + defs + inc + ["-I", str(CSRC)]
    hash_flags = ARCH_FLAGS + NVCC_FLAGS + defs
    (BUILD / "obj").mkdir(parents=True, exist_ok=True)
    jobs, objs = [], []
    for src in sources():
        obj = BUILD / "obj" / f"{src.stem}.{_digest(src, hash_flags)}.o"
        objs.append(obj)
        if force or not obj.exists():
            for stale in (BUILD / "obj").glob(f"{src.stem}.*.o"):
                stale.unlink()
            jobs.append((src, obj))
    logs = []
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            futs = [pool.submit(_compile_one, nvcc, s, o, flags, verbose) for s, o in jobs]
            logs = [f.result() for f in futs]
    stamp = BUILD / "manifest.txt"
    want = manifest()
    if jobs or force or not LIB.exists() or not stamp.exists() or stamp.read_text() != want:
        link = ["g++", "-shared", "-o", str(LIB)] + [str(o) for o in objs]
        for d in libdirs:
            link += [f"-L{d}", f"-Wl,-rpath,{d}"]
        link += ["-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda", "-ltorch_cuda", "-lcudart"]
        proc = subprocess.run(link, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
        stamp.write_text(want)
    if verbose:
        from ..logger import logger
        LAST_PTXAS_LOG[:] = logs
        for lg in logs:
            logger.info("nvcc -Xptxas -v:\n%s", lg)
    return LIB


def is_current() -> bool:
    stamp = BUILD / "manifest.txt"
    try:
        return LIB.exists() and stamp.exists() and stamp.read_text() == manifest()
    except Exception:
        return LIB.exists()


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    for report in LAST_PTXAS_LOG:
        print(report, file=sys.stderr)
