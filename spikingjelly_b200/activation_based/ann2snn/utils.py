"""Resumable HTTP download (used by the examples to fetch pretrained ANN weights).
Parity: ``spikingjelly/activation_based/ann2snn/utils.py:11-176``."""
from __future__ import annotations

import os
import re
import time

from ...logger import logger

__all__ = ["download_url"]

_UA = {"User-Agent": "Mozilla/5.0 (Windows NT 10.0; Win64; x64; rv:67.0) Gecko/20100101 Firefox/67.0"}


def _range_ok(resp, first_byte: int, size: int) -> bool:
    if resp.status_code not in (200, 206):
        resp.raise_for_status()
    if resp.status_code == 200:
        return first_byte == 0
    m = re.match(r"bytes (\d+)-(\d+)/(\d+)", resp.headers.get("Content-Range", ""), re.IGNORECASE)
    return m is not None and (int(m.group(1)), int(m.group(2)), int(m.group(3))) == (first_byte, size - 1, size)


def _stream(resp, dst, mode, bar) -> int:
    written = 0
    with open(dst, mode) as f:
        for chunk in resp.iter_content(chunk_size=1 << 16):
            if chunk:
                f.write(chunk)
                written += len(chunk)
                bar.update(len(chunk))
    return written


def download_url(url: str, dst: str) -> int:
    """Download ``url`` to ``dst``; an existing partial file is continued with an HTTP range request
    (restarted from zero when the server does not honour it).  Returns the file size in bytes."""
    import requests
    from tqdm import tqdm
    t0 = time.perf_counter()
    head = requests.get(url, headers=_UA, stream=True, timeout=30)
    try:
        head.raise_for_status()
        length = head.headers.get("content-length")
    finally:
        head.close()
    resumed = False
    if length is None:
        with tqdm(unit="B", unit_scale=True, desc=dst) as bar:
            resp = requests.get(url, headers=_UA, stream=True, timeout=30)
            try:
                resp.raise_for_status()
                size = _stream(resp, dst, "wb", bar)
            finally:
                resp.close()
    else:
        size = int(length)
        first = os.path.getsize(dst) if os.path.exists(dst) else 0
        if first < size:
            resumed = first > 0
            with tqdm(total=size, initial=first, unit="B", unit_scale=True, desc=dst) as bar:
                resp = requests.get(url, headers={**_UA, "Range": f"bytes={first}-{size - 1}"}, stream=True, timeout=30)
                try:
                    ok, mode = _range_ok(resp, first, size), "ab"
                    if first > 0 and not ok:
                        logger.warning("ann2snn_download_resume_restarted destination=%s existing_bytes=%s", dst, first)
                        resp.close()
                        first, resumed, mode = 0, False, "wb"
                        bar.reset(total=size)
                        resp = requests.get(url, headers={**_UA, "Range": f"bytes=0-{size - 1}"}, stream=True, timeout=30)
                        ok = _range_ok(resp, 0, size)
                    if not ok:
                        raise RuntimeError("Invalid response for download.")
                    written = _stream(resp, dst, mode, bar)
                    if written != size - first:
                        raise RuntimeError(f"Downloaded {written} bytes, but expected {size - first} bytes.")
                finally:
                    resp.close()
    logger.info("ann2snn_download_summary destination=%s resumed=%s bytes=%s elapsed_ms=%.3f", dst, resumed, size, (time.perf_counter() - t0) * 1e3)
    return size
