"""NavGesture (walk / sit): 6 navigation gestures recorded with an ATIS on a phone, 240 x 304, ``_td.dat`` files
(``spikingjelly/datasets/nav_gesture.py:28-496``)."""
import os
import shutil
from pathlib import Path
from typing import Callable, Optional, Tuple

import numpy as np
from torchvision.datasets.utils import extract_archive

from ..logger import logger
from . import utils
from .base import NeuromorphicDatasetFolder, extract_all, run_in_pool

__all__ = ["NAVGestureWalk", "NAVGestureSit"]


def _readATIS_tddat(file_name, orig_at_zero=True, drop_negative_dt=True, events_restriction=(0, np.inf)):
    """kAER ``_td.dat``: ``%`` comment lines, optional 2-byte (type, size) header, then 64-bit little-endian events
    with the timestamp in bits 0-31, x in 32-40, y in 41-48 and polarity in bit 49.  Events whose timestamp is smaller
    than the previous kept one are dropped; what remains is made monotone by repeatedly deleting the second element of
    every decreasing pair.  Returns ``(timestamps, coords[N, 2], polarities, number of removed events)``."""
    with open(file_name, "rb") as f:
        header = False
        while f.peek(1)[:1] == b"%":
            f.readline()
            header = True
        if header:
            ev_type, ev_size = f.read(1)[0], f.read(1)[0]
            if ev_size != 8:
                logger.error("Invalid event size in %s: expected 8, got %s; aborting.", file_name, ev_size)
                return -1, -1, -1, -1
        words = np.frombuffer(f.read(), dtype="<u8")
    lo = int(events_restriction[0])
    hi = words.size if np.isinf(events_restriction[1]) else min(words.size, int(events_restriction[1]) + 2)
    words = words[:hi]
    ts_all = (words & 0xFFFFFFFF).astype(np.int64)
    # sequential rule: event i is kept when i >= lo and ts >= the stored timestamp of slot i-1 (0 if that slot was dropped)
    stored = np.zeros(words.size, dtype=np.int64)
    kept = np.zeros(words.size, dtype=bool)
    prev = 0
    for i in range(words.size):
        if i >= lo and ts_all[i] >= prev:
            kept[i] = True
            stored[i] = ts_all[i]
        prev = stored[i]
    n = int(kept.sum())
    # the reader keeps slot order and truncates to the number of accepted events
    ts = stored[:n].copy()
    x = np.where(kept, (words >> np.uint64(32)) & np.uint64(0x1FF), 0).astype(np.int64)[:n]
    y = np.where(kept, (words >> np.uint64(41)) & np.uint64(0xFF), 0).astype(np.int64)[:n]
    pol = np.where(kept, (words >> np.uint64(49)) & np.uint64(1), 0).astype(np.int64)[:n]
    coords = np.stack([x, y], axis=1)
    if orig_at_zero and n:
        ts = ts - ts[0]
    removed = -1
    if drop_negative_dt:
        removed = 0
        while True:
            bad = np.flatnonzero(np.diff(ts) < 0) + 1
            if bad.size == 0:
                break
            # inside a run of consecutive offenders a pass drops every other one, starting with the first
            start = np.concatenate([[True], np.diff(bad) > 1])
            run_first = np.maximum.accumulate(np.where(start, np.arange(bad.size), 0))
            bad = bad[(np.arange(bad.size) - run_first) % 2 == 0]
            ts, pol, coords = np.delete(ts, bad), np.delete(pol, bad), np.delete(coords, bad, axis=0)
            removed += bad.size
    return ts, coords, pol, removed


def _read_aedat_save_to_np(bin_file, np_file):
    t, xy, p, _ = _readATIS_tddat(bin_file)
    utils.np_savez(np_file, t=t, x=xy[:, 0], y=239 - xy[:, 1], p=p)
    logger.debug("Save [%s] to [%s].", bin_file, np_file)


class NAVGestureWalk(NeuromorphicDatasetFolder):
    _archive = "navgesture-walk.zip"
    _md5 = "5d305266f13005401959e819abe206f0"

    def __init__(self, root: str, data_type: str = "event", frames_number: int = None, split_by: str = None,
                 duration: int = None, custom_integrate_function: Callable = None,
                 custom_integrated_frames_dir_name: str = None, transform: Optional[Callable] = None,
                 target_transform: Optional[Callable] = None):
        super().__init__(root, None, data_type, frames_number, split_by, duration, custom_integrate_function,
                         custom_integrated_frames_dir_name, transform, target_transform)

    @classmethod
    def get_H_W(cls) -> Tuple:
        return 240, 304          # the sensor is 240 x 320 but x never exceeds 303

    @classmethod
    def resource_url_md5(cls) -> list:
        return [(cls._archive, f"https://www.neuromorphic-vision.com/public/downloads/navgesture/{cls._archive}", cls._md5)]

    @classmethod
    def downloadable(cls) -> bool:
        logger.warning("The NavGesture host no longer serves the archives; obtain them manually.")
        return False

    @classmethod
    def extract_downloaded_files(cls, download_root: Path, extract_root: Path):
        tmp = download_root / "temp_ext"
        tmp.mkdir()
        extract_archive(download_root / cls._archive, tmp)
        extract_all([tmp / z for z in os.listdir(tmp) if z.endswith(".zip")], extract_root, max_workers=4)
        shutil.rmtree(tmp)

    @classmethod
    def create_raw_from_extracted(cls, extract_root: Path, raw_root: Path):
        for label in ("le", "ri", "up", "do", "ho", "se"):
            (raw_root / label).mkdir()
        tasks = []
        for user in sorted(os.listdir(extract_root)):
            for name in sorted(os.listdir(extract_root / user)):
                stem = os.path.splitext(name)[0]
                tasks.append((extract_root / user / name, raw_root / stem.split("_")[1] / (stem + ".npz")))
        run_in_pool(_read_aedat_save_to_np, tasks)


class NAVGestureSit(NAVGestureWalk):
    _archive = "navgesture-sit.zip"
    _md5 = "1571753ace4d9e0946e6503313712c22"
