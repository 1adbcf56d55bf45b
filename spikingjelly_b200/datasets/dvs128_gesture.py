"""DVS128 Gesture: 11 hand gestures, 29 subjects, 3 lighting conditions, 128 x 128, AEDAT 3.1 recordings that
hold several labelled trials each (``spikingjelly/datasets/dvs128_gesture.py:20-629``)."""
import os
from pathlib import Path
from typing import Callable, Optional, Tuple

import numpy as np
from torchvision.datasets.utils import extract_archive

from ..logger import logger
from . import utils
from .base import NeuromorphicDatasetFolder, run_in_pool

__all__ = ["DVS128Gesture"]


def _split_aedat_files_to_np(fname: str, aedat_file: Path, csv_file: Path, output_dir: Path):
    """Cuts one recording into its trials by the ``(class, startTime_usec, endTime_usec)`` rows of the label file.
    Labels become 0..10; a class that occurs several times in one recording gets a running suffix.  Each row is cut
    on its own because some label files have overlapping intervals."""
    events = utils.load_aedat_v3(aedat_file)
    rows = np.atleast_2d(np.loadtxt(csv_file, dtype=np.uint32, delimiter=",", skiprows=1))
    seen = [0] * 11
    for label_1, t0, t1 in rows:
        label = int(label_1) - 1
        mask = (events["t"] >= t0) & (events["t"] < t1)
        out = output_dir / str(label) / f"{fname}_{seen[label]}.npz"
        utils.np_savez(out, t=events["t"][mask], x=events["x"][mask], y=events["y"][mask], p=events["p"][mask])
        seen[label] += 1
    logger.debug("[%s] split into [%s] samples.", aedat_file, len(rows))


class DVS128Gesture(NeuromorphicDatasetFolder):
    def __init__(self, root: str, train: bool = True, data_type: str = "event", frames_number: int = None,
                 split_by: str = None, duration: int = None, custom_integrate_function: Callable = None,
                 custom_integrated_frames_dir_name: str = None, transform: Optional[Callable] = None,
                 target_transform: Optional[Callable] = None):
        if train is None:
            raise ValueError("`train` must be `True` or `False`")
        super().__init__(root, train, data_type, frames_number, split_by, duration, custom_integrate_function,
                         custom_integrated_frames_dir_name, transform, target_transform)

    @classmethod
    def get_H_W(cls) -> Tuple:
        return 128, 128

    @classmethod
    def resource_url_md5(cls) -> list:
        url = "https://ibm.ent.box.com/s/3hiq58ww1pbbjrinh367ykfdf60xsfm8/folder/50167556794"
        return [("DvsGesture.tar.gz", url, "8a5c71fb11e24e5ca5b11866ca6c00a1"),
                ("gesture_mapping.csv", url, "109b2ae64a0e1f3ef535b18ad7367fd1"),
                ("LICENSE.txt", url, "065e10099753156f18f51941e6e44b66"),
                ("README.txt", url, "a0663d3b1d8307c329a43d949ee32d19")]

    @classmethod
    def downloadable(cls) -> bool:
        return False

    @classmethod
    def extract_downloaded_files(cls, download_root: Path, extract_root: Path):
        extract_archive(download_root / "DvsGesture.tar.gz", extract_root)

    @classmethod
    def create_raw_from_extracted(cls, extract_root: Path, raw_root: Path):
        aedat_dir = extract_root / "DvsGesture"
        tasks = []
        for split in ("train", "test"):
            out = raw_root / split
            out.mkdir()
            for label in range(11):
                (out / str(label)).mkdir()
            with open(aedat_dir / f"trials_to_{split}.txt") as f:
                for line in f:
                    name = line.strip()
                    if name:
                        stem = os.path.splitext(name)[0]
                        tasks.append((stem, aedat_dir / name, aedat_dir / f"{stem}_labels.csv", out))
        run_in_pool(_split_aedat_files_to_np, tasks)
