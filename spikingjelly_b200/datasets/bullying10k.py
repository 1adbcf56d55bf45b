"""Bullying10K (classification): 10 interaction classes recorded with a DAVIS346, 260 x 346; every fifth file in
directory-walk order is a test sample, as in the dataset's own loader
(``spikingjelly/datasets/bullying10k.py:21-331``)."""
import os
import shutil
from pathlib import Path
from typing import Callable, List, Optional, Tuple

import numpy as np

from . import utils
from .base import NeuromorphicDatasetFolder, extract_all, run_in_pool

__all__ = ["BULLYING10K_CATEGORY_LABEL", "Bullying10kClassification"]

BULLYING10K_CATEGORY_LABEL = {"handshake": 0, "slapping": 1, "punching": 2, "walking": 3, "fingerguess": 4,
                              "strangling": 5, "greeting": 6, "pushing": 7, "hairgrabs": 8, "kicking": 9}

_FILES = {"handshake": (41268834, "681d70f499e736a1e805305284ddc425"), "slapping": (41247021, "84b41d6805958f9f62f425223916ffc2"),
          "punching": (41263314, "40954f480ab210099d448b7b88fc4719"), "walking": (41247024, "56e4cac9c0814ce701c3b2292c15b6a9"),
          "fingerguess": (41253057, "f83114e5b4f0ea57cac86fb080c7e4d7"), "strangling": (41261904, "8185ecd6f3147e9b609d22f06270aa86"),
          "greeting": (41268792, "4a763fad728b04c8356db8544f1121fe"), "pushing": (41268951, "7986c74ade7149a98672120a89b13ba8"),
          "hairgrabs": (41277855, "a9cf690ed0a3305da4a4b8e110f64db1"), "kicking": (41278008, "6c3218f977de4ac29c84a10b17779c33")}


def _convert_npy_to_npz(src_path: Path, dst_dir: Path, label: int):
    """A source file is an object array of packets of ``(t, x, y, p, ...)`` records."""
    records = [rec for packet in np.load(src_path, allow_pickle=True) for rec in packet]
    cols = [np.array([r[k] for r in records]) for k in range(4)]
    utils.np_savez(Path(dst_dir) / str(label) / f"{Path(src_path).stem}.npz", t=cols[0], x=cols[1], y=cols[2], p=cols[3])


class Bullying10kClassification(NeuromorphicDatasetFolder):
    def __init__(self, root: str, train: bool = True, data_type: str = "event", frames_number: int = None,
                 split_by: str = None, duration: int = None, custom_integrate_function: Callable = None,
                 custom_integrated_frames_dir_name: str = None, transform: Optional[Callable] = None,
                 target_transform: Optional[Callable] = None):
        if train is None:
            raise ValueError("The argument `train` must be specified as a boolean value.")
        super().__init__(root, train, data_type, frames_number, split_by, duration, custom_integrate_function,
                         custom_integrated_frames_dir_name, transform, target_transform)

    @classmethod
    def get_H_W(cls) -> Tuple:
        return 260, 346

    @classmethod
    def resource_url_md5(cls) -> List[Tuple[str, str, str]]:
        return [(f"{name}.zip", f"https://figshare.com/ndownloader/files/{fid}", md5) for name, (fid, md5) in _FILES.items()]

    @classmethod
    def downloadable(cls) -> bool:
        return True

    @classmethod
    def extract_downloaded_files(cls, download_root: Path, extract_root: Path):
        archives = []
        for name in os.listdir(download_root):
            if name.endswith(".zip"):
                archives.append(download_root / name)
            else:
                shutil.copy(download_root / name, extract_root / name)       # annotation json files
        extract_all(archives, extract_root, max_workers=10)

    @classmethod
    def create_raw_from_extracted(cls, extract_root: Path, raw_root: Path):
        for split in ("train", "test"):
            (raw_root / split).mkdir()
            for label in range(10):
                (raw_root / split / str(label)).mkdir()
        files = []
        for c in os.listdir(extract_root):
            if c.endswith(".json") or c.startswith("."):
                continue
            for d, _, names in os.walk(extract_root / c):
                files += [(Path(d) / n, BULLYING10K_CATEGORY_LABEL[c]) for n in names]
        tasks = [(path, raw_root / ("test" if i % 5 == 0 else "train"), label) for i, (path, label) in enumerate(files)]
        run_in_pool(_convert_npy_to_npz, tasks)
        shutil.rmtree(extract_root)          # the extracted object arrays are several times larger than the result
