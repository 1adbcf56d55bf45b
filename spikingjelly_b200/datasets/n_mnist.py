"""N-MNIST: MNIST digits recorded by a moving ATIS sensor, 34 x 34, 10 classes
(``spikingjelly/datasets/n_mnist.py:19-304``)."""
import os
from pathlib import Path
from typing import Callable, Optional, Tuple

from . import utils
from .base import NeuromorphicDatasetFolder, convert_class_tree, extract_all

__all__ = ["NMNIST"]


class NMNIST(NeuromorphicDatasetFolder):
    def __init__(self, root: str, train: bool = True, data_type: Optional[str] = "event", frames_number: Optional[int] = None,
                 split_by: Optional[str] = None, duration: Optional[int] = None,
                 custom_integrate_function: Optional[Callable] = None, custom_integrated_frames_dir_name: Optional[str] = None,
                 transform: Optional[Callable] = None, target_transform: Optional[Callable] = None) -> None:
        if train is None:
            raise ValueError("`train` must be `True` or `False`")
        super().__init__(root, train, data_type, frames_number, split_by, duration, custom_integrate_function,
                         custom_integrated_frames_dir_name, transform, target_transform)

    @classmethod
    def get_H_W(cls) -> Tuple:
        return 34, 34

    @classmethod
    def resource_url_md5(cls) -> list:
        url = "https://www.garrickorchard.com/datasets/n-mnist"
        return [("Train.zip", url, "20959b8e626244a1b502305a9e6e2031"), ("Test.zip", url, "69ca8762b2fe404d9b9bad1103e97832")]

    @classmethod
    def downloadable(cls) -> bool:
        return False

    @classmethod
    def extract_downloaded_files(cls, download_root: Path, extract_root: Path):
        extract_all([download_root / f for f in os.listdir(download_root)], extract_root, max_workers=2)

    @classmethod
    def create_raw_from_extracted(cls, extract_root: Path, raw_root: Path):
        for split in ("Train", "Test"):
            target = raw_root / split.lower()
            target.mkdir()
            convert_class_tree(extract_root / split, target, utils._save_atis_bin_as_npz)
