"""DVS-Lip: 100 spoken words recorded with a DAVIS346 and cropped to the mouth, 128 x 128; samples are ``.npy``
structured arrays with fields ``t, x, y, p`` (field access makes them interchangeable with the ``.npz`` files of the
other datasets) (``spikingjelly/datasets/dvs_lip.py:14-180``)."""
from pathlib import Path
from typing import Callable, Optional, Tuple

from torchvision.datasets.utils import extract_archive

from .base import NeuromorphicDatasetFolder, link_tree

__all__ = ["DVSLip"]


class DVSLip(NeuromorphicDatasetFolder):
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
        return 128, 128

    @classmethod
    def resource_url_md5(cls) -> list:
        return [("DVS-Lip.zip", "https://sites.google.com/view/event-based-lipreading", "2dcb959255122d4cdeb6094ca282494b")]

    @classmethod
    def downloadable(cls) -> bool:
        return False

    @classmethod
    def extract_downloaded_files(cls, download_root: Path, extract_root: Path):
        extract_archive(download_root / "DVS-Lip.zip", extract_root)

    @classmethod
    def create_raw_from_extracted(cls, extract_root: Path, raw_root: Path):
        for split in ("train", "test"):
            (raw_root / split).mkdir()
            link_tree(extract_root / "DVS-Lip" / split, raw_root / split)
