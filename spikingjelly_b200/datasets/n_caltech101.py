"""N-Caltech101: Caltech101 images seen by a moving ATIS sensor, 180 x 240, 101 classes, no official split
(``spikingjelly/datasets/n_caltech101.py:19-293``)."""
from pathlib import Path
from typing import Callable, Optional, Tuple

from torchvision.datasets.utils import extract_archive

from . import utils
from .base import NeuromorphicDatasetFolder, convert_class_tree

__all__ = ["NCaltech101"]


class NCaltech101(NeuromorphicDatasetFolder):
    def __init__(self, root: str, data_type: str = "event", frames_number: int = None, split_by: str = None,
                 duration: int = None, custom_integrate_function: Callable = None,
                 custom_integrated_frames_dir_name: str = None, transform: Optional[Callable] = None,
                 target_transform: Optional[Callable] = None) -> None:
        super().__init__(root, None, data_type, frames_number, split_by, duration, custom_integrate_function,
                         custom_integrated_frames_dir_name, transform, target_transform)

    @classmethod
    def get_H_W(cls) -> Tuple:
        return 180, 240

    @classmethod
    def resource_url_md5(cls) -> list:
        url = "https://www.garrickorchard.com/datasets/n-caltech101"
        return [("Caltech101.zip", url, "66201824eabb0239c7ab992480b50ba3"),
                ("Caltech101_annotations.zip", url, "25e64cea645291e368db1e70f214988e"),
                ("ReadMe(Caltech101)-SINAPSE-G.txt", url, "d464b81684e0af3b5773555eb1d5b95c"),
                ("ReadMe(Caltech101).txt", url, "33632a7a5c46074c70509f960d0dd5e5")]

    @classmethod
    def downloadable(cls) -> bool:
        return False

    @classmethod
    def extract_downloaded_files(cls, download_root: Path, extract_root: Path):
        extract_archive(download_root / "Caltech101.zip", extract_root)

    @classmethod
    def create_raw_from_extracted(cls, extract_root: Path, raw_root: Path):
        convert_class_tree(extract_root / "Caltech101", raw_root, utils._save_atis_bin_as_npz)
