"""HARDVS (mini release): 300 human-activity classes recorded with a DAVIS346, 260 x 346, train / val / test lists
(``spikingjelly/datasets/hardvs.py:15-188``)."""
import shutil
from pathlib import Path
from typing import Callable, Optional, Tuple

from torchvision.datasets.utils import extract_archive

from .base import NeuromorphicDatasetFolder, run_in_pool

__all__ = ["HARDVS"]


class HARDVS(NeuromorphicDatasetFolder):
    def __init__(self, root: str, train_test_val: str = None, data_type: str = "event", frames_number: int = None,
                 split_by: str = None, duration: int = None, custom_integrate_function: Callable = None,
                 custom_integrated_frames_dir_name: str = None, transform: Optional[Callable] = None,
                 target_transform: Optional[Callable] = None):
        if train_test_val not in ("train", "test", "val"):
            raise ValueError("train_test_val must be 'train', 'test' or 'val'")
        self.train_test_val = train_test_val
        super().__init__(root, None, data_type, frames_number, split_by, duration, custom_integrate_function,
                         custom_integrated_frames_dir_name, transform, target_transform)

    def get_root_when_train_is_none(self, _root: Path):
        return _root / self.train_test_val

    @classmethod
    def get_H_W(cls) -> Tuple:
        return 260, 346

    @classmethod
    def resource_url_md5(cls) -> list:
        url = "https://github.com/Event-AHU/HARDVS"
        return [("MINI_HARDVS_files.zip", url, "9c4cc0d9ba043faa17f6f1a9e9aff982"),
                ("test_label.txt", url, "5b664af5843f9b476a9c22626f7f5a59"),
                ("train_label.txt", url, "0d642b6e6871034f151b2649a89d8d3c"),
                ("val_label.txt", url, "cd2cebcba80e4552102bbacf2b5df812")]

    @classmethod
    def downloadable(cls) -> bool:
        return False

    @classmethod
    def extract_downloaded_files(cls, download_root: Path, extract_root: Path):
        tmp = download_root / "temp_ext"
        tmp.mkdir()
        extract_archive(download_root / "MINI_HARDVS_files.zip", tmp)
        names = [f"action_{i:03d}" for i in range(1, 301)]
        run_in_pool(extract_archive, [(tmp / "MINI_HARDVS_files" / f"{n}.zip", extract_root / n) for n in names], 2)
        shutil.rmtree(tmp)
        for split in ("train", "val", "test"):
            shutil.copy(download_root / f"{split}_label.txt", extract_root / f"{split}_label.txt")

    @classmethod
    def create_raw_from_extracted(cls, extract_root: Path, raw_root: Path):
        for split in ("train", "val", "test"):
            out = raw_root / split
            out.mkdir()
            for i in range(1, 301):
                (out / f"action_{i:03d}").mkdir()
            with open(extract_root / f"{split}_label.txt") as f:
                for line in f:
                    if len(line) <= 1:
                        continue
                    class_name, sample = line.split(" ")[0].split("/")      # "action_001/dvSave-2021_10_15_19_18_02 0"
                    (out / class_name / f"{sample}.npz").symlink_to(extract_root / class_name / f"{sample}.npz")
