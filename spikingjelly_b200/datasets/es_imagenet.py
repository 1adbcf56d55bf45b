"""ES-ImageNet: ImageNet-1k converted to events by the omnidirectional discrete gradient algorithm, 256 x 256,
samples are ``.npz`` files with ``pos`` / ``neg`` arrays of ``(x, y, t)`` rows
(``spikingjelly/datasets/es_imagenet.py:22-364``)."""
import os
from pathlib import Path
from typing import Callable, Optional, Tuple, Union

import numpy as np

from ..logger import logger
from . import utils
from .base import (EventBuilder, FrameCustomIntegrateBuilder, FrameFixedDurationBuilder, FrameFixedNumberBuilder,
                   NeuromorphicDatasetFolder, link_tree)

__all__ = ["ESImageNet"]

_PART_MD5 = ("900bdd57b5641f7d81cd4620283fef76 5982532009e863a8f4e18e793314c54b 8f408c1f5a1d4604e48d0d062a8289a0 "
             "5c5b5cf0a55954eb639964e3da510097 51feb661b4c9fa87860b63e76b914673 fcd007a2b17b7c13f338734c53f6db31 "
             "d3e74b96d9c5df15714bbc3abcd329fc 65b9cf7fa63e18d2e7d92ff45a42a5e5 241c9a37a83ff9efd305fe46d012211e "
             "ceee96971008e30d0cdc34086c49fd75 4fbfefbe6e48758fbb72427c81f119cf c8cc163be4e5f6451201dccbded4ec24 "
             "08c9dff32f6b42c49ef7cd78e37c728e 43aa157dc5bd5fcea81315a46e0322cf 480a69b050f465ef01efcc44ae29f7df "
             "11abd24d92b93e7f85acd63abd4a18ab 3891486a6862c63a325c5f16cd01fdd1 cf8bb0525b514f411bca9d7c2d681f7c "
             "3766bc35572ccacc03f0f293c571d0ae bf73a5e338644122220e41da7b5630e6 564de4a2609cbb0bb67ffa1bc51f2487 "
             "60a9e52db1acadfccc9a9809073f0b04 373b5484826d40d7ec35f0e1605cb6ea a50612e889b20f99cc7b2725dfd72e9e "
             "0802ccdeb0cff29237faf55164524101").split()


def _load_events(fname: Union[str, Path]):
    """Merges the positive and negative event lists, sorted by time (stable), as ``x, y, t, p`` float arrays; the file's
    first column is the row (y), the second the column (x)."""
    d = np.load(fname)
    pos, neg = d["pos"], d["neg"]
    ev = np.vstack((np.hstack((pos, np.ones((pos.shape[0], 1)))), np.hstack((neg, np.zeros((neg.shape[0], 1))))))
    ev = ev[np.argsort(ev[:, 2])]
    return {"x": ev[:, 1], "y": ev[:, 0], "t": ev[:, 2], "p": ev[:, 3]}


class ESImageNetEventBuilder(EventBuilder):
    def get_loader(self) -> Callable:
        return _load_events


class ESImageNetFrameFixedNumberBuilder(FrameFixedNumberBuilder):
    _event_loader = staticmethod(_load_events)


class ESImageNetFrameFixedDurationBuilder(FrameFixedDurationBuilder):
    _event_loader = staticmethod(_load_events)


class ESImageNetFrameCustomIntegrateBuilder(FrameCustomIntegrateBuilder):
    _event_loader = staticmethod(_load_events)


class ESImageNet(NeuromorphicDatasetFolder):
    def __init__(self, root: str, train: bool = True, data_type: str = "event", frames_number: int = None,
                 split_by: str = None, duration: int = None, custom_integrate_function: Callable = None,
                 custom_integrated_frames_dir_name: str = None, transform: Optional[Callable] = None,
                 target_transform: Optional[Callable] = None):
        if train is None:
            raise ValueError("The argument `train` must be specified as a boolean value.")
        super().__init__(root, train, data_type, frames_number, split_by, duration, custom_integrate_function,
                         custom_integrated_frames_dir_name, transform, target_transform)

    def get_dataset_builder(self):
        if self.cfg.data_type == "event":
            return ESImageNetEventBuilder(self.cfg, self.raw_root)
        H, W = self.get_H_W()
        if self.cfg.frames_number is not None:
            return ESImageNetFrameFixedNumberBuilder(self.cfg, self.raw_root, H, W)
        if self.cfg.duration is not None:
            return ESImageNetFrameFixedDurationBuilder(self.cfg, self.raw_root, H, W)
        if self.cfg.custom_integrate_function is not None:
            return ESImageNetFrameCustomIntegrateBuilder(self.cfg, self.raw_root, H, W)
        raise NotImplementedError("Please specify the frames number or duration or custom integrate function.")

    @classmethod
    def get_H_W(cls) -> Tuple:
        return 256, 256

    @classmethod
    def resource_url_md5(cls) -> list:
        base = "https://cloud.tsinghua.edu.cn/d/94873ab4ec2a4eb497b3/files/?p=%2F{}&dl=1"
        names = [f"ES-imagenet-0.18.part{i:02d}.rar" for i in range(1, 26)]
        return [(n, base.format(n), md5) for n, md5 in zip(names, _PART_MD5)]

    @classmethod
    def downloadable(cls) -> bool:
        return True

    @classmethod
    def extract_downloaded_files(cls, download_root: Path, extract_root: Path):
        """Needs the optional ``rarfile`` package (multi-part archive, opened through its first part)."""
        import rarfile
        with rarfile.RarFile(download_root / "ES-imagenet-0.18.part01.rar") as rf:
            rf.extractall(extract_root)

    @classmethod
    def create_raw_from_extracted(cls, extract_root: Path, raw_root: Path):
        src = extract_root / "ES-imagenet-0.18"
        (raw_root / "train").mkdir()
        link_tree(src / "train", raw_root / "train")
        test = raw_root / "test"
        test.mkdir()
        utils.create_same_directory_structure(src / "train", test)
        names = np.loadtxt(src / "vallabel.txt", delimiter=" ", usecols=(0,), dtype=str)
        labels = np.loadtxt(src / "vallabel.txt", delimiter=" ", usecols=(1,), dtype=int)
        for name, label in zip(np.atleast_1d(names), np.atleast_1d(labels), strict=True):
            (test / f"class{label}" / f"{name}").symlink_to(src / "val" / name)
        logger.info("Files in [%s] are links into [%s]; keep the latter while events are in use.", raw_root, extract_root)
