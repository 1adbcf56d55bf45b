"""CIFAR10-DVS: CIFAR-10 images shown to a DVS128, 128 x 128, 10 classes x 1000 samples, stored as AEDAT 2
(big-endian ``(address, timestamp)`` u32 pairs).  ``CIFAR10DVSTEBNSplit`` applies the fixed split used by TEBN:
samples 0-99 of each class test, 100-999 train (``spikingjelly/datasets/cifar10_dvs.py:24-533``)."""
from pathlib import Path
from typing import Callable, Optional, Tuple, Union

import numpy as np

from ..logger import logger
from . import utils
from .base import NeuromorphicDatasetFolder, convert_class_tree, extract_all

__all__ = ["CIFAR10DVS_CLASS_NAMES", "CIFAR10DVS", "CIFAR10DVSTEBNSplit"]

CIFAR10DVS_CLASS_NAMES = ("airplane", "automobile", "bird", "cat", "deer", "dog", "frog", "horse", "ship", "truck")

# Event type codes and the address layout of the DAVIS-style 32-bit event word (the defaults of the reference's generic AEDAT
# reader).  The CIFAR10-DVS files themselves come from a DVS128 and are decoded with the 16-bit layout in ``_load_origin_data``.
EVT_DVS, EVT_APS = 0, 1
y_mask, y_shift = 0x7FC00000, 22
x_mask, x_shift = 0x003FF000, 12
polarity_mask, polarity_shift = 0x800, 11
valid_mask, valid_shift = 0x80000000, 31


def _load_origin_data(file_name: Union[str, Path]) -> dict:
    """AEDAT 2 of the DVS128: skip ``#`` header lines; address bits 1-7 = x, 8-14 = y, bit 0 = polarity; the image
    is mirrored on both axes and the polarity inverted to match the other datasets."""
    with open(file_name, "rb") as f:
        pos = 0
        line = f.readline()
        while line[:1] == b"#":
            pos += len(line)
            line = f.readline()
        f.seek(pos)
        words = np.frombuffer(f.read(), dtype=">u4")
    if words.size % 2:
        raise ValueError(f"odd number of data elements in {file_name}")
    addr, stamp = words[0::2], words[1::2]
    x, y, pol = (addr & 0xFE) >> 1, (addr & 0x7F00) >> 8, (addr & 1).astype(bool)
    return {"t": stamp, "x": 127 - y, "y": 127 - x, "p": 1 - pol.astype(int)}


def _read_aedat_save_to_np(bin_file, np_file):
    ev = _load_origin_data(bin_file)
    utils.np_savez(np_file, t=ev["t"], x=ev["x"], y=ev["y"], p=ev["p"])
    logger.debug("Save [%s] to [%s].", bin_file, np_file)


class CIFAR10DVS(NeuromorphicDatasetFolder):
    _FIGSHARE = {"airplane": (7712788, "0afd5c4bf9ae06af762a77b180354fdd"), "automobile": (7712791, "8438dfeba3bc970c94962d995b1b9bdd"),
                 "bird": (7712794, "a9c207c91c55b9dc2002dc21c684d785"), "cat": (7712812, "52c63c677c2b15fa5146a8daf4d56687"),
                 "deer": (7712815, "b6bf21f6c04d21ba4e23fc3e36c8a4a3"), "dog": (7712818, "f379ebdf6703d16e0a690782e62639c3"),
                 "frog": (7712842, "cad6ed91214b1c7388a5f6ee56d08803"), "horse": (7712851, "e7cbbf77bec584ffbf913f00e682782a"),
                 "ship": (7712836, "41c7bd7d6b251be82557c6cce9a7d5c9"), "truck": (7712839, "89f3922fd147d9aeff89e76a2b0b70a7")}

    def __init__(self, root: str, data_type: str = "event", frames_number: int = None, split_by: str = None,
                 duration: int = None, custom_integrate_function: Callable = None,
                 custom_integrated_frames_dir_name: str = None, transform: Optional[Callable] = None,
                 target_transform: Optional[Callable] = None):
        super().__init__(root, None, data_type, frames_number, split_by, duration, custom_integrate_function,
                         custom_integrated_frames_dir_name, transform, target_transform)

    @classmethod
    def get_H_W(cls) -> Tuple:
        return 128, 128

    @classmethod
    def resource_url_md5(cls) -> list:
        return [(f"{name}.zip", f"https://ndownloader.figshare.com/files/{fid}", md5) for name, (fid, md5) in cls._FIGSHARE.items()]

    @classmethod
    def downloadable(cls) -> bool:
        return True

    @classmethod
    def extract_downloaded_files(cls, download_root: Path, extract_root: Path):
        extract_all(list(download_root.iterdir()), extract_root, max_workers=10)

    @classmethod
    def create_raw_from_extracted(cls, extract_root: Path, raw_root: Path):
        convert_class_tree(extract_root, raw_root, _read_aedat_save_to_np)


def _move_data(root: Union[str, Path]):
    root = Path(root)
    for cn in CIFAR10DVS_CLASS_NAMES:
        for split, ids in (("test", range(100)), ("train", range(100, 1000))):
            target = root / split / cn
            if target.exists():
                continue
            target.mkdir(parents=True)
            for i in ids:
                (target / f"cifar10_{cn}_{i}.npz").symlink_to(root / cn / f"cifar10_{cn}_{i}.npz")


class CIFAR10DVSTEBNSplit(CIFAR10DVS):
    def __init__(self, root: str, train: bool = True, data_type: str = "event", frames_number: int = None,
                 split_by: str = None, duration: int = None, custom_integrate_function: Callable = None,
                 custom_integrated_frames_dir_name: str = None, transform: Optional[Callable] = None,
                 target_transform: Optional[Callable] = None):
        if train is None:
            raise ValueError("`train` must be `True` or `False`")
        self._configure(root, train, data_type, frames_number, split_by, duration, custom_integrate_function,
                        custom_integrated_frames_dir_name, transform, target_transform)
        loader = self._prepare()
        split_root = self.processed_root / ("train" if train else "test")
        if not split_root.exists():
            logger.info("Splitting [%s] into train/test following TEBN.", self.processed_root)
            _move_data(self.processed_root)
        self._index(split_root, loader)
