"""Spiking Heidelberg Digits (20 classes) and Spiking Speech Commands (35 classes): 700 cochlea channels, HDF5 files
with ragged ``spikes/times`` (seconds), ``spikes/units`` and ``labels``.  Events are ``{"t", "x"}``; frames are
``[T, 700]`` spike counts.  ``duration`` is in milliseconds (``spikingjelly/datasets/shd.py:33-749``)."""
import math
import os
from pathlib import Path
from typing import Callable, Optional, Tuple

import numpy as np

from ..logger import logger
from . import utils
from .base import EventBuilder, NeuromorphicDatasetBuilder, NeuromorphicDatasetConfig, NeuromorphicDatasetFolder, extract_all

__all__ = ["SHD_N_CLASSES", "SpikingHeidelbergDigits", "SSC_N_CLASSES", "SpikingSpeechCommands"]

SHD_N_CLASSES = 20
SSC_N_CLASSES = 35


def _h5py():
    try:
        import h5py
    except ImportError as e:            # pragma: no cover - depends on the environment
        raise ImportError("SHD / SSC need the optional `h5py` package") from e
    return h5py


def _cal_fixed_frames_number_segment_index(events_t: np.ndarray, split_by: str, frames_num: int) -> tuple:
    """As ``utils.cal_fixed_frames_number_segment_index`` but with a real-valued window (times are in seconds)."""
    n = events_t.size
    j_l, j_r = np.zeros(frames_num, dtype=int), np.zeros(frames_num, dtype=int)
    if split_by == "number":
        di = n // frames_num
        j_l[:] = np.arange(frames_num) * di
        j_r[:] = j_l + di
    elif split_by == "time":
        dt = (events_t[-1] - events_t[0]) / frames_num
        for i in range(frames_num):
            lo = dt * i + events_t[0]
            hit = np.flatnonzero((events_t >= lo) & (events_t < lo + dt))
            j_l[i], j_r[i] = hit[0], hit[-1] + 1
    else:
        raise NotImplementedError(split_by)
    j_r[-1] = n
    return j_l, j_r


def _integrate_events_segment_to_frame(x: np.ndarray, W: int, j_l: int = 0, j_r: int = -1) -> np.ndarray:
    return np.bincount(x[j_l:j_r].astype(int), minlength=W)[:W].astype(float)


def _integrate_events_by_fixed_frames_number(events: dict, split_by: str, frames_num: int, W: int) -> np.ndarray:
    j_l, j_r = _cal_fixed_frames_number_segment_index(events["t"], split_by, frames_num)
    return np.stack([_integrate_events_segment_to_frame(events["x"], W, j_l[i], j_r[i]) for i in range(frames_num)])


def _integrate_events_by_fixed_duration(events: dict, duration: int, W: int) -> np.ndarray:
    x, t = events["x"], 1000 * events["t"]
    t = t - t[0]
    frames_num = int(math.ceil(t[-1] / duration))
    bounds = np.searchsorted(t // duration, np.arange(1, frames_num), side="left")
    j_l, j_r = np.concatenate([[0], bounds]).astype(int), np.concatenate([bounds, [t.size]]).astype(int)
    return np.stack([_integrate_events_segment_to_frame(x, W, j_l[i], j_r[i]) for i in range(frames_num)])


def _sample(h5_file, i):
    return {"t": h5_file["spikes"]["times"][i], "x": h5_file["spikes"]["units"][i]}, h5_file["labels"][i]


def _integrate_events_file_to_frames_file_by_fixed_frames_number(h5_file, i, output_dir, split_by, frames_num, W, print_save=False):
    events, label = _sample(h5_file, i)
    fname = os.path.join(output_dir, str(label), str(i))
    utils.np_savez(fname, frames=_integrate_events_by_fixed_frames_number(events, split_by, frames_num, W))
    if print_save:
        logger.debug("Frames [%s] saved.", fname)


def _integrate_events_file_to_frames_file_by_fixed_duration(h5_file, i, output_dir, duration, W, print_save=False):
    events, label = _sample(h5_file, i)
    frames = _integrate_events_by_fixed_duration(events, duration, W)
    fname = os.path.join(output_dir, str(label), str(i))
    utils.np_savez(fname, frames=frames)
    if print_save:
        logger.debug("Frames [%s] saved.", fname)
    return frames.shape[0]


class NullBuilder(EventBuilder):
    def get_loader(self) -> Callable:
        return lambda x: x


class _SHDFrameBuilder(NeuromorphicDatasetBuilder):
    def __init__(self, cfg: NeuromorphicDatasetConfig, raw_root: Path, W: int, dataset_name: str = "shd",
                 splits: Tuple[str] = ("train", "test"), n_classes: int = SHD_N_CLASSES):
        super().__init__(cfg, raw_root)
        self.W, self.dataset_name, self.splits, self.n_classes = W, dataset_name, splits, n_classes

    def _build_samples(self, process: Callable) -> None:
        h5py = _h5py()
        for split in self.splits:
            out = self.processed_root / split
            out.mkdir()
            for c in range(self.n_classes):
                (out / str(c)).mkdir()
            with h5py.File(self.raw_root / f"{self.dataset_name}_{split}.h5") as f:
                self._run_preprocess_tasks(process, ((f, i, out) for i in range(len(f["labels"]))))

    def get_loader(self):
        return utils.load_npz_frames


class SHDFrameFixedNumberBuilder(_SHDFrameBuilder):
    def build_impl(self):
        self._build_samples(lambda f, i, out: _integrate_events_file_to_frames_file_by_fixed_frames_number(
            f, i, out, self.cfg.split_by, self.cfg.frames_number, self.W, True))

    @property
    def processed_root(self) -> Path:
        return self.cfg.root / f"frames_number_{self.cfg.frames_number}_split_by_{self.cfg.split_by}"


class SHDFrameFixedDurationBuilder(_SHDFrameBuilder):
    def build_impl(self):
        self._build_samples(lambda f, i, out: _integrate_events_file_to_frames_file_by_fixed_duration(
            f, i, out, self.cfg.duration, self.W, True))

    @property
    def processed_root(self) -> Path:
        return self.cfg.root / f"duration_{self.cfg.duration}"


class SHDFrameCustomIntegrateBuilder(_SHDFrameBuilder):
    def build_impl(self):
        self._build_samples(lambda f, i, out: self.cfg.custom_integrate_function(f, i, out, self.W))

    @property
    def processed_root(self) -> Path:
        return self.cfg.root / (self.cfg.custom_integrated_frames_dir_name or self.cfg.custom_integrate_function.__name__)


class _H5SpikeDataset(NeuromorphicDatasetFolder):
    """Event mode reads straight from the HDF5 file (a plain map-style dataset); frame mode is a ``DatasetFolder``."""
    _name = "shd"
    _splits: Tuple[str, ...] = ("train", "test")
    _n_classes = SHD_N_CLASSES

    def _init_common(self, split: str, cfg_args: tuple, transform, target_transform):
        self._split = split
        self._configure(*cfg_args)
        loader = self._prepare()
        if self.cfg.data_type == "event":
            self.transform, self.target_transform = transform, target_transform
        else:
            self._index(self.processed_root / split, loader)

    @property
    def raw_root(self) -> Path:
        return self.cfg.root / "events_h5"

    def get_dataset_builder(self):
        if self.cfg.data_type == "event":
            self.h5_file = _h5py().File(self.raw_root / f"{self._name}_{self._split}.h5")
            self.length = len(self.h5_file["labels"])
            return NullBuilder(self.cfg, self.raw_root)
        _, W = self.get_H_W()
        kw = dict(dataset_name=self._name, splits=self._splits, n_classes=self._n_classes)
        if self.cfg.frames_number is not None:
            return SHDFrameFixedNumberBuilder(self.cfg, self.raw_root, W, **kw)
        if self.cfg.duration is not None:
            return SHDFrameFixedDurationBuilder(self.cfg, self.raw_root, W, **kw)
        if self.cfg.custom_integrate_function is not None:
            return SHDFrameCustomIntegrateBuilder(self.cfg, self.raw_root, W, **kw)
        raise NotImplementedError("Please specify the frames number or duration or custom integrate function.")

    @classmethod
    def get_H_W(cls) -> Tuple:
        return None, 700

    @classmethod
    def resource_url_md5(cls) -> list:
        md5 = {"shd_train": "f3252aeb598ac776c1b526422d90eecb", "shd_test": "1503a5064faa34311c398fb0a1ed0a6f"}
        return [(f"{cls._name}_{s}.h5.zip", f"https://zenkelab.org/datasets/{cls._name}_{s}.h5.zip", md5.get(f"{cls._name}_{s}"))
                for s in cls._splits]

    @classmethod
    def downloadable(cls) -> bool:
        return True

    @classmethod
    def extract_downloaded_files(cls, download_root: Path, extract_root: Path):
        extract_all(list(download_root.iterdir()), extract_root, max_workers=2)

    @classmethod
    def create_raw_from_extracted(cls, extract_root: Path, raw_root: Path):
        for f in extract_root.iterdir():
            if not (raw_root / f.name).exists():
                (raw_root / f.name).symlink_to(f)

    def __len__(self):
        return self.length if self.cfg.data_type == "event" else super().__len__()

    def __getitem__(self, index):
        if self.cfg.data_type != "event":
            return super().__getitem__(index)
        events, label = _sample(self.h5_file, index)
        if self.transform is not None:
            events = self.transform(events)
        if self.target_transform is not None:
            label = self.target_transform(label)
        return events, label


class SpikingHeidelbergDigits(_H5SpikeDataset):
    def __init__(self, root: str, train: bool = True, data_type: str = "event", frames_number: Optional[int] = None,
                 split_by: Optional[str] = None, duration: Optional[int] = None,
                 custom_integrate_function: Optional[Callable] = None, custom_integrated_frames_dir_name: Optional[str] = None,
                 transform: Optional[Callable] = None, target_transform: Optional[Callable] = None):
        if train is None:
            raise ValueError("`train` must be `True` or `False`")
        self._init_common("train" if train else "test",
                          (root, train, data_type, frames_number, split_by, duration, custom_integrate_function,
                           custom_integrated_frames_dir_name, transform, target_transform), transform, target_transform)


class SpikingSpeechCommands(_H5SpikeDataset):
    _name = "ssc"
    _splits = ("train", "valid", "test")
    _n_classes = SSC_N_CLASSES

    def __init__(self, root: str, split: str = "train", data_type: str = "event", frames_number: Optional[int] = None,
                 split_by: Optional[str] = None, duration: Optional[int] = None,
                 custom_integrate_function: Optional[Callable] = None, custom_integrated_frames_dir_name: Optional[str] = None,
                 transform: Optional[Callable] = None, target_transform: Optional[Callable] = None):
        self.splits = self._splits
        if split not in self.splits:
            raise ValueError(f"Invalid split: {split}; valid splits are {self.splits}")
        self.split = split
        self._init_common(split, (root, None, data_type, frames_number, split_by, duration, custom_integrate_function,
                                  custom_integrated_frames_dir_name, transform, target_transform), transform, target_transform)

    def get_root_when_train_is_none(self, _root: Path):
        return _root / self.split
