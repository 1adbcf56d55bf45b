"""Neuromorphic dataset scaffolding: a frozen configuration, one *builder* per representation (raw events,
fixed number of frames, fixed-duration frames, user-defined integration) and the ``DatasetFolder`` subclass
that drives download-check -> extract -> raw ``.npz`` conversion -> build -> index.

Directory contract under ``root`` (``spikingjelly/datasets/base.py:30-1277``): ``download/`` (archives),
``extract/``, ``events_np/`` (one ``.npz`` with ``t, x, y, p`` per sample, class sub-directories, optional
``train``/``test`` level), and one directory per frame representation
(``frames_number_{T}_split_by_{mode}``, ``duration_{d}``, or the custom function's name).
"""
from __future__ import annotations

import abc
import os
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Iterable, Optional, Tuple, Union

import numpy as np
from torchvision.datasets import DatasetFolder
from torchvision.datasets.utils import check_integrity, download_url

from .. import configure
from ..logger import logger
from . import utils

__all__ = ["NeuromorphicDatasetFolder", "NeuromorphicDatasetBuilder", "EventBuilder", "FrameFixedNumberBuilder",
           "FrameFixedDurationBuilder", "FrameCustomIntegrateBuilder", "NeuromorphicDatasetConfig"]


@dataclass(frozen=True)
class NeuromorphicDatasetConfig:
    root: Path
    train: Optional[bool]
    data_type: str = "event"
    frames_number: Optional[int] = None
    split_by: Optional[str] = None
    duration: Optional[int] = None
    custom_integrate_function: Optional[Callable] = None
    custom_integrated_frames_dir_name: Optional[str] = None
    transform: Optional[Callable] = None
    target_transform: Optional[Callable] = None

    def __post_init__(self):
        if self.data_type not in ("event", "frame"):
            raise ValueError(f'data_type must be "event" or "frame", but got {self.data_type}')
        if self.data_type == "event":
            return
        chosen = [self.frames_number is not None, self.duration is not None, self.custom_integrate_function is not None]
        if sum(chosen) != 1:
            raise ValueError('When data_type="frame", one and only one of "frames_number", "duration", or '
                             '"custom_integrate_function" should be set.')
        if self.frames_number is not None:
            if not isinstance(self.frames_number, int) or self.frames_number <= 0:
                raise ValueError("frames_number must be a positive integer")
            if self.split_by not in ("time", "number"):
                raise ValueError('split_by must be "time" or "number"')
        if self.duration is not None and (not isinstance(self.duration, int) or self.duration <= 0):
            raise ValueError("duration must be a positive integer")


def run_in_pool(fn: Callable, tasks: Iterable[tuple], max_workers: Optional[int] = None) -> None:
    """Runs ``fn(*task)`` for every task on a thread pool and re-raises the first failure."""
    workers = max_workers or configure.max_threads_number_for_datasets_preprocess
    workers = max(1, min(workers, os.cpu_count() or 1, configure.max_threads_number_for_datasets_preprocess))
    t0 = time.time()
    with ThreadPoolExecutor(max_workers=workers) as pool:
        for fut in [pool.submit(fn, *task) for task in tasks]:
            fut.result()
    logger.info("Used time = [%ss] with [%s] workers.", round(time.time() - t0, 2), workers)


class NeuromorphicDatasetBuilder(abc.ABC):
    """Turns the raw event tree into one representation; ``build()`` is idempotent per directory."""

    def __init__(self, cfg: NeuromorphicDatasetConfig, raw_root: Path):
        self.cfg, self.raw_root = cfg, raw_root

    @property
    @abc.abstractmethod
    def processed_root(self) -> Path:
        return self.cfg.root / "processed"

    def build(self) -> Tuple[Path, Callable]:
        if self.processed_root.exists():
            logger.info("The directory [%s] already exists.", self.processed_root)
        else:
            self.processed_root.mkdir()
            logger.info("Mkdir [%s].", self.processed_root)
            self.build_impl()
        return self.processed_root, self.get_loader()

    def build_impl(self) -> None:
        raise NotImplementedError

    @abc.abstractmethod
    def get_loader(self) -> Callable:
        ...

    def _run_preprocess_tasks(self, process: Callable, tasks) -> None:
        run_in_pool(process, tasks)

    def _build_from_event_files(self, process: Callable) -> None:
        utils.create_same_directory_structure(self.raw_root, self.processed_root)

        def tasks():
            for event_root, _, files in os.walk(self.raw_root):
                event_root = Path(event_root)
                out = self.processed_root / event_root.relative_to(self.raw_root)
                for name in files:
                    yield event_root / name, out

        self._run_preprocess_tasks(process, tasks())


class EventBuilder(NeuromorphicDatasetBuilder):
    """Raw events are used as they are."""

    def build(self):
        return self.processed_root, self.get_loader()

    @property
    def processed_root(self) -> Path:
        return self.raw_root

    def get_loader(self) -> Callable:
        return np.load


class _FrameBuilder(NeuromorphicDatasetBuilder):
    _event_loader = staticmethod(np.load)

    def __init__(self, cfg: NeuromorphicDatasetConfig, raw_root: Path, H: int, W: int):
        super().__init__(cfg, raw_root)
        self.H, self.W = H, W

    def get_loader(self) -> Callable:
        return utils.load_npz_frames


class FrameFixedNumberBuilder(_FrameBuilder):
    def build_impl(self) -> None:
        self._build_from_event_files(lambda f, out: utils.integrate_events_file_to_frames_file_by_fixed_frames_number(
            self._event_loader, f, out, self.cfg.split_by, self.cfg.frames_number, self.H, self.W, True))

    @property
    def processed_root(self) -> Path:
        return self.cfg.root / f"frames_number_{self.cfg.frames_number}_split_by_{self.cfg.split_by}"


class FrameFixedDurationBuilder(_FrameBuilder):
    def build_impl(self) -> None:
        self._build_from_event_files(lambda f, out: utils.integrate_events_file_to_frames_file_by_fixed_duration(
            self._event_loader, f, out, self.cfg.duration, self.H, self.W, True))

    @property
    def processed_root(self) -> Path:
        return self.cfg.root / f"duration_{self.cfg.duration}"


class FrameCustomIntegrateBuilder(_FrameBuilder):
    def build_impl(self) -> None:
        fn = self.cfg.custom_integrate_function
        self._build_from_event_files(lambda f, out: utils.save_frames_to_npz_and_print(
            out / f.name, fn(self._event_loader(f), self.H, self.W)))

    @property
    def processed_root(self) -> Path:
        name = self.cfg.custom_integrated_frames_dir_name or self.cfg.custom_integrate_function.__name__
        return self.cfg.root / name


class NeuromorphicDatasetFolder(DatasetFolder):
    """Subclasses state the sensor size, the resource list and how to extract / convert; everything else is here."""

    def __init__(self, root: Union[str, Path], train: Optional[bool] = None, data_type: str = "event",
                 frames_number: Optional[int] = None, split_by: Optional[str] = None, duration: Optional[int] = None,
                 custom_integrate_function: Optional[Callable] = None,
                 custom_integrated_frames_dir_name: Optional[str] = None, transform: Optional[Callable] = None,
                 target_transform: Optional[Callable] = None):
        self._configure(root, train, data_type, frames_number, split_by, duration, custom_integrate_function,
                        custom_integrated_frames_dir_name, transform, target_transform)
        loader = self._prepare()
        if self.cfg.train is not None:
            split_root = self.processed_root / ("train" if self.cfg.train else "test")
        else:
            split_root = self.get_root_when_train_is_none(self.processed_root)
        self._index(split_root, loader)

    # ---- construction steps (split so that subclasses with unusual layouts can reuse them)
    def _configure(self, root, train, data_type, frames_number, split_by, duration, custom_integrate_function,
                   custom_integrated_frames_dir_name, transform, target_transform) -> None:
        self.cfg = NeuromorphicDatasetConfig(
            root=Path(root), train=train, data_type=data_type, frames_number=frames_number, split_by=split_by,
            duration=duration, custom_integrate_function=custom_integrate_function,
            custom_integrated_frames_dir_name=custom_integrated_frames_dir_name, transform=transform,
            target_transform=target_transform)

    def _prepare(self) -> Callable:
        self.prepare_raw_dataset()
        self.processed_root, loader = self.get_dataset_builder().build()
        return loader

    def _index(self, split_root: Path, loader: Callable) -> None:
        DatasetFolder.__init__(self, root=split_root, loader=loader, extensions=self.get_extensions(),
                               transform=self.cfg.transform, target_transform=self.cfg.target_transform)

    # ---- layout
    @property
    def raw_root(self) -> Path:
        return self.cfg.root / "events_np"

    @classmethod
    def _fetch(cls, name: str, url: str, md5: Optional[str], download_root: Path) -> None:
        if not cls.downloadable():
            raise NotImplementedError(f"This dataset can not be downloaded by SpikingJelly, please download [{name}] "
                                      f"from [{url}] manually and put files at {download_root}.")
        logger.info("Download [%s] from [%s] to [%s]", name, url, download_root)
        download_url(url=url, root=download_root, filename=name, md5=md5)

    @classmethod
    def _check_downloaded_files(cls, download_root: Path):
        for name, url, md5 in cls.resource_url_md5():
            path = download_root / name
            if check_integrity(fpath=path, md5=md5):
                continue
            logger.warning("The downloaded file [%s] is missing or corrupted.", path)
            if path.exists():
                path.unlink()
            cls._fetch(name, url, md5, download_root)

    @classmethod
    def _download_all_files(cls, download_root: Path):
        resources = cls.resource_url_md5()
        if not cls.downloadable():
            raise NotImplementedError(f"This dataset can not be downloaded by SpikingJelly, please download files manually "
                                      f"and put files at [{download_root}]. The resources file_name, url, and md5 are: "
                                      f"\n{resources}")
        for name, url, md5 in resources:
            cls._fetch(name, url, md5, download_root)

    def prepare_raw_dataset(self):
        if self.raw_root.exists():
            return
        download_root = self.cfg.root / "download"
        if download_root.exists():
            logger.info("The [%s] directory for saving downloaded files already exists, check files...", download_root)
            self._check_downloaded_files(download_root)
        else:
            download_root.mkdir(parents=True)
            self._download_all_files(download_root)
        extract_root = self.cfg.root / "extract"
        if extract_root.exists():
            logger.warning("The extracted directory [%s] already exists; its integrity is not checked. Delete it manually "
                           "if it is corrupted.", extract_root)
        else:
            extract_root.mkdir()
            self.extract_downloaded_files(download_root, extract_root)
        self.raw_root.mkdir(exist_ok=True)
        logger.info("Start to convert the extracted dataset from [%s] to raw dataset in [%s].", extract_root, self.raw_root)
        self.create_raw_from_extracted(extract_root, self.raw_root)

    def get_dataset_builder(self):
        if self.cfg.data_type == "event":
            return EventBuilder(self.cfg, self.raw_root)
        H, W = self.get_H_W()
        if self.cfg.frames_number is not None:
            return FrameFixedNumberBuilder(self.cfg, self.raw_root, H, W)
        if self.cfg.duration is not None:
            return FrameFixedDurationBuilder(self.cfg, self.raw_root, H, W)
        if self.cfg.custom_integrate_function is not None:
            return FrameCustomIntegrateBuilder(self.cfg, self.raw_root, H, W)
        raise NotImplementedError("Please specify the frames number or duration or custom integrate function.")

    def get_root_when_train_is_none(self, _root: Path) -> Path:
        return _root

    @classmethod
    def get_extensions(cls) -> Tuple[str]:
        return (".npy", ".npz")

    # ---- what a dataset declares
    @classmethod
    @abc.abstractmethod
    def get_H_W(cls) -> Tuple[int]:
        ...

    @classmethod
    @abc.abstractmethod
    def resource_url_md5(cls) -> list:
        ...

    @classmethod
    @abc.abstractmethod
    def downloadable(cls) -> bool:
        ...

    @classmethod
    @abc.abstractmethod
    def extract_downloaded_files(cls, download_root: Path, extract_root: Path):
        ...

    @classmethod
    @abc.abstractmethod
    def create_raw_from_extracted(cls, extract_root: Path, raw_root: Path):
        ...


# ---- helpers shared by the concrete datasets -----------------------------------------------------
def extract_all(archives: Iterable[Path], extract_root: Path, max_workers: int = 4) -> None:
    from torchvision.datasets.utils import extract_archive
    run_in_pool(extract_archive, [(a, extract_root) for a in archives], max_workers)


def convert_class_tree(source_root: Path, target_root: Path, convert: Callable[[Path, Path], None]) -> None:
    """``source_root/<class>/<file>`` -> ``target_root/<class>/<stem>.npz`` through ``convert(src, dst)``."""
    tasks = []
    for class_name in sorted(os.listdir(source_root)):
        src_dir = source_root / class_name
        if not src_dir.is_dir():
            continue
        dst_dir = target_root / class_name
        dst_dir.mkdir()
        tasks += [(src_dir / f, dst_dir / (os.path.splitext(f)[0] + ".npz")) for f in sorted(os.listdir(src_dir))]
    run_in_pool(convert, tasks)


def link_tree(source_root: Path, target_root: Path) -> None:
    """Mirrors ``source_root/<class>/<file>`` as symbolic links."""
    for class_name in sorted(os.listdir(source_root)):
        src_dir = source_root / class_name
        if not src_dir.is_dir():
            continue
        dst_dir = target_root / class_name
        dst_dir.mkdir(parents=True, exist_ok=True)
        for f in os.listdir(src_dir):
            (dst_dir / f).symlink_to(src_dir / f)
