"""Event-file readers, event -> frame integration, dataset splitting and collation helpers.

Events are dictionaries of equally long 1-D arrays ``t, x, y, p``; frames are ``[T, 2, H, W]`` counts
(channel = polarity).  The integration routines are vectorised (one ``bincount`` per sample instead of
one per frame) but produce exactly the arrays of ``spikingjelly/datasets/utils.py:473-1004``.
"""
from __future__ import annotations

import math
import os
import shutil
import struct
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Callable, Optional, Union

import numpy as np
import torch
import torch.utils.data

from .. import configure
from ..logger import logger

__all__ = [
    "np_savez", "save_as_pic", "save_every_frame_of_an_entire_DVS_dataset", "play_frame", "load_aedat_v3",
    "load_ATIS_bin", "load_npz_frames", "integrate_events_segment_to_frame", "cal_fixed_frames_number_segment_index",
    "integrate_events_by_fixed_frames_number", "integrate_events_file_to_frames_file_by_fixed_frames_number",
    "integrate_events_by_fixed_duration", "integrate_events_file_to_frames_file_by_fixed_duration",
    "save_frames_to_npz_and_print", "create_same_directory_structure", "split_to_train_test_set",
    "fast_split_to_train_test_set", "pad_sequence_collate", "padded_sequence_mask", "create_sub_dataset",
]

np_savez = np.savez_compressed if configure.save_datasets_compressed else np.savez


# ------------------------------------------------------------------------------- pictures
def _frame_to_rgb(frame: np.ndarray) -> np.ndarray:
    """``[2, H, W]`` -> ``[H, W, 3]`` float image: polarity 0 in red, polarity 1 in green."""
    img = np.zeros((frame.shape[1], frame.shape[2], 3), dtype=np.float32)
    img[..., 0], img[..., 1] = frame[0], frame[1]
    return img


def _to_pil(frame):
    from PIL import Image
    return Image.fromarray((np.clip(_frame_to_rgb(frame), 0.0, 1.0) * 255).astype(np.uint8))


def save_as_pic(x: Union[torch.Tensor, np.ndarray], save_pic_to: str = "./", pic_first_name: str = "pic") -> None:
    """Saves every frame of ``x`` (``[T, 2, H, W]``) as ``<pic_first_name>_<t>.png``."""
    x = x.detach().cpu().numpy() if isinstance(x, torch.Tensor) else np.asarray(x)
    for t in range(x.shape[0]):
        _to_pil(x[t]).save(os.path.join(save_pic_to, f"{pic_first_name}_{t}.png"))


def save_every_frame_of_an_entire_DVS_dataset(dataset: str, dataset_path: str, time_steps: int, save_pic_to: str = "./",
                                              number_of_threads: int = 4) -> None:
    """Dumps all frames of the train and test splits of ``DVS128Gesture`` / ``CIFAR10DVS`` / ``NCALTECH101`` as pictures."""
    from . import cifar10_dvs, dvs128_gesture, n_caltech101
    kw = dict(data_type="frame", frames_number=time_steps, split_by="number")
    if dataset == "DVS128Gesture":
        sets = {"train": dvs128_gesture.DVS128Gesture(dataset_path, train=True, **kw),
                "test": dvs128_gesture.DVS128Gesture(dataset_path, train=False, **kw)}
    elif dataset == "CIFAR10DVS":
        sets = {"all": cifar10_dvs.CIFAR10DVS(dataset_path, **kw)}
    elif dataset == "NCALTECH101":
        sets = {"all": n_caltech101.NCaltech101(dataset_path, **kw)}
    else:
        raise ValueError("dataset must be one of 'DVS128Gesture', 'CIFAR10DVS', 'NCALTECH101'")

    def dump(ds, split, lo, hi):
        for i in range(lo, hi):
            frames, label = ds[i]
            out = os.path.join(save_pic_to, split, str(label))
            os.makedirs(out, exist_ok=True)
            save_as_pic(frames, out, f"sample{i}")

    with ThreadPoolExecutor(max_workers=number_of_threads) as pool:
        jobs = []
        for split, ds in sets.items():
            step = max(1, math.ceil(len(ds) / number_of_threads))
            jobs += [pool.submit(dump, ds, split, lo, min(lo + step, len(ds))) for lo in range(0, len(ds), step)]
        for j in jobs:
            j.result()


def play_frame(x: Union[torch.Tensor, np.ndarray], save_gif_to: str = None) -> None:
    """Shows ``[T, 2, H, W]`` frames as an animation, or writes them to a GIF."""
    x = x.detach().cpu().numpy() if isinstance(x, torch.Tensor) else np.asarray(x)
    imgs = [_to_pil(x[t]) for t in range(x.shape[0])]
    if save_gif_to is None:
        from matplotlib import pyplot as plt
        while True:
            for im in imgs:
                plt.imshow(im)
                plt.pause(0.01)
    imgs[0].save(save_gif_to, save_all=True, append_images=imgs[1:], loop=0)
    logger.info("Save frames to [%s].", save_gif_to)


# ------------------------------------------------------------------------------- readers
def load_aedat_v3(file_name: Union[str, Path]) -> dict:
    """AEDAT 3.1 polarity events.  Every packet has a 28-byte header (type u16 @0, event size u32 @4, timestamp
    overflow u32 @12, capacity u32 @16); polarity packets (type 1) hold ``(data u32, timestamp u32)`` pairs with
    ``x = data[17:32]``, ``y = data[2:17]``, ``p = data[1]``."""
    t, x, y, p = [], [], [], []
    with open(file_name, "rb") as f:
        line = f.readline()
        while line.startswith(b"#") and line != b"#!END-HEADER\r\n":
            line = f.readline()
        while True:
            header = f.read(28)
            if len(header) < 28:
                break
            e_type = struct.unpack_from("<H", header, 0)[0]
            e_size, = struct.unpack_from("<I", header, 4)
            overflow, capacity = struct.unpack_from("<I", header, 12)[0], struct.unpack_from("<I", header, 16)[0]
            payload = f.read(e_size * capacity)
            if e_type != 1 or e_size < 8:
                continue
            n = len(payload) // e_size
            words = np.frombuffer(payload[: n * e_size], dtype="<u4").reshape(n, e_size // 4)
            data, stamp = words[:, 0].astype(np.int64), words[:, 1].astype(np.int64)
            x.append((data >> 17) & 0x7FFF)
            y.append((data >> 2) & 0x7FFF)
            p.append((data >> 1) & 1)
            t.append(stamp | (overflow << 31))
    cat = lambda parts: np.concatenate(parts) if parts else np.zeros(0, dtype=np.int64)
    return {"t": cat(t), "x": cat(x), "y": cat(y), "p": cat(p)}


def load_ATIS_bin(file_name: Union[str, Path]) -> dict:
    """N-MNIST / N-Caltech101 binary events: 5 bytes each — ``x``, ``y``, then polarity (1 bit) and a 23-bit timestamp."""
    raw = np.fromfile(file_name, dtype=np.uint8).astype(np.uint32)
    raw = raw[: raw.size // 5 * 5]
    b2 = raw[2::5]
    return {"t": ((b2 & 127) << 16) | (raw[3::5] << 8) | raw[4::5], "x": raw[0::5], "y": raw[1::5], "p": (b2 & 128) >> 7}


def _save_atis_bin_as_npz(bin_file, np_file):
    ev = load_ATIS_bin(bin_file)
    np_savez(np_file, t=ev["t"], x=ev["x"], y=ev["y"], p=ev["p"])
    logger.debug("Save [%s] to [%s].", bin_file, np_file)


def load_npz_frames(file_name: Union[str, Path]) -> np.ndarray:
    return np.load(file_name, allow_pickle=True)["frames"].astype(np.float32)


# ------------------------------------------------------------------------------- integration
def integrate_events_segment_to_frame(x: np.ndarray, y: np.ndarray, p: np.ndarray, H: int, W: int, j_l: int = 0,
                                      j_r: Optional[int] = None) -> np.ndarray:
    """Counts events ``j_l <= j < j_r`` into a ``[2, H, W]`` frame (channel 1 = non-zero polarity)."""
    xs, ys = x[j_l:j_r].astype(np.int64), y[j_l:j_r].astype(np.int64)
    pos = (p[j_l:j_r] != 0).astype(np.int64) * (H * W) + ys * W + xs
    return np.bincount(pos, minlength=2 * H * W).reshape(2, H, W).astype(float)


def cal_fixed_frames_number_segment_index(events_t: np.ndarray, split_by: str, frames_num: int) -> tuple:
    """Left/right event indices of ``frames_num`` slices with equal event count (``"number"``) or equal
    duration (``"time"``, integer ``dt``); the last slice always runs to the final event."""
    n = events_t.size
    j_l, j_r = np.zeros(frames_num, dtype=int), np.zeros(frames_num, dtype=int)
    if split_by == "number":
        di = n // frames_num
        j_l[:] = np.arange(frames_num) * di
        j_r[:] = j_l + di
    elif split_by == "time":
        dt = (events_t[-1] - events_t[0]) // frames_num
        for i in range(frames_num):
            lo = dt * i + events_t[0]
            hit = np.flatnonzero((events_t >= lo) & (events_t < lo + dt))
            j_l[i], j_r[i] = hit[0], hit[-1] + 1
    else:
        raise NotImplementedError(split_by)
    j_r[-1] = n
    return j_l, j_r


def _frames_from_slices(x, y, p, H, W, j_l, j_r) -> np.ndarray:
    """All slices in one ``bincount``: events outside every slice are dropped, overlapping slices fall back."""
    T = len(j_l)
    if T == 0:
        return np.zeros([0, 2, H, W])
    if np.any(j_r[:-1] > j_l[1:]) or np.any(j_r < j_l):
        return np.stack([integrate_events_segment_to_frame(x, y, p, H, W, j_l[i], j_r[i]) for i in range(T)])
    n = x.shape[0]
    idx = np.arange(n)
    frame = np.searchsorted(j_r, idx, side="right")
    frame = np.minimum(frame, T - 1)
    keep = (idx >= j_l[frame]) & (idx < j_r[frame])
    pos = frame[keep] * (2 * H * W) + (p[keep] != 0).astype(np.int64) * (H * W) + y[keep].astype(np.int64) * W + x[keep].astype(np.int64)
    return np.bincount(pos, minlength=T * 2 * H * W).reshape(T, 2, H, W).astype(float)


def integrate_events_by_fixed_frames_number(events: dict, split_by: str, frames_num: int, H: int, W: int) -> np.ndarray:
    t, x, y, p = (events[k] for k in ("t", "x", "y", "p"))
    j_l, j_r = cal_fixed_frames_number_segment_index(t, split_by, frames_num)
    return _frames_from_slices(x, y, p, H, W, j_l, j_r)


def integrate_events_file_to_frames_file_by_fixed_frames_number(loader: Callable, events_np_file: str, output_dir: str,
                                                                split_by: str, frames_num: int, H: int, W: int,
                                                                print_save: bool = False) -> None:
    fname = os.path.join(output_dir, os.path.basename(events_np_file))
    np_savez(fname, frames=integrate_events_by_fixed_frames_number(loader(events_np_file), split_by, frames_num, H, W))
    if print_save:
        logger.debug("Frames [%s] saved.", fname)


def integrate_events_by_fixed_duration(events: dict, duration: int, H: int, W: int) -> np.ndarray:
    """Consecutive windows of ``duration`` time units from the first event; ``ceil(span / duration)`` frames, the
    last one absorbing everything that is left."""
    x, y, p = events["x"], events["y"], events["p"]
    t = events["t"] - events["t"].min()
    frames_num = int(math.ceil(t[-1] / duration))
    bounds = np.searchsorted(t // duration, np.arange(1, frames_num), side="left")
    j_l = np.concatenate([[0], bounds]).astype(int)
    j_r = np.concatenate([bounds, [t.size]]).astype(int)
    return _frames_from_slices(x, y, p, H, W, j_l, j_r)


def integrate_events_file_to_frames_file_by_fixed_duration(loader: Callable, events_np_file: str, output_dir: str,
                                                           duration: int, H: int, W: int, print_save: bool = False) -> int:
    frames = integrate_events_by_fixed_duration(loader(events_np_file), duration, H, W)
    stem, _ = os.path.splitext(os.path.basename(events_np_file))
    fname = os.path.join(output_dir, f"{stem}_{frames.shape[0]}.npz")
    np_savez(fname, frames=frames)
    if print_save:
        logger.debug("Frames [%s] saved.", fname)
    return frames.shape[0]


def save_frames_to_npz_and_print(fname: str, frames: np.ndarray):
    np_savez(fname, frames=frames)
    logger.debug("Frames [%s] saved.", fname)


# ------------------------------------------------------------------------------- directories and splits
def create_same_directory_structure(source_dir: Union[str, Path], target_dir: Union[str, Path]) -> None:
    """Re-creates the sub-directory tree of ``source_dir`` (no files) under the existing ``target_dir``."""
    for name in os.listdir(source_dir):
        src = os.path.join(source_dir, name)
        if os.path.isdir(src):
            dst = os.path.join(target_dir, name)
            os.mkdir(dst)
            logger.debug("Mkdir [%s].", dst)
            create_same_directory_structure(src, dst)


def _class_index(item):
    label = item[1]
    return label.item() if isinstance(label, (np.ndarray, torch.Tensor)) else label


def _split_class_indices(label_idx, train_ratio, random_split):
    train_idx, test_idx = [], []
    for indices in label_idx:
        if random_split:
            np.random.shuffle(indices)
        pos = math.ceil(len(indices) * train_ratio)
        train_idx.extend(indices[:pos])
        test_idx.extend(indices[pos:])
    return train_idx, test_idx


def split_to_train_test_set(train_ratio: float, origin_dataset: torch.utils.data.Dataset, num_classes: int,
                            random_split: bool = False):
    """Per-class split: the first ``ceil(ratio * n_c)`` samples of every class train, the rest test."""
    label_idx = [[] for _ in range(num_classes)]
    for i, item in enumerate(origin_dataset):
        label_idx[_class_index(item)].append(i)
    tr, te = _split_class_indices(label_idx, train_ratio, random_split)
    return torch.utils.data.Subset(origin_dataset, tr), torch.utils.data.Subset(origin_dataset, te)


def fast_split_to_train_test_set(train_ratio: float, origin_dataset: torch.utils.data.Dataset, num_classes: int,
                                 random_split: bool = False, batch_size: int = 16):
    """Same split; the labels are read by a thread pool, or taken from ``.targets`` / ``.samples`` when the dataset
    exposes them (no sample is loaded at all then)."""
    label_idx = [[] for _ in range(num_classes)]
    targets = getattr(origin_dataset, "targets", None)
    if targets is not None and getattr(origin_dataset, "target_transform", None) is None and len(targets) == len(origin_dataset):
        for i, label in enumerate(targets):
            label_idx[int(label)].append(i)
    else:
        n = len(origin_dataset)
        read = lambda lo, hi: [(i, _class_index(origin_dataset[i])) for i in range(lo, hi)]
        with ThreadPoolExecutor() as pool:
            for fut in [pool.submit(read, lo, min(lo + batch_size, n)) for lo in range(0, n, batch_size)]:
                for i, label in fut.result():
                    label_idx[label].append(i)
    tr, te = _split_class_indices(label_idx, train_ratio, random_split)
    return torch.utils.data.Subset(origin_dataset, tr), torch.utils.data.Subset(origin_dataset, te)


def pad_sequence_collate(batch: list):
    """``[(x[T_i, ...], y)]`` -> ``(x padded to [B, T_max, ...], y[B], lengths[B])``."""
    xs = [torch.as_tensor(x) for x, _ in batch]
    return (torch.nn.utils.rnn.pad_sequence(xs, batch_first=True), torch.as_tensor([y for _, y in batch]),
            torch.as_tensor([x.shape[0] for x in xs]))


def padded_sequence_mask(sequence_len: torch.Tensor, T: Optional[int] = None):
    """``mask[t, b] = t < sequence_len[b]`` with shape ``[T, B]``."""
    if T is None:
        T = int(sequence_len.max().item())
    return torch.arange(T, device=sequence_len.device)[:, None] < sequence_len[None, :]


def create_sub_dataset(source_dir: str, target_dir: str, ratio: float, use_soft_link=True, randomly=False):
    """Copies (or links) the first / a random ``ratio`` of every directory's files into a mirror tree."""
    if not os.path.exists(target_dir):
        os.makedirs(target_dir)
    create_same_directory_structure(source_dir, target_dir)
    for root, _, files in os.walk(source_dir, followlinks=True):
        if not files:
            continue
        out = os.path.join(target_dir, os.path.relpath(root, source_dir))
        count = len(files) if ratio >= 1.0 else int(ratio * len(files))
        if count == 0:
            logger.warning("No samples selected from [%s] for output [%s].", root, out)
        if randomly:
            np.random.shuffle(files)
        for name in files[:count]:
            src, dst = os.path.join(root, name), os.path.join(out, name)
            os.symlink(src, dst) if use_soft_link else shutil.copyfile(src, dst)
        logger.debug("[%s] files in [%s] were %s to [%s].", count, root, "linked" if use_soft_link else "copied", out)
