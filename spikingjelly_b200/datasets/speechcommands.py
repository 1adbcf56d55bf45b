"""Google Speech Commands as a waveform dataset with a label dictionary, optional synthetic ``_silence_`` samples cut
from the background-noise recordings, and class-balancing sample weights for the training split
(``spikingjelly/datasets/speechcommands.py:32-303``).  Needs ``torchaudio`` to decode audio."""
import os
from pathlib import Path
from random import choice
from typing import Callable, Optional, Tuple

import numpy as np
import torch
from torch import Tensor
from torch.utils.data import Dataset
from torchvision.datasets.utils import download_url, extract_archive, verify_str_arg

__all__ = ["SpeechCommands", "SPEECHCOMMANDS"]

FOLDER_IN_ARCHIVE = "SpeechCommands"
URL = "speech_commands_v0.02"
HASH_DIVIDER = "_nohash_"
EXCEPT_FOLDER = "_background_noise_"
_BASE_URL = "https://storage.googleapis.com/download.tensorflow.org/data/"
_CHECKSUMS = {_BASE_URL + "speech_commands_v0.01.tar.gz": "3cd23799cb2bbdec517f1cc028f8d43c",
              _BASE_URL + "speech_commands_v0.02.tar.gz": "6b74f3901214cb2c2934e98196829835"}
VAL_RECORD, TEST_RECORD, TRAIN_RECORD = "validation_list.txt", "testing_list.txt", "training_list.txt"


def _load_audio(path: str):
    import torchaudio
    return torchaudio.load(path)


def _load_speechcommands_item(relpath: str, path: str) -> Tuple[Tensor, int, str, str, int]:
    label, filename = os.path.split(relpath)
    speaker_id, utterance = os.path.splitext(filename)[0].split(HASH_DIVIDER)
    waveform, sample_rate = _load_audio(os.path.join(path, relpath))
    return waveform, sample_rate, label, speaker_id, int(utterance)


def _read_list(path: str):
    with open(path) as f:
        return [line.rstrip("\n") for line in f]


class SpeechCommands(Dataset):
    def __init__(self, label_dict: dict, root: str, silence_cnt: Optional[int] = 0, silence_size: Optional[int] = 16000,
                 transform: Optional[Callable] = None, url: Optional[str] = URL, split: Optional[str] = "train",
                 folder_in_archive: Optional[str] = FOLDER_IN_ARCHIVE, download: Optional[bool] = False) -> None:
        self.split = verify_str_arg(split, "split", ("train", "val", "test"))
        self.label_dict, self.transform = label_dict, transform
        self.silence_cnt, self.silence_size = silence_cnt, silence_size
        if silence_cnt < 0:
            raise ValueError(f"Invalid silence_cnt parameter: {silence_cnt}")
        if silence_size <= 0:
            raise ValueError(f"Invalid silence_size parameter: {silence_size}")
        if url in ("speech_commands_v0.01", "speech_commands_v0.02"):
            url = _BASE_URL + url + ".tar.gz"
        basename = os.path.basename(url)
        archive = os.path.join(root, basename)
        self._path = os.path.join(root, folder_in_archive, basename.rsplit(".", 2)[0])
        if download:
            if not os.path.isdir(self._path):
                if not os.path.isfile(archive):
                    download_url(url, root, md5=_CHECKSUMS.get(url))
                extract_archive(archive, self._path)
        elif not os.path.isdir(self._path):
            raise FileNotFoundError('Audio data not found. Please specify "download=True" and try again.')
        self.noise_list = sorted(str(p) for p in Path(self._path).glob(f"{EXCEPT_FOLDER}/*.wav"))

        if self.split != "train":
            self._walker = _read_list(os.path.join(self._path, VAL_RECORD if self.split == "val" else TEST_RECORD))
            return
        record = os.path.join(self._path, TRAIN_RECORD)
        if os.path.exists(record):
            self._walker = _read_list(record)
        else:
            # everything that is neither a validation nor a test file trains; the list is cached beside the data
            every = {os.path.relpath(str(p), self._path) for p in Path(self._path).glob("*/*.wav")
                     if HASH_DIVIDER in str(p) and EXCEPT_FOLDER not in str(p)}
            held_out = set(_read_list(os.path.join(self._path, VAL_RECORD))) | set(_read_list(os.path.join(self._path, TEST_RECORD)))
            self._walker = sorted(every - held_out)
            with open(record, "w") as f:
                f.write("\n".join(self._walker))
        labels = [self.label_dict.get(os.path.split(rel)[0]) for rel in self._walker]
        class_w = 1.0 / np.unique(labels, return_counts=True)[1]
        silence_w = 1.0 / self.silence_cnt if self.silence_cnt else 0.0
        total = class_w.sum() + silence_w
        self.weights = torch.DoubleTensor([class_w[l] / total for l in labels] + [silence_w / total] * self.silence_cnt)

    def __getitem__(self, n: int) -> Tuple[Tensor, int]:
        if n < len(self._walker):
            waveform, _, label, _, _ = _load_speechcommands_item(self._walker[n], self._path)
        else:
            waveform, _ = _load_audio(choice(self.noise_list))
            offset = np.random.randint(waveform.shape[1] - self.silence_size)
            waveform = waveform[:, offset: offset + self.silence_size]
            label = "_silence_"
        peak = waveform.abs().max()
        if peak > 0:
            waveform = waveform / peak
        if self.transform is not None:
            waveform = self.transform(waveform)
        return waveform, self.label_dict.get(label)

    def __len__(self) -> int:
        return len(self._walker) + self.silence_cnt


SPEECHCOMMANDS = SpeechCommands
