"""CIFAR10-DVS frames for the memory-optimisation example: the TEBN split, neuromorphic data augmentation (one of roll /
rotate / cut-out per sample) on the training side, plain resizing on the test side (``examples/memopt/data_module.py`` of the
reference, without the Lightning base class).  ``synthetic=True`` replaces the files by random event frames whose density
depends on the class, so the example runs where the dataset is absent."""
import numpy as np
import torch
from torch.utils.data import DataLoader, TensorDataset


class Cutout:
    """Zero ``n_holes`` square patches of side ``length`` (or a random side below ``max_length``) in the last two axes."""

    def __init__(self, n_holes, length=None, max_length=None):
        self.n_holes, self.length, self.max_length = n_holes, length, max_length

    def __call__(self, img):
        h, w = img.size(-2), img.size(-1)
        mask = torch.ones(h, w, dtype=img.dtype)
        for _ in range(self.n_holes):
            y, x = np.random.randint(h), np.random.randint(w)
            side = self.length if self.max_length is None else np.random.randint(1, self.max_length)
            mask[max(y - side // 2, 0):min(y + side // 2, h), max(x - side // 2, 0):min(x + side // 2, w)] = 0
        return img * mask


class CIFAR10DVSNDA:
    """``M`` operations drawn from {roll by up to ``2N + 1`` pixels, rotate by up to ``15N`` degrees, cut out ``8N`` pixels}."""

    def __init__(self, M=1, N=2):
        self.M, self.N = M, N

    def __call__(self, data):
        from torchvision import transforms
        rotate, cut, a = transforms.RandomRotation(degrees=15 * self.N), Cutout(n_holes=1, length=8 * self.N), self.N * 2 + 1
        ops = (lambda d: torch.roll(d, shifts=(np.random.randint(-a, a + 1), np.random.randint(-a, a + 1)), dims=(2, 3)), rotate, cut)
        for i in np.random.randint(0, len(ops), self.M):
            data = ops[i](data)
        return data


class CIFAR10DVSDataModule:
    def __init__(self, data_dir: str = None, T: int = 10, batch_size: int = 128, num_workers: int = 4, synthetic: bool = False,
                 synthetic_samples: int = 256, resolution: int = 48):
        self.data_dir, self.T, self.batch_size, self.num_workers = data_dir, T, batch_size, num_workers
        self.synthetic, self.synthetic_samples, self.resolution = synthetic or data_dir is None, synthetic_samples, resolution
        self.train_set = self.test_set = None

    def _split(self, train: bool, transform=None):
        from ....datasets.cifar10_dvs import CIFAR10DVSTEBNSplit
        return CIFAR10DVSTEBNSplit(self.data_dir, train=train, data_type="frame", frames_number=self.T, split_by="number", transform=transform)

    def prepare_data(self):
        if not self.synthetic:                            # builds the frame cache once, before workers start
            self._split(True), self._split(False)

    def _synthetic(self, n, seed):
        g = torch.Generator().manual_seed(seed)
        y = torch.randint(0, 10, (n,), generator=g)
        x = (torch.rand(n, self.T, 2, self.resolution, self.resolution, generator=g) < (0.05 + 0.01 * y.view(-1, 1, 1, 1, 1))).float()
        return TensorDataset(x, y)

    def setup(self, stage: str = "fit"):
        if self.synthetic:
            self.train_set, self.test_set = self._synthetic(self.synthetic_samples, 1), self._synthetic(max(self.synthetic_samples // 4, 1), 2)
            return
        import PIL.Image
        from torchvision import transforms
        to_tensor = transforms.Lambda(lambda x: torch.tensor(x, dtype=torch.float32))
        size = (self.resolution, self.resolution)
        self.train_set = self._split(True, transforms.Compose([
            to_tensor, transforms.RandomResizedCrop(128, scale=(0.7, 1.0), interpolation=PIL.Image.NEAREST), transforms.Resize(size=size),
            transforms.RandomHorizontalFlip(p=0.5), CIFAR10DVSNDA(M=1, N=2)]))
        self.test_set = self._split(False, transforms.Compose([to_tensor, transforms.Resize(size=size)]))

    def _loader(self, dataset, train: bool):
        return DataLoader(dataset, batch_size=self.batch_size, shuffle=train, num_workers=0 if self.synthetic else self.num_workers,
                          pin_memory=torch.cuda.is_available(), drop_last=train)

    def train_dataloader(self):
        return self._loader(self.train_set, True)

    def val_dataloader(self):
        return self._loader(self.test_set, False)

    test_dataloader = predict_dataloader = val_dataloader
