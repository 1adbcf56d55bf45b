"""Train / eval image pipelines for classification (torchvision transforms).

Parity: ``spikingjelly/activation_based/model/tv_ref_classify/presets.py:6-108``.
"""
from __future__ import annotations

import torch
from torchvision.transforms import autoaugment, transforms
from torchvision.transforms.functional import InterpolationMode

__all__ = ["ClassificationPresetTrain", "ClassificationPresetEval"]

IMAGENET_MEAN, IMAGENET_STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)


class ClassificationPresetTrain:
    """random-resized-crop, flip, optional auto-augment policy (``"ra"``, ``"ta_wide"`` or an
    AutoAugment policy name), to-tensor, normalise, optional random erasing."""

    def __init__(self, crop_size, mean=IMAGENET_MEAN, std=IMAGENET_STD, interpolation=InterpolationMode.BILINEAR,
                 hflip_prob=0.5, auto_augment_policy=None, random_erase_prob=0.0):
        steps = [transforms.RandomResizedCrop(crop_size, interpolation=interpolation)]
        if hflip_prob > 0:
            steps.append(transforms.RandomHorizontalFlip(hflip_prob))
        if auto_augment_policy is not None:
            if auto_augment_policy == "ra":
                steps.append(autoaugment.RandAugment(interpolation=interpolation))
            elif auto_augment_policy == "ta_wide":
                steps.append(autoaugment.TrivialAugmentWide(interpolation=interpolation))
            else:
                steps.append(autoaugment.AutoAugment(policy=autoaugment.AutoAugmentPolicy(auto_augment_policy),
                                                     interpolation=interpolation))
        steps += [transforms.PILToTensor(), transforms.ConvertImageDtype(torch.float), transforms.Normalize(mean=mean, std=std)]
        if random_erase_prob > 0:
            steps.append(transforms.RandomErasing(p=random_erase_prob))
        self.transforms = transforms.Compose(steps)

    def __call__(self, img):
        return self.transforms(img)


class ClassificationPresetEval:
    """resize, centre crop, to-tensor, normalise."""

    def __init__(self, crop_size, resize_size=256, mean=IMAGENET_MEAN, std=IMAGENET_STD,
                 interpolation=InterpolationMode.BILINEAR):
        self.transforms = transforms.Compose([
            transforms.Resize(resize_size, interpolation=interpolation), transforms.CenterCrop(crop_size),
            transforms.PILToTensor(), transforms.ConvertImageDtype(torch.float), transforms.Normalize(mean=mean, std=std)])

    def __call__(self, img):
        return self.transforms(img)
