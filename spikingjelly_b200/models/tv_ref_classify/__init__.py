"""Helpers of the classification trainer: metric meters, distributed set-up, augmentation presets,
batch-level mixup / cutmix and the repeated-augmentation sampler."""
from . import presets, sampler, transforms, utils  # noqa: F401
