"""Helpers around the training loop that are not part of the SNN API itself."""
from .prefetch import DeferredScalar, DevicePrefetcher

__all__ = ["DevicePrefetcher", "DeferredScalar"]
