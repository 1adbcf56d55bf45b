"""Array conversion, lazy matplotlib import and the drawing-independent data preparation of the plots."""
from __future__ import annotations

from typing import List, Tuple, Union

import numpy as np
import torch


def _to_numpy(x: Union[np.ndarray, torch.Tensor]) -> np.ndarray:
    if isinstance(x, torch.Tensor):
        return x.detach().float().cpu().numpy() if x.dtype in (torch.bfloat16, torch.float16) else x.detach().cpu().numpy()
    if isinstance(x, np.ndarray):
        return x
    raise TypeError(f"Expected np.ndarray or torch.Tensor, got {type(x).__name__}")


def _mpl():
    """``(matplotlib, pyplot)``; on a machine without a display the non-interactive Agg canvas is selected."""
    import os
    import matplotlib
    if not os.environ.get("DISPLAY") and not os.environ.get("MPLBACKEND"):
        matplotlib.use("Agg", force=False)
    import matplotlib.gridspec  # noqa: F401
    import matplotlib.pyplot as plt
    import matplotlib.ticker  # noqa: F401
    return matplotlib, plt


def _expect_ndim(a: np.ndarray, ndim: int, what: str = "array") -> None:
    if a.ndim != ndim:
        suffix = f" for {what}" if what in ("v", "s") else ""
        raise ValueError(f"Expected {ndim}D array{suffix}, got {a.ndim}D array instead")


def feature_map_grid(x3d: np.ndarray, nrows: int, ncols: int, space: int) -> np.ndarray:
    """Tiles ``C = nrows * ncols`` maps of ``[C, h, w]`` into one image with ``space`` pixels of the maximum value
    between neighbours (half of it at the borders)."""
    C, h, w = x3d.shape
    if nrows * ncols != C:
        raise ValueError(f"nrows * ncols ({nrows} * {ncols} = {nrows * ncols}) != C ({C})")
    canvas = np.full(((h + space) * nrows, (w + space) * ncols), float(x3d.max()))
    tiles = canvas.reshape(nrows, h + space, ncols, w + space)
    off = space // 2
    tiles[:, off:off + h, :, off:off + w] = x3d.reshape(nrows, ncols, h, w).transpose(0, 2, 1, 3)
    return canvas


def spike_events(spikes_tn: np.ndarray) -> List[np.ndarray]:
    """Per neuron, the time steps at which ``spikes[T, N]`` equals one."""
    return [np.flatnonzero(spikes_tn[:, i] == 1) for i in range(spikes_tn.shape[1])]


def firing_rates(spikes_tn: np.ndarray) -> np.ndarray:
    return spikes_tn.mean(axis=0, keepdims=True).T          # [N, 1]
