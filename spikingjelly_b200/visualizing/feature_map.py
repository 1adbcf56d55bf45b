"""Grid of 2-D feature maps (``spikingjelly/visualizing/feature_map.py:15-142``)."""
from __future__ import annotations

from typing import Tuple

from ._utils import _expect_ndim, _mpl, _to_numpy, feature_map_grid

__all__ = ["plot_2d_feature_map"]


def plot_2d_feature_map(x3d, nrows: int, ncols: int, space: int, title: str, figsize: Tuple[float, float] = (12, 8),
                        dpi: int = 200):
    a = _to_numpy(x3d)
    _expect_ndim(a, 3)
    canvas = feature_map_grid(a, nrows, ncols, space)
    _, plt = _mpl()
    fig, ax = plt.subplots(figsize=figsize, dpi=dpi)
    ax.set_title(title)
    ax.imshow(canvas, cmap="gray")
    ax.get_xaxis().set_visible(False)
    ax.get_yaxis().set_visible(False)
    return fig, ax
