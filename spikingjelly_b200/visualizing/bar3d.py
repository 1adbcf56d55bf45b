"""One bar chart per column of a ``[T, N]`` array, staggered in depth (``spikingjelly/visualizing/bar3d.py:15-156``)."""
from __future__ import annotations

import numpy as np

from ._utils import _expect_ndim, _mpl, _to_numpy

__all__ = ["plot_2d_bar_in_3d"]


def plot_2d_bar_in_3d(array, title: str, xlabel: str, ylabel: str, zlabel: str, int_x_ticks: bool = True,
                      int_y_ticks: bool = True, int_z_ticks: bool = False, dpi: int = 200):
    a = _to_numpy(array)
    _expect_ndim(a, 2)
    mpl, plt = _mpl()
    fig = plt.figure(dpi=dpi)
    ax = fig.add_subplot(111, projection="3d")
    ax.set_title(title)
    colors = plt.get_cmap("tab10")
    steps = np.arange(a.shape[0])
    for i in range(a.shape[1]):
        ax.bar(steps, a[:, i], i, zdir="x", color=colors(i % 10), alpha=0.8)
    ax.set_xlabel(xlabel)
    ax.set_ylabel(ylabel)
    ax.set_zlabel(zlabel)
    for axis, integer in ((ax.xaxis, int_x_ticks), (ax.yaxis, int_y_ticks), (ax.zaxis, int_z_ticks)):
        axis.set_major_locator(mpl.ticker.MaxNLocator(integer=integer))
    return fig, ax
