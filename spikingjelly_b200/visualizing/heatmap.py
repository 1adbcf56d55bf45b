"""Heat map of a ``[T, N]`` quantity over time (``spikingjelly/visualizing/heatmap.py:15-185``)."""
from __future__ import annotations

from typing import Optional, Tuple

from ._utils import _expect_ndim, _mpl, _to_numpy

__all__ = ["plot_2d_heatmap"]


def plot_2d_heatmap(array, title: str, xlabel: str, ylabel: str, int_x_ticks: bool = True, int_y_ticks: bool = True,
                    plot_colorbar: bool = True, colorbar_y_label: str = "magnitude", x_max: Optional[float] = None,
                    figsize: Tuple[float, float] = (12, 8), dpi: int = 200):
    """``array[t, i]`` is drawn at column ``t``, row ``i``; ``x_max`` rescales the time axis to ``[-0.5, x_max]``."""
    a = _to_numpy(array)
    _expect_ndim(a, 2)
    mpl, plt = _mpl()
    fig, ax = plt.subplots(figsize=figsize, dpi=dpi)
    extent = None if x_max is None else [-0.5, x_max, a.shape[1] - 0.5, -0.5]
    im = ax.imshow(a.T, aspect="auto", extent=extent)
    ax.set(title=title, xlabel=xlabel, ylabel=ylabel)
    for axis, integer in ((ax.xaxis, int_x_ticks), (ax.yaxis, int_y_ticks)):
        axis.set_major_locator(mpl.ticker.MaxNLocator(integer=integer))
        axis.set_minor_locator(mpl.ticker.NullLocator())
    if plot_colorbar:
        bar = fig.colorbar(im)
        bar.ax.set_ylabel(colorbar_y_label, rotation=90, va="top")
        bar.ax.yaxis.set_minor_locator(mpl.ticker.NullLocator())
    return fig, ax
