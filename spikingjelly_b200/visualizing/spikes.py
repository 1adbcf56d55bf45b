"""Spike rasters (with per-neuron firing rate) and the voltage/spike trace of one neuron
(``spikingjelly/visualizing/spikes.py:15-359``)."""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np

from ._utils import _expect_ndim, _mpl, _to_numpy, firing_rates, spike_events

__all__ = ["plot_1d_spikes", "plot_one_neuron_v_s"]


def plot_1d_spikes(spikes, title: str, xlabel: str, ylabel: str, int_x_ticks: bool = True, int_y_ticks: bool = True,
                   plot_firing_rate: bool = True, firing_rate_map_title: str = "firing rate",
                   figsize: Tuple[float, float] = (12, 8), dpi: int = 200):
    """``spikes[T, N]``: one raster row per neuron; optionally a narrow column with each neuron's mean rate."""
    s = _to_numpy(spikes)
    _expect_ndim(s, 2)
    mpl, plt = _mpl()
    T, N = s.shape
    if plot_firing_rate:
        fig = plt.figure(tight_layout=True, figsize=figsize, dpi=dpi)
        grid = mpl.gridspec.GridSpec(1, 5)
        raster, rate_ax = fig.add_subplot(grid[0, 0:4]), fig.add_subplot(grid[0, 4])
    else:
        fig, raster = plt.subplots(figsize=figsize, dpi=dpi)
    raster.set(title=title, xlabel=xlabel, ylabel=ylabel, xlim=(-0.5, T - 0.5), ylim=(-0.5, N - 0.5))
    for axis, integer in ((raster.xaxis, int_x_ticks), (raster.yaxis, int_y_ticks)):
        axis.set_major_locator(mpl.ticker.MaxNLocator(integer=integer))
        axis.set_minor_locator(mpl.ticker.NullLocator())
    raster.invert_yaxis()
    colors = plt.get_cmap("tab10")
    for i, times in enumerate(spike_events(s)):
        raster.eventplot(times, lineoffsets=i, colors=colors(i % 10))
    if plot_firing_rate:
        rate = firing_rates(s)
        hi, lo = rate.max(), rate.min()
        rate_ax.yaxis.set_major_locator(mpl.ticker.MaxNLocator(integer=True))
        rate_ax.yaxis.set_minor_locator(mpl.ticker.NullLocator())
        rate_ax.imshow(rate, cmap="magma", aspect="auto")
        for i in range(N):
            dark_cell = rate[i, 0] < 0.7 * hi or lo == hi
            rate_ax.text(0, i, f"{rate[i, 0]:.2f}", ha="center", va="center", color="w" if dark_cell else "black")
        rate_ax.get_xaxis().set_visible(False)
        rate_ax.set_title(firing_rate_map_title)
    return fig, raster


def plot_one_neuron_v_s(v, s, v_threshold: float = 1.0, v_reset: Optional[float] = 0.0,
                        title: str = "$V[t]$ and $S[t]$ of the neuron", figsize: Tuple[float, float] = (12, 8), dpi: int = 200):
    """Upper two thirds: membrane potential with threshold (and reset) lines; lower third: the spike train."""
    v, s = _to_numpy(v), _to_numpy(s)
    _expect_ndim(v, 1, "v")
    _expect_ndim(s, 1, "s")
    mpl, plt = _mpl()
    fig = plt.figure(figsize=figsize, dpi=dpi)
    T = s.shape[0]
    ax_v = plt.subplot2grid((3, 1), (0, 0), rowspan=2)
    ax_v.set_title(title)
    ax_v.plot(np.arange(T), v)
    ax_v.set_xlim(-0.5, T - 0.5)
    ax_v.set_ylabel("voltage")
    ax_v.axhline(v_threshold, label="$V_{threshold}$", linestyle="-.", c="r")
    if v_reset is not None:
        ax_v.axhline(v_reset, label="$V_{reset}$", linestyle="-.", c="g")
    ax_v.legend(frameon=True)
    ax_s = plt.subplot2grid((3, 1), (2, 0))
    ax_s.eventplot(np.flatnonzero(s == 1), lineoffsets=0, colors="r")
    ax_s.set_xlim(-0.5, T - 0.5)
    ax_s.set_xlabel("simulating step")
    ax_s.set_ylabel("spike")
    ax_s.set_yticks([])
    ax_s.xaxis.set_major_locator(mpl.ticker.MaxNLocator(integer=True))
    return fig, ax_v, ax_s
