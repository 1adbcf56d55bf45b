"""Matplotlib plots for spikes, voltages and feature maps (headless: Agg canvas).  Matplotlib is imported when a
plot function is called, so the package imports on machines without it."""
from .bar3d import plot_2d_bar_in_3d
from .feature_map import plot_2d_feature_map
from .heatmap import plot_2d_heatmap
from .spikes import plot_1d_spikes, plot_one_neuron_v_s

__all__ = ["plot_1d_spikes", "plot_2d_bar_in_3d", "plot_2d_feature_map", "plot_2d_heatmap", "plot_one_neuron_v_s"]
