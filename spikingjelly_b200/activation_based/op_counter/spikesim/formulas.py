"""Closed-form energy of one convolution stage from its counted activity, dense and event-driven accounting
(``op_counter/spikesim/formulas.py`` of the reference)."""
from __future__ import annotations

import math
from typing import Any, Dict, Mapping

from .config import ROW_DIVISOR, SpikeSimEnergyConfig

__all__ = ["compute_spikesim_dense_energy_breakdown", "compute_spikesim_event_energy_breakdown"]


def compute_spikesim_dense_energy_breakdown(stats: Mapping[str, Any], metadata: Mapping[str, Any],
                                            config: SpikeSimEnergyConfig) -> Dict[str, float]:
    total = float(stats["dense_pe_cycle_count"]) * config.pe_cycle_energy_for_kernel_pj(metadata["kernel_size"])
    return {"pe_cycle_pj": total, "total_pj": total}


def compute_spikesim_event_energy_breakdown(stats: Mapping[str, Any], metadata: Mapping[str, Any],
                                            config: SpikeSimEnergyConfig) -> Dict[str, float]:
    if config.activity_mode != "event":
        return compute_spikesim_dense_energy_breakdown(stats, metadata, config)
    q = float(metadata["out_channel_tiles"])
    p = math.ceil(metadata["in_channels"] / config.xbar_size)
    patch = q * float(stats["active_patch_tile_count"]) * config.patch_control_energy_pj
    rows_by_tile, tile_channels = stats.get("active_row_count_by_tile"), metadata.get("input_tile_channels")
    if (rows_by_tile is None) != (tile_channels is None):
        raise ValueError("active_row_count_by_tile and input_tile_channels must either both be present or both be absent.")
    if rows_by_tile is not None:
        if len(rows_by_tile) != len(tile_channels):
            raise ValueError("active_row_count_by_tile and input_tile_channels must have the same length, but got "
                             f"len(active_row_count_by_tile)={len(rows_by_tile)} and len(input_tile_channels)={len(tile_channels)}.")
        xbar = q * sum(float(r) * config.xbar_row_energy_pj(int(c)) for r, c in zip(rows_by_tile, tile_channels))
    else:
        xbar = q * float(stats["active_row_count"]) * config.xbar_row_energy_pj(metadata["in_channels"])
    neuron = float(p) * float(stats["active_output_tile_site_count"]) * config.neuron_pj
    return {"patch_control_pj": patch, "xbar_pj": xbar, "neuron_pj": neuron, "total_pj": patch + xbar + neuron}


# ------------------------------------------------------------------------------------------------------------- counter
