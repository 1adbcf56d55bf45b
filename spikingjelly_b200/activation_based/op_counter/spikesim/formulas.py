"""Reference import path ``op_counter.spikesim.formulas``."""
from ._impl import compute_spikesim_dense_energy_breakdown, compute_spikesim_event_energy_breakdown  # noqa: F401

__all__ = ['compute_spikesim_dense_energy_breakdown', 'compute_spikesim_event_energy_breakdown']
