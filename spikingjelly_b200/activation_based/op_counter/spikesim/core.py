"""Reference import path ``op_counter.spikesim.core``."""
from ._impl import SpikeSimEnergyConfig, SpikeSimCounter, SpikeSimEnergyReport, SpikeSimEnergyProfiler, estimate_spikesim_event_energy  # noqa: F401

__all__ = ['SpikeSimEnergyConfig', 'SpikeSimCounter', 'SpikeSimEnergyReport', 'SpikeSimEnergyProfiler', 'estimate_spikesim_event_energy']
