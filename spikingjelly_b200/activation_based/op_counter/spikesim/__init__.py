"""SpikeSim crossbar-energy estimate (``_impl.py``); ``config`` / ``formulas`` / ``counter`` / ``core`` are the import
paths of the reference package."""
from ._impl import (SpikeSimCounter, SpikeSimEnergyConfig, SpikeSimEnergyProfiler, SpikeSimEnergyReport,
                    estimate_spikesim_event_energy)

__all__ = ["SpikeSimEnergyConfig", "SpikeSimCounter", "SpikeSimEnergyProfiler", "SpikeSimEnergyReport",
           "estimate_spikesim_event_energy"]
