"""SpikeSim crossbar-energy estimate: constants (``config``), stage formulas (``formulas``), the activity counter
(``counter``) and the profiler / one-call estimate (``core``)."""
from .config import SpikeSimEnergyConfig
from .core import SpikeSimEnergyProfiler, SpikeSimEnergyReport, estimate_spikesim_event_energy
from .counter import SpikeSimCounter
from .formulas import compute_spikesim_dense_energy_breakdown, compute_spikesim_event_energy_breakdown

__all__ = ["SpikeSimEnergyConfig", "SpikeSimCounter", "SpikeSimEnergyProfiler", "SpikeSimEnergyReport",
           "estimate_spikesim_event_energy", "compute_spikesim_dense_energy_breakdown", "compute_spikesim_event_energy_breakdown"]
