"""NeuroMC energy model: memory hierarchy, primitive-operation counters and the run-time energy profiler."""
from .config import MemoryHierarchyConfig, MemoryInstanceSpec
from .core import NeuroMCEnergyProfiler, NeuroMCRuntimeEnergyReport, estimate_neuromc_runtime_energy
from .counters import (NeuroMCAddCounter, NeuroMCBaseCounter, NeuroMCCmpCounter, NeuroMCMulCounter, NeuroMCMuxCounter, NeuroMCSqrtCounter)
from .memory_residency_counter import NeuroMCMemoryResidencyCounter
from ..memory_residency import MemoryResidencySimulator

__all__ = ["MemoryInstanceSpec", "MemoryHierarchyConfig", "MemoryResidencySimulator", "NeuroMCMemoryResidencyCounter", "NeuroMCEnergyProfiler",
           "NeuroMCRuntimeEnergyReport", "estimate_neuromc_runtime_energy", "NeuroMCBaseCounter", "NeuroMCAddCounter", "NeuroMCMulCounter",
           "NeuroMCCmpCounter", "NeuroMCMuxCounter", "NeuroMCSqrtCounter"]
