"""Memory-residency counting under the NeuroMC name (``op_counter/neuromc/memory_residency_counter.py`` of the reference):
the generic residency counter, with the capacities of the NeuroMC hierarchy when none are given."""
from __future__ import annotations

from typing import Any, Callable, Dict, Optional

from ..memory_residency import MemoryResidencyCounter, MemoryResidencySimulator
from .config import MemoryHierarchyConfig

__all__ = ["NeuroMCMemoryResidencyCounter", "MemoryResidencySimulator"]


class NeuroMCMemoryResidencyCounter(MemoryResidencyCounter):
    """``capacity_bits``: ``{"reg": ..., "sram": ..., "dram": ...}``.  Passing a :class:`MemoryHierarchyConfig` as
    ``config`` derives them from its instances: the registers of one processing element, the two shared SRAM buffers,
    and the DRAM."""

    def __init__(self, extra_rules: Optional[Dict[Any, Callable]] = None, extra_ignore_modules: Optional[list] = None, *,
                 config: Any = None, capacity_bits: Optional[Dict[str, float]] = None):
        if capacity_bits is None and isinstance(config, MemoryHierarchyConfig):
            inst = config.memory_instances
            capacity_bits = {"reg": float(sum(inst[n].size_bits for n in ("reg_1b", "reg_16b", "reg_32b"))),
                             "sram": float(inst["sram_2MB"].size_bits + inst["sram_6MB"].size_bits), "dram": float(inst["dram"].size_bits)}
            config = None
        super().__init__(config=config, capacity_bits=capacity_bits, extra_rules=extra_rules, extra_ignore_modules=extra_ignore_modules)
