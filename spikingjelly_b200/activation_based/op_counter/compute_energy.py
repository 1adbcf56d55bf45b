"""Compute-energy estimate: ``E = #MAC * e_mac + #AC * e_ac`` (45 nm figures of Horowitz, ISSCC 2014,
by default), measured by running the model once under the counters.
Parity: ``spikingjelly/activation_based/op_counter/compute_energy.py:16-371``."""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from ...logger import logger
from .base import DispatchCounterMode, call_model
from .counters import ACCounter, FlopCounter, MACCounter, SynOpCounter

__all__ = ["ComputeEnergyCostConfig", "ComputeEnergyConfig", "ComputeEnergyProfiler", "ComputeEnergyReport", "estimate_compute_energy"]


@dataclass
class ComputeEnergyCostConfig:
    """Energy per operation in pJ."""
    e_mac_pj: float = 4.6
    e_ac_pj: float = 0.9

    @classmethod
    def fp32(cls):
        return cls(4.6, 0.9)

    @classmethod
    def fp16(cls):
        return cls(1.5, 0.4)

    @classmethod
    def int8(cls):
        return cls(0.23, 0.03)


@dataclass
class ComputeEnergyConfig:
    strict: bool = False
    cost_config: ComputeEnergyCostConfig = field(default_factory=ComputeEnergyCostConfig)
    extra_ignore_modules: Optional[List[type]] = None


@dataclass
class ComputeEnergyReport:
    energy_total_pj: float
    energy_mac_pj: float
    energy_ac_pj: float
    breakdown_pj: Dict[str, float]              # {"mac_pj", "ac_pj"}
    counts: Dict[str, int]
    warnings: List[str]
    per_module_pj: Dict[str, float] = field(default_factory=dict, compare=False)     # energy by module scope ("Global" = all)


class ComputeEnergyProfiler:
    """Context manager: everything executed inside is counted; ``report()`` afterwards."""

    def __init__(self, *, config: Optional[ComputeEnergyConfig] = None):
        self.config = copy.deepcopy(config or ComputeEnergyConfig())
        ignore = list(self.config.extra_ignore_modules or [])
        self.mac_counter, self.ac_counter = MACCounter(extra_ignore_modules=ignore), ACCounter(extra_ignore_modules=ignore)
        self.synop_counter, self.flop_counter = SynOpCounter(extra_ignore_modules=ignore), FlopCounter(extra_ignore_modules=ignore)
        self._mode = DispatchCounterMode([self.mac_counter, self.ac_counter, self.synop_counter, self.flop_counter], strict=False)

    def __enter__(self):
        for c in (self.mac_counter, self.ac_counter, self.synop_counter, self.flop_counter):
            c.reset()
        self._mode.__enter__()
        return self

    def __exit__(self, *exc):
        return self._mode.__exit__(*exc)

    def report(self) -> ComputeEnergyReport:
        cost = self.config.cost_config
        mac, ac = self.mac_counter.get_total(), self.ac_counter.get_total()
        synop, flop = self.synop_counter.get_total(), self.flop_counter.get_total()
        e_mac, e_ac = mac * cost.e_mac_pj, ac * cost.e_ac_pj
        per_module = {}
        for scope in set(self.mac_counter.records) | set(self.ac_counter.records):
            per_module[scope] = sum(self.mac_counter.records[scope].values()) * cost.e_mac_pj + \
                sum(self.ac_counter.records[scope].values()) * cost.e_ac_pj
        notes = []
        counters = (self.mac_counter, self.ac_counter, self.synop_counter, self.flop_counter)
        if not any(c.get_counts().get("Global") for c in counters):
            message = ("ComputeEnergyProfiler did not match any supported operators. "
                       "The model may not contain supported operators for this estimator.")
            if self.config.strict:
                raise RuntimeError(message)
            notes.append(message)
        rep = ComputeEnergyReport(e_mac + e_ac, e_mac, e_ac, {"mac_pj": e_mac, "ac_pj": e_ac},
                                  {"mac": mac, "ac": ac, "synop": synop, "flop": flop}, notes, per_module)
        logger.info("compute_energy_summary total_pj=%.3f mac=%s ac=%s synop=%s flop=%s", rep.energy_total_pj, mac, ac, synop, flop)
        return rep

    # the reference's accessor names
    def get_report(self) -> ComputeEnergyReport:
        return self.report()

    def get_total(self) -> float:
        return self.report().energy_total_pj

    def get_counts(self) -> dict:
        return self.report().counts


def estimate_compute_energy(model: nn.Module, inputs, *, config: Optional[ComputeEnergyConfig] = None, reset: bool = True) -> ComputeEnergyReport:
    """One inference pass of ``model`` on ``inputs`` under the profiler (neuron state reset afterwards)."""
    prof = ComputeEnergyProfiler(config=config)
    with torch.no_grad(), prof:
        call_model(model, inputs)
    if reset:
        from .. import functional
        functional.reset_net(model)
    return prof.report()
