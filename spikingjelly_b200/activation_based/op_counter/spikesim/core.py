"""SpikeSim-style energy estimate of the Conv2d inference stages of a spiking network mapped onto in-memory-computing
crossbars (Moitra et al., "SpikeSim"), same figures as the reference's
``spikingjelly/activation_based/op_counter/spikesim/{config,formulas,counter,core}.py``.

A convolution ``[C_out, C_in, kh, kw]`` is tiled onto ``ceil(C_in / B) x ceil(C_out / B)`` crossbars of size ``B``.

* ``activity_mode="dense"`` (SpikeSim's own accounting): every output site costs one processing-element cycle per
  (input tile, output tile) pair; a PE cycle = patch control (H-tree, fetch, tile buffer, subtractors, temporary
  buffer, ADC + mux) + neuron + crossbar array energy scaled by ``B / 8 * kh * kw``.
* ``activity_mode="event"`` (sparse extension): per stage, with binary inputs,
  ``A`` = number of (site, input tile) pairs whose receptive field holds at least one spike,
  ``R`` = number of active crossbar rows (spikes inside receptive fields), per input tile,
  ``Z`` = output tiles x sites with any active input tile;
  energy = ``Q A E_patch + Q sum_tile R_tile E_row(tile) + P Z E_neuron`` with ``P, Q`` the input / output tile counts.
  Non-binary inputs fall back to the dense counts of the same quantities.

Only forward inference of ``nn.Conv2d`` modules (eval mode, grad disabled, groups = 1) is inside the model's scope; anything
else is reported as a warning (or raised with ``strict=True``).
"""
from __future__ import annotations

import math
from collections import defaultdict
from dataclasses import asdict, dataclass, field, replace
from typing import Any, Dict, List, Mapping, Optional, Tuple

import torch
import torch.nn as nn

from ...neuron.base_node import BaseNode, SimpleBaseNode
from ...neuron import IFNode, LIFNode
from ..base import DispatchCounterMode, call_model
from .config import SpikeSimEnergyConfig
from .counter import SpikeSimCounter
from .formulas import compute_spikesim_dense_energy_breakdown, compute_spikesim_event_energy_breakdown

__all__ = ["SpikeSimEnergyReport", "SpikeSimEnergyProfiler", "estimate_spikesim_event_energy"]

try:                                                    # the lightweight neuron variants, when this build has them
    from ...neuron import SimpleIFNode, SimpleLIFNode
    _SUPPORTED_NEURONS: tuple = (IFNode, LIFNode, SimpleIFNode, SimpleLIFNode)
except ImportError:                                     # pragma: no cover
    _SUPPORTED_NEURONS = (IFNode, LIFNode)


@dataclass
class SpikeSimEnergyReport:
    energy_total_pj: float
    energy_by_stage: Dict[str, float]
    energy_by_component: Dict[str, Any]
    event_stats_by_stage: Dict[str, Dict[str, Any]]
    stage_metadata: Dict[str, Dict[str, Any]]
    warnings: List[str]
    breakdown_pj: Dict[str, float]
    counts: Dict[str, int]


class SpikeSimEnergyProfiler:
    """Context manager: run the model inside it, then :meth:`get_report`."""

    def __init__(self, *, config: Optional[SpikeSimEnergyConfig] = None, strict: bool = False):
        self.config = (config or SpikeSimEnergyConfig()).copy()
        self.config.validate()
        self.strict = strict
        self._counter = SpikeSimCounter(config=self.config, strict=strict)
        self._mode = DispatchCounterMode([self._counter], strict=False)
        self._warnings: List[str] = []

    def __enter__(self):
        self._mode.__enter__()
        return self

    def __exit__(self, exc_type, exc, tb):
        return self._mode.__exit__(exc_type, exc, tb)

    def add_warnings(self, messages: List[str]) -> None:
        self._warnings.extend(messages)

    def get_report(self) -> SpikeSimEnergyReport:
        stats, meta = self._counter.get_stage_stats(), self._counter.get_stage_metadata()
        event = self.config.activity_mode == "event"
        fn = compute_spikesim_event_energy_breakdown if event else compute_spikesim_dense_energy_breakdown
        by_stage = {s: fn(stats=st, metadata=meta[s], config=self.config) for s, st in stats.items()}
        totals: Dict[str, float] = defaultdict(float)
        for parts in by_stage.values():
            for k, v in parts.items():
                if k != "total_pj":
                    totals[k] += v
        energy_by_stage = {s: parts["total_pj"] for s, parts in by_stage.items()}
        warnings = list(self._warnings) + list(self._counter.warnings)
        if not energy_by_stage:
            warnings.append("No supported Conv2d forward inference stages were profiled by SpikeSim energy.")
        if event:
            warnings.append("SpikeSim activity_mode='event' is an experimental sparse runtime extension; activity_mode='dense' "
                            "is the original SpikeSim-aligned default.")
        total = sum(energy_by_stage.values())
        totals = dict(totals)
        return SpikeSimEnergyReport(
            energy_total_pj=total, energy_by_stage=energy_by_stage,
            energy_by_component={"totals": {**totals, "total_pj": total}, "by_stage": by_stage},
            event_stats_by_stage=stats, stage_metadata=meta, warnings=warnings, breakdown_pj=totals,
            counts={"dense_pe_cycle_count": int(self._counter.get_total()), "stage_count": len(meta)})

    def get_total(self) -> float:
        return self.get_report().energy_total_pj

    def get_counts(self) -> Dict[str, Any]:
        r = self.get_report()
        return {"event_stats_by_stage": r.event_stats_by_stage, "stage_metadata": r.stage_metadata}


def estimate_spikesim_event_energy(model: nn.Module, inputs, *, config: Optional[SpikeSimEnergyConfig] = None,
                                   strict: bool = False) -> SpikeSimEnergyReport:
    """One forward pass of ``model`` (which should be in eval mode) under the profiler."""
    profiler = SpikeSimEnergyProfiler(config=config, strict=strict)
    training_message = "SpikeSim energy only covers forward inference; call model.eval() before profiling."
    if model.training and strict:
        raise ValueError(training_message)
    notes: List[str] = []
    if profiler.config.require_if_lif_neurons:
        odd = [(n or type(m).__name__, type(m).__name__) for n, m in model.named_modules()
               if isinstance(m, (BaseNode, SimpleBaseNode)) and not isinstance(m, _SUPPORTED_NEURONS)]
        if odd:
            message = ("SpikeSim assumes IF/LIF neuronal modules. Unsupported neuron modules found: "
                       + ", ".join(f"{n} ({c})" for n, c in odd) + ".")
            if strict:
                raise ValueError(message)
            notes.append(message)
    with profiler:
        profiler.add_warnings(notes)
        with torch.no_grad():
            call_model(model, inputs)
    report = profiler.get_report()
    if model.training:
        report.warnings.insert(0, training_message)
    return report
