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
import torch.nn.functional as F

from ...neuron.base_node import BaseNode, SimpleBaseNode
from ...neuron import IFNode, LIFNode
from ..base import BaseCounter, DispatchCounterMode, call_model, is_binary_tensor

try:                                                    # the lightweight neuron variants, when this build has them
    from ...neuron import SimpleIFNode, SimpleLIFNode
    _SUPPORTED_NEURONS: tuple = (IFNode, LIFNode, SimpleIFNode, SimpleLIFNode)
except ImportError:                                     # pragma: no cover
    _SUPPORTED_NEURONS = (IFNode, LIFNode)

aten = torch.ops.aten
_ROW_DIVISOR = 8.0          # SpikeSim's crossbar term scales as (B / 8) * kh * kw


@dataclass
class SpikeSimEnergyConfig:
    """Energies in pJ (SpikeSim's 65 nm figures).  ``device``: ``"rram"`` or ``"sram"`` crossbars."""
    xbar_size: int = 64
    device: str = "rram"
    activity_mode: str = "dense"
    require_if_lif_neurons: bool = True
    tile_buffer_pj: float = 397.0
    temp_buffer_pj: float = 0.2
    sub_pj: float = 1.15e-6
    adc_pj: float = 2.03084
    htree_pj: float = 19.64 * 8.0
    mux_pj: float = 0.094245
    mem_fetch_pj: float = 4.64
    neuron_pj: float = 1.274 * 4.0
    rram_xbar_pj: float = 1.76423
    sram_xbar_pj: float = 671.089

    def copy(self) -> "SpikeSimEnergyConfig":
        return replace(self)

    def validate(self) -> None:
        if self.xbar_size <= 0:
            raise ValueError(f"xbar_size must be positive, got {self.xbar_size}.")
        if self.device not in ("rram", "sram"):
            raise ValueError(f"device must be 'rram' or 'sram', got {self.device}.")
        if self.activity_mode not in ("dense", "event"):
            raise ValueError(f"activity_mode must be 'dense' or 'event', got {self.activity_mode}.")

    @property
    def xbar_array_energy_pj(self) -> float:
        if self.device not in ("rram", "sram"):
            raise ValueError(f"device must be 'rram' or 'sram', got {self.device}.")
        return self.rram_xbar_pj if self.device == "rram" else self.sram_xbar_pj

    @property
    def patch_control_energy_pj(self) -> float:
        g = float(self.xbar_size) / _ROW_DIVISOR
        return (self.htree_pj + self.mem_fetch_pj + self.tile_buffer_pj + g * 16.0 * self.sub_pj + g * self.temp_buffer_pj
                + g * g * (self.adc_pj + self.mux_pj))

    def pe_cycle_energy_for_kernel_pj(self, kernel_size: Tuple[int, int]) -> float:
        if len(kernel_size) != 2:
            raise ValueError(f"kernel_size must be a tuple of length 2, got {kernel_size}.")
        kh, kw = kernel_size
        if kh <= 0 or kw <= 0:
            raise ValueError(f"kernel_size dimensions must be positive, got ({kh}, {kw}).")
        return (self.patch_control_energy_pj + self.neuron_pj
                + (self.xbar_size / _ROW_DIVISOR) * float(kh) * float(kw) * self.xbar_array_energy_pj)

    def xbar_row_energy_pj(self, tile_channels: int) -> float:
        if tile_channels <= 0:
            raise ValueError(f"tile_channels must be positive, got {tile_channels}.")
        if self.xbar_size <= 0:
            raise ValueError(f"xbar_size must be positive, got {self.xbar_size}.")
        padded = math.ceil(tile_channels / self.xbar_size) * self.xbar_size / float(tile_channels)
        return (self.xbar_array_energy_pj / _ROW_DIVISOR) * padded


# ------------------------------------------------------------------------------------------------------------ formulas
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
@dataclass
class _StageStats:
    dense_pe_cycle_count: int = 0
    active_patch_tile_count: int = 0
    active_row_count: int = 0
    active_row_count_by_tile: Optional[List[int]] = None
    active_output_tile_site_count: int = 0
    dense_patch_tile_count: int = 0
    dense_row_count: int = 0
    dense_row_count_by_tile: Optional[List[int]] = None
    dense_output_tile_site_count: int = 0


@dataclass
class _StageMetadata:
    scope: str
    in_channels: int
    out_channels: int
    kernel_size: Tuple[int, int]
    stride: Tuple[int, int]
    padding: Tuple[int, int]
    dilation: Tuple[int, int]
    input_shape: Tuple[int, ...]
    output_shape: Tuple[int, ...]
    out_channel_tiles: int
    input_tile_channels: List[int] = field(default_factory=list)
    total_calls: int = 0
    event_driven_calls: int = 0
    dense_fallback_calls: int = 0
    shape_mismatch_detected: bool = False


def _pair(v) -> Tuple[int, int]:
    if isinstance(v, int):
        return (int(v), int(v))
    if len(v) != 2:
        raise ValueError(f"expected a pair, but got {v}.")
    return (int(v[0]), int(v[1]))


def _accumulate_list(into: Optional[List[int]], first: bool, values: List[int]) -> Optional[List[int]]:
    """Element-wise running sum; a change of length (a stage called with another channel count) drops the list."""
    if first:
        return list(values)
    if into is None or len(into) != len(values):
        return None
    return [a + b for a, b in zip(into, values)]


class SpikeSimCounter(BaseCounter):
    """Dispatch-level counter of ``aten.convolution``: its count is the dense PE-cycle number; the per-stage event
    statistics are kept beside it (``get_stage_stats`` / ``get_stage_metadata``)."""

    def __init__(self, *, config: SpikeSimEnergyConfig, strict: bool):
        super().__init__()
        self.config, self.strict = config, strict
        self.stage_stats: Dict[str, _StageStats] = defaultdict(_StageStats)
        self.stage_metadata: Dict[str, _StageMetadata] = {}
        self.warnings: List[str] = []
        self._warned: set = set()
        self.rules = {aten.convolution.default: self._rule}

    def count(self, func, args, kwargs, out, active_modules=None, parent_names=None) -> int:
        return int(self.rules[func](args, kwargs, out, active_modules=active_modules, parent_names=parent_names))

    # ---- helpers
    def _warn_or_raise(self, key: str, message: str) -> None:
        if key in self._warned:
            return
        self._warned.add(key)
        if self.strict:
            raise NotImplementedError(message)
        self.warnings.append(message)

    @staticmethod
    def _leaf_scope(parent_names) -> str:
        names = [n for n in (parent_names or ()) if n != "Global"]
        return max(names, key=lambda n: (n.count("."), len(n))) if names else "Global"

    def _tiles(self, channels: int) -> List[int]:
        b = self.config.xbar_size
        return [min(b, channels - s) for s in range(0, channels, b)]

    @staticmethod
    def _forward_inference_conv(active_modules) -> bool:
        convs = [m for m in (active_modules or ()) if isinstance(m, nn.Conv2d)]
        return len(convs) == 1 and not convs[0].training and not torch.is_grad_enabled()

    def _event_counts(self, x, w, stride, padding, dilation, q_tiles):
        """(A, R, R per input tile, Z) from the spikes: spikes per (tile, pixel) summed over receptive fields by a grouped
        convolution with a kernel of ones."""
        b = self.config.xbar_size
        n, c, h, wd = x.shape
        tiles = math.ceil(c / b)
        if tiles * b != c:
            x = F.pad(x, (0, 0, 0, 0, 0, tiles * b - c))
        per_tile = x.reshape(n, tiles, b, h, wd).sum(dim=2).to(torch.float32)
        ones = per_tile.new_ones((tiles, 1, w.shape[2], w.shape[3]))
        with torch.no_grad(), torch._C._ExcludeDispatchKeyGuard(torch._C.DispatchKeySet(torch._C.DispatchKey.Python)):
            rows = F.conv2d(per_tile, ones, None, stride, padding, dilation, tiles)
        active = rows.gt(0)
        r_tile = [int(v) for v in rows.sum(dim=(0, 2, 3), dtype=torch.float64).tolist()]
        return int(active.sum().item()), int(sum(r_tile)), r_tile, q_tiles * int(active.any(dim=1).sum().item())

    def _rule(self, args, kwargs, out, *, active_modules=None, parent_names=None) -> int:
        scope = self._leaf_scope(parent_names)
        x, w = args[0], args[1]
        stride, padding, dilation, transposed, groups = args[3], args[4], args[5], bool(args[6]), int(args[8])
        if transposed:
            self._warn_or_raise(f"transposed-conv:{scope}", "SpikeSim energy only covers original SpikeSim Conv2d inference "
                                f"stages; transposed convolutions are outside scope: {scope}.")
            return 0
        if not self._forward_inference_conv(active_modules):
            self._warn_or_raise(f"outside-scope:{scope}", "SpikeSim energy only covers Conv2d forward inference stages from "
                                f"nn.Conv2d modules: {scope}.")
            return 0
        if groups != 1:
            self._warn_or_raise(f"grouped-conv:{scope}", f"SpikeSim event energy does not support grouped/depthwise convolutions: {scope}.")
            return 0
        if x.dim() != 4 or w.dim() != 4 or out.dim() != 4:
            self._warn_or_raise(f"conv-rank:{scope}", "SpikeSim event energy only supports Conv2d-like calls, but got "
                                f"x.shape={tuple(x.shape)}, w.shape={tuple(w.shape)}, out.shape={tuple(out.shape)}.")
            return 0
        stride, padding, dilation = _pair(stride), _pair(padding), _pair(dilation)
        b = self.config.xbar_size
        c_out, c_in, kh, kw = (int(v) for v in w.shape)
        q_tiles, p_tiles = math.ceil(c_out / b), math.ceil(c_in / b)
        in_shape, out_shape = tuple(int(v) for v in x.shape), tuple(int(v) for v in out.shape)
        meta = self.stage_metadata.get(scope)
        if meta is None:
            meta = self.stage_metadata[scope] = _StageMetadata(scope, c_in, c_out, (kh, kw), stride, padding, dilation, in_shape,
                                                               out_shape, q_tiles, self._tiles(c_in))
        elif (meta.input_shape, meta.output_shape, meta.kernel_size, meta.stride, meta.padding, meta.dilation) != \
                (in_shape, out_shape, (kh, kw), stride, padding, dilation):
            meta.shape_mismatch_detected = True
            self._warn_or_raise(f"shape-mismatch:{scope}", f"SpikeSim stage '{scope}' was invoked with inconsistent shapes; "
                                "runtime energy is accumulated across calls anyway.")
        first = meta.total_calls == 0
        meta.total_calls += 1
        sites = out_shape[0] * out_shape[2] * out_shape[3]
        tiles = self._tiles(c_in)
        dense_a, dense_r_tile, dense_z = sites * len(tiles), [sites * t * kh * kw for t in tiles], q_tiles * sites
        dense_r = sum(dense_r_tile)
        if self.config.activity_mode == "event" and is_binary_tensor(x):
            meta.event_driven_calls += 1
            act_a, act_r, act_r_tile, act_z = self._event_counts(x, w, stride, padding, dilation, q_tiles)
        else:
            meta.dense_fallback_calls += 1
            act_a, act_r, act_r_tile, act_z = dense_a, dense_r, dense_r_tile, dense_z
        cycles = p_tiles * q_tiles * sites
        st = self.stage_stats[scope]
        st.dense_pe_cycle_count += cycles
        st.active_patch_tile_count += act_a
        st.active_row_count += act_r
        st.active_row_count_by_tile = _accumulate_list(st.active_row_count_by_tile, first, act_r_tile)
        st.active_output_tile_site_count += act_z
        st.dense_patch_tile_count += dense_a
        st.dense_row_count += dense_r
        st.dense_row_count_by_tile = _accumulate_list(st.dense_row_count_by_tile, first, dense_r_tile)
        st.dense_output_tile_site_count += dense_z
        return cycles

    def get_stage_stats(self) -> Dict[str, Dict[str, Any]]:
        return {k: asdict(v) for k, v in self.stage_stats.items()}

    def get_stage_metadata(self) -> Dict[str, Dict[str, Any]]:
        return {k: asdict(v) for k, v in self.stage_metadata.items()}


# ------------------------------------------------------------------------------------------------------------ profiler
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
