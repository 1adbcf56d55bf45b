"""Dispatch-mode counter that records, per convolution stage, the activity the SpikeSim formulas need
(``op_counter/spikesim/counter.py`` of the reference)."""
from __future__ import annotations

import math
from collections import defaultdict
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..base import BaseCounter, is_binary_tensor
from .config import ROW_DIVISOR, SpikeSimEnergyConfig

__all__ = ["SpikeSimCounter"]

aten = torch.ops.aten


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
