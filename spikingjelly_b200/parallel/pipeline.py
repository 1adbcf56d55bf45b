"""Pipeline parallelism for SNNs on ``torch.distributed.pipelining`` (NCCL / gloo point-to-point).

A model is cut into *units* (Spikformer: patch stem, every block, head; VGG-like nets: every child of
``features`` and ``classifier``); units are costed by one timed forward + backward on a micro-batch
and grouped into ``world_size * virtual_stages`` contiguous logical stages of balanced cost (binary
search on the bottleneck) or by an explicit layout.  Every stage resets its neurons at the start of
each micro-batch: the membrane state of one micro-batch must not leak into the next.

Parity: ``spikingjelly/activation_based/distributed/pipeline/{partition,runtime,memopt,spikformer,
cifar10dvs_vgg}.py``.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass
from typing import Any, List, Mapping, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..activation_based.functional.net_config import collect_reset_modules, reset_collected_modules
from ..logger import logger

try:
    from torch.distributed.pipelining import (PipelineStage, Schedule1F1B, ScheduleGPipe, ScheduleInterleaved1F1B,
                                              ScheduleInterleavedZeroBubble)
    PIPELINING_AVAILABLE = True
except ImportError:                                       # pragma: no cover
    PipelineStage = Schedule1F1B = ScheduleGPipe = ScheduleInterleaved1F1B = ScheduleInterleavedZeroBubble = None
    PIPELINING_AVAILABLE = False

__all__ = ["PIPELINING_AVAILABLE", "SNNPipelineRuntime", "parse_pipeline_layout", "resolve_pipeline_schedule_kind",
           "recommend_pipeline_memopt_stages", "apply_pipeline_stage_memopt", "configure_snn_pipeline",
           "configure_spikformer_pipeline", "configure_cifar10dvs_vgg_pipeline", "snn_sequence_cross_entropy"]


# --------------------------------------------------------------------------------- partitioning
def _even_partition_sizes(num_items: int, num_parts: int) -> List[int]:
    if num_parts <= 0:
        raise ValueError(f"num_parts must be positive, but got {num_parts}.")
    q, r = divmod(num_items, num_parts)
    return [q + (1 if i < r else 0) for i in range(num_parts)]


def _partition_costs_contiguously(costs: Sequence[float], num_parts: int) -> List[int]:
    """Sizes of ``num_parts`` contiguous groups minimising the largest group cost."""
    if num_parts <= 0:
        raise ValueError(f"num_parts must be positive, but got {num_parts}.")
    n = len(costs)
    if n == 0:
        return [0] * num_parts
    if n < num_parts:
        return _even_partition_sizes(n, num_parts)
    costs = [float(c) for c in costs]

    def parts_needed(limit: float) -> int:
        parts, acc = 1, 0.0
        for c in costs:
            if acc == 0.0 or acc + c <= limit:
                acc += c
            else:
                parts, acc = parts + 1, c
        return parts

    lo, hi = max(costs), sum(costs)
    for _ in range(48):
        mid = 0.5 * (lo + hi)
        lo, hi = (lo, mid) if parts_needed(mid) <= num_parts else (mid, hi)
    sizes, acc, count, left = [], 0.0, 0, num_parts
    for idx in range(n - 1, -1, -1):                       # fill from the back so that early stages are never empty
        if count > 0 and left > 1 and (acc + costs[idx] > hi or idx + 1 < left):
            sizes.append(count)
            left, acc, count = left - 1, 0.0, 0
        acc += costs[idx]
        count += 1
    sizes.append(count)
    sizes.reverse()
    return [0] * (num_parts - len(sizes)) + sizes


def parse_pipeline_layout(layout: Optional[Union[str, Sequence[int]]], num_logical_stages: int, total_units: int) -> Optional[Tuple[int, ...]]:
    """``"3|4|4|2"`` / ``"3,4,4,2"`` / a sequence -> units per logical stage (validated)."""
    if layout is None:
        return None
    counts = tuple(int(t.strip()) for t in layout.replace(",", "|").split("|") if t.strip()) if isinstance(layout, str) \
        else tuple(int(v) for v in layout)
    if len(counts) != num_logical_stages:
        raise ValueError(f"Pipeline layout must provide {num_logical_stages} stage counts, but got {len(counts)} from {layout!r}.")
    if any(c < 0 for c in counts):
        raise ValueError(f"Pipeline layout counts must be non-negative, but got {counts}.")
    if sum(counts) != total_units:
        raise ValueError(f"Pipeline layout {counts} covers {sum(counts)} units, but the model requires {total_units} units.")
    return counts


def resolve_pipeline_schedule_kind(schedule_kind: str, virtual_pipeline_size: int, delayed_wgrad: bool) -> str:
    kind = schedule_kind.lower()
    if kind not in ("auto", "gpipe", "1f1b", "interleaved", "zero_bubble"):
        raise ValueError(f"Unsupported pp schedule '{schedule_kind}'. Expected one of: auto, gpipe, 1f1b, interleaved, zero_bubble.")
    if kind == "auto":
        kind = "zero_bubble" if delayed_wgrad else ("interleaved" if virtual_pipeline_size > 1 else "1f1b")
    if kind == "gpipe" and delayed_wgrad:
        raise ValueError("pp_delay_wgrad is incompatible with pp_schedule='gpipe'.")
    if kind in ("gpipe", "1f1b") and virtual_pipeline_size != 1:
        raise ValueError(f"pp_schedule='{kind}' does not support pp_virtual_stages={virtual_pipeline_size}. "
                         "Use pp_schedule='interleaved' or 'zero_bubble' when pp_virtual_stages > 1.")
    if kind in ("interleaved", "zero_bubble") and virtual_pipeline_size < 2:
        raise ValueError(f"pp_schedule='{kind}' requires pp_virtual_stages >= 2, but got {virtual_pipeline_size}.")
    return kind


# -------------------------------------------------------------------------------------- runtime
@dataclass
class SNNPipelineRuntime:
    """What one rank holds of a pipeline: its schedule, local stage modules and bookkeeping."""
    schedule: Any
    stage_module: nn.Module
    stage_modules: Tuple[nn.Module, ...]
    local_stage_indices: Tuple[int, ...]
    stage_index: int
    num_stages: int
    device: torch.device
    n_microbatches: int
    model_family: str
    split_points: Tuple[str, ...]
    group: Optional[Any] = None
    stage_costs: Tuple[float, ...] = ()
    stage_input_examples: Tuple[Any, ...] = ()
    memopt_selected_stage_indices: Tuple[int, ...] = ()
    schedule_kind: str = "gpipe"
    virtual_pipeline_size: int = 1
    pp_layout: Optional[Tuple[int, ...]] = None
    delayed_wgrad: bool = False

    @property
    def is_first(self) -> bool:
        return bool(self.local_stage_indices) and self.local_stage_indices[0] == 0

    @property
    def is_last(self) -> bool:
        return bool(self.local_stage_indices) and self.local_stage_indices[-1] == self.num_stages - 1

    @property
    def stage_input_example(self) -> Optional[Any]:
        return self.stage_input_examples[0] if self.stage_input_examples else None

    def step(self, inputs: Optional[torch.Tensor] = None, target: Optional[torch.Tensor] = None):
        """One pipelined forward + backward over ``n_microbatches``: the first stage feeds
        ``inputs``, the last stage ``target``; returns the per-micro-batch losses on the last stage."""
        losses: list = []
        kwargs = {}
        if self.is_last and target is not None:
            kwargs = {"target": target, "losses": losses}
        if self.is_first and inputs is not None:
            self.schedule.step(inputs, **kwargs)
        else:
            self.schedule.step(**kwargs)
        return losses


def _tree(fn, value):
    if isinstance(value, torch.Tensor):
        return fn(value)
    if isinstance(value, tuple):
        return tuple(_tree(fn, v) for v in value)
    if isinstance(value, list):
        return [_tree(fn, v) for v in value]
    if isinstance(value, Mapping):
        return type(value)((k, _tree(fn, v)) for k, v in value.items())
    return value


def _leaves(value):
    if isinstance(value, torch.Tensor):
        yield value
    elif isinstance(value, (tuple, list)):
        for v in value:
            yield from _leaves(v)
    elif isinstance(value, Mapping):
        for v in value.values():
            yield from _leaves(v)


def _standalone(t: torch.Tensor) -> torch.Tensor:
    # stage outputs are detached in place by some schedules: they must own contiguous storage
    if t._is_view():
        return t.clone(memory_format=torch.contiguous_format)
    return t if t.is_contiguous() else t.contiguous()


def _measure_module_cost(module: nn.Module, input_value: Any) -> Tuple[Any, float]:
    """(output, cost): forward ms + backward ms + small terms for activation and parameter volume."""
    resets = collect_reset_modules(module)
    first = next(_leaves(input_value), None)
    cuda = first is not None and first.is_cuda

    def timed(fn):
        if cuda:
            torch.cuda.synchronize(first.device)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn()
            e1.record()
            torch.cuda.synchronize(first.device)
            return out, float(e0.elapsed_time(e1))
        t0 = time.perf_counter()
        out = fn()
        return out, (time.perf_counter() - t0) * 1e3

    with torch.no_grad():
        reset_collected_modules(resets)
        output, fwd_ms = timed(lambda: module(input_value))
        reset_collected_modules(resets)
    bwd_ms = 0.0
    module.zero_grad(set_to_none=True)
    try:
        with torch.enable_grad():
            x = _tree(lambda t: t.detach().clone().requires_grad_(t.is_floating_point()), input_value)
            total = None
            for leaf in _leaves(module(x)):
                if leaf.is_floating_point():
                    total = leaf.sum() if total is None else total + leaf.sum()
            if total is not None and total.requires_grad:
                _, bwd_ms = timed(total.backward)
    finally:
        module.zero_grad(set_to_none=True)
        reset_collected_modules(resets)
    signal = sum(t.numel() for t in _leaves(output))
    params = sum(p.numel() for p in module.parameters())
    return output, max(fwd_ms, 1e-6) + bwd_ms + signal / 1e6 + params / 1e7


def snn_sequence_cross_entropy(outputs: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    """Cross entropy of the firing rate (mean over the leading time axis of a 3-D output)."""
    full = getattr(outputs, "full_tensor", None)
    if callable(full):
        outputs = full()
    if outputs.ndim >= 3:
        outputs = outputs.mean(dim=0)
    if target.ndim > 1:
        target = target.argmax(dim=-1) if target.shape[-1] > 1 else target.squeeze(-1)
    return F.cross_entropy(outputs, target)


class _PipelineSequentialModule(nn.Module):
    def __init__(self, stages: Sequence[nn.Module], stage_costs: Sequence[float] = ()):
        super().__init__()
        self.stages = nn.ModuleList(list(stages))
        self.stage_costs = tuple(float(c) for c in stage_costs)

    def forward(self, x):
        for s in self.stages:
            x = s(x)
        return x


class _MicrobatchResetStage(nn.Module):
    """Resets the neurons of ``inner`` before every call (= every micro-batch)."""

    def __init__(self, inner: nn.Module):
        super().__init__()
        self.inner = inner
        self._resets = collect_reset_modules(inner)

    def refresh_reset_modules(self):
        self._resets = collect_reset_modules(self.inner)

    def forward(self, *args, **kwargs):
        reset_collected_modules(self._resets)
        return _tree(_standalone, self.inner(*args, **kwargs))


def _example_microbatch(example_input: torch.Tensor, n_microbatches: int, batch_dim: int = 0) -> torch.Tensor:
    if n_microbatches <= 0:
        raise ValueError(f"n_microbatches must be positive, but got {n_microbatches}.")
    b = example_input.shape[batch_dim]
    if b <= 0:
        raise ValueError("example_input must contain at least one sample on the batch dimension.")
    if b < n_microbatches:
        raise ValueError(f"example_input batch size ({b}) must be >= n_microbatches ({n_microbatches}).")
    return example_input.narrow(batch_dim, 0, max(1, b // n_microbatches)).contiguous()


def _build_snn_pipeline_runtime(pipeline_module: nn.Module, example_input: torch.Tensor, device: torch.device, n_microbatches: int,
                                stage_index: Optional[int], model_family: str, schedule_kind: str = "auto",
                                virtual_pipeline_size: int = 1, delayed_wgrad: bool = False,
                                pp_layout: Optional[Tuple[int, ...]] = None, group=None, loss_fn=snn_sequence_cross_entropy) -> SNNPipelineRuntime:
    if not PIPELINING_AVAILABLE:
        raise RuntimeError("torch.distributed.pipelining is unavailable in this PyTorch build.")
    if not dist.is_initialized():
        raise RuntimeError("Pipeline parallel requires torch.distributed to be initialized.")
    physical = dist.get_world_size(group)
    if virtual_pipeline_size <= 0:
        raise ValueError(f"virtual_pipeline_size must be positive, but got {virtual_pipeline_size}.")
    kind = resolve_pipeline_schedule_kind(schedule_kind, virtual_pipeline_size, delayed_wgrad)
    num_stages = physical * virtual_pipeline_size
    if n_microbatches < num_stages:
        raise ValueError(f"n_microbatches ({n_microbatches}) must be >= number of stages ({num_stages}).")
    stage_index = dist.get_rank(group) if stage_index is None else stage_index
    if not hasattr(pipeline_module, "stages"):
        raise TypeError("pipeline_module must expose a 'stages' attribute.")
    if not 0 <= stage_index < physical:
        raise ValueError(f"stage_index={stage_index} is out of range for num_stages={physical}.")
    if len(pipeline_module.stages) != num_stages:
        raise ValueError(f"pipeline_module exposes {len(pipeline_module.stages)} logical stages, but {num_stages} are required for "
                         f"physical_num_stages={physical} and virtual_pipeline_size={virtual_pipeline_size}.")
    local = tuple(stage_index + physical * k for k in range(virtual_pipeline_size))
    wrapped = tuple(_MicrobatchResetStage(pipeline_module.stages[i]) for i in local)
    pipeline_module = pipeline_module.to(device)
    micro = _example_microbatch(example_input, n_microbatches).to(device)
    ins, outs = [], []
    resets = collect_reset_modules(pipeline_module)
    with torch.no_grad():
        cur = micro
        reset_collected_modules(resets)
        for s in pipeline_module.stages:
            ins.append(cur)
            cur = s(cur)
            outs.append(cur)
        reset_collected_modules(resets)
    stages = [PipelineStage(wrapped[k], stage_index=i, num_stages=num_stages, device=device, input_args=ins[i], output_args=outs[i],
                            group=group) for k, i in enumerate(local)]
    schedule = {"gpipe": lambda: ScheduleGPipe(stages[0], n_microbatches=n_microbatches, loss_fn=loss_fn),
                "1f1b": lambda: Schedule1F1B(stages[0], n_microbatches=n_microbatches, loss_fn=loss_fn),
                "interleaved": lambda: ScheduleInterleaved1F1B(stages, n_microbatches=n_microbatches, loss_fn=loss_fn),
                "zero_bubble": lambda: ScheduleInterleavedZeroBubble(stages, n_microbatches=n_microbatches, loss_fn=loss_fn)}[kind]()
    rt = SNNPipelineRuntime(schedule=schedule, stage_module=wrapped[0] if len(wrapped) == 1 else _PipelineSequentialModule(wrapped),
                            stage_modules=wrapped, local_stage_indices=local, stage_index=stage_index, num_stages=num_stages,
                            device=device, n_microbatches=n_microbatches, model_family=model_family,
                            split_points=tuple(f"stages.{i}" for i in range(1, num_stages)), group=group,
                            stage_costs=tuple(getattr(pipeline_module, "stage_costs", ())),
                            stage_input_examples=tuple(ins[i] for i in local), schedule_kind=kind,
                            virtual_pipeline_size=virtual_pipeline_size, pp_layout=pp_layout, delayed_wgrad=delayed_wgrad)
    logger.info("distributed_pipeline_runtime_summary model_family=%s stage_index=%s local_stage_indices=%s num_stages=%s "
                "n_microbatches=%s schedule=%s device=%s", model_family, stage_index, local, num_stages, n_microbatches, kind, device)
    return rt


# ------------------------------------------------------------------------------- model front ends
class _UnitStage(nn.Module):
    """A run of units; ``pre`` / ``post`` are applied around them on the first / last stage."""

    def __init__(self, units: Sequence[nn.Module], pre=None, post_before_last=None):
        super().__init__()
        self.units = nn.ModuleList(list(units))
        self._pre, self._glue = pre, post_before_last or {}

    def forward(self, x):
        if self._pre is not None:
            x = self._pre(x)
        for i, u in enumerate(self.units):
            if i in self._glue:
                x = self._glue[i](x)
            x = u(x)
        return x


def configure_snn_pipeline(units: Sequence[nn.Module], example_input: torch.Tensor, n_microbatches: int, *, device=None,
                           model_family: str = "generic", schedule_kind: str = "auto", virtual_pipeline_size: int = 1,
                           delayed_wgrad: bool = False, layout: Optional[Union[str, Sequence[int]]] = None, group=None,
                           stage_index: Optional[int] = None, pre=None, glue: Optional[Mapping[int, Any]] = None,
                           loss_fn=snn_sequence_cross_entropy) -> SNNPipelineRuntime:
    """Cut ``units`` (applied in order; ``glue[i]`` is a stateless function applied before unit ``i``,
    ``pre`` before the first) into pipeline stages and build this rank's runtime."""
    if not dist.is_initialized():
        raise RuntimeError("Pipeline parallel requires torch.distributed to be initialized.")
    device = torch.device(device) if device is not None else example_input.device
    num_logical = dist.get_world_size(group) * virtual_pipeline_size
    if num_logical < 2:
        raise ValueError("pipeline parallel requires at least 2 stages.")
    glue = dict(glue or {})
    units = [u.to(device) for u in units]
    micro = _example_microbatch(example_input, n_microbatches).to(device)
    cur = pre(micro) if pre is not None else micro
    costs = []
    for i, u in enumerate(units):
        if i in glue:
            cur = glue[i](cur)
        cur, c = _measure_module_cost(u, cur)
        costs.append(c)
    counts = parse_pipeline_layout(layout, num_logical, len(units))
    if counts is None:
        if dist.get_world_size(group) > 1:                 # every rank must cut at the same places
            t = torch.tensor(costs, dtype=torch.float64, device=device if device.type == "cuda" else "cpu")
            dist.broadcast(t, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
            costs = t.tolist()
        counts = tuple(_partition_costs_contiguously(costs, num_logical))
    stages, stage_costs, at = [], [], 0
    for s, n in enumerate(counts):
        idx = range(at, at + n)
        stages.append(_UnitStage([units[i] for i in idx], pre if s == 0 else None, {i - at: glue[i] for i in idx if i in glue}))
        stage_costs.append(sum(costs[i] for i in idx))
        at += n
    module = _PipelineSequentialModule(stages, stage_costs)
    return _build_snn_pipeline_runtime(module, example_input, device, n_microbatches, stage_index, model_family, schedule_kind,
                                       virtual_pipeline_size, delayed_wgrad, counts, group, loss_fn)


def _pipeline_arguments(device, n_microbatches, pp_schedule, pp_virtual_stages, pp_layout, pp_delay_wgrad, stage_index, group, kwargs) -> dict:
    """The reference's argument names (``device, n_microbatches, pp_schedule, pp_virtual_stages, pp_layout, pp_delay_wgrad``) mapped
    onto :func:`configure_snn_pipeline`'s.  ``(module, example_input, n_microbatches)``, the older positional form, is still read."""
    if n_microbatches is None and isinstance(device, int) and not isinstance(device, bool):
        device, n_microbatches = None, device
    if n_microbatches is None:
        raise TypeError("n_microbatches is required")
    out = dict(kwargs)
    out.setdefault("device", device)
    out.setdefault("schedule_kind", pp_schedule)
    out.setdefault("virtual_pipeline_size", pp_virtual_stages)
    out.setdefault("layout", pp_layout)
    out.setdefault("delayed_wgrad", pp_delay_wgrad)
    out.setdefault("stage_index", stage_index)
    out.setdefault("group", group)
    return {"n_microbatches": int(n_microbatches), **out}


def configure_spikformer_pipeline(module: nn.Module, example_input: torch.Tensor, device=None, n_microbatches: Optional[int] = None,
                                  pp_schedule: str = "auto", pp_virtual_stages: int = 1, pp_layout=None, pp_delay_wgrad: bool = False,
                                  stage_index: Optional[int] = None, group=None, **kwargs) -> SNNPipelineRuntime:
    """Units: patch stem, every block, head (features are averaged over the spatial axes before the
    head).  A 4-D ``[N, C, H, W]`` input is repeated over ``module.T`` time-steps by the first stage.
    Micro-batches are cut along the batch axis, so inputs are ``[N, ...]`` (time is added inside)."""
    if not (hasattr(module, "patch_embed") and hasattr(module, "blocks") and hasattr(module, "head")):
        raise TypeError("Expected a Spikformer-like module with patch_embed, blocks, and head.")
    if example_input.ndim != 4:
        raise ValueError(f"expected a 4D [N, C, H, W] example input (time is added by the first stage), but got {tuple(example_input.shape)}")
    T = getattr(module, "T", None)
    if T is None:
        raise RuntimeError("Spikformer pipeline stage requires module.T to be set.")
    if hasattr(module, "fused"):
        module.fused = False
    units = [module.patch_embed, *module.blocks, module.head]

    def add_time(x):
        return x.unsqueeze(0).expand(int(T), *x.shape) if x.ndim == 4 else x

    def pool(x):
        return x.flatten(3).mean(dim=-1)

    class _ToBatchFirst(nn.Module):                       # schedules merge micro-batches on dim 0
        def __init__(self, inner):
            super().__init__()
            self.inner = inner

        def forward(self, x):
            return self.inner(x).transpose(0, 1)

    units[-1] = _ToBatchFirst(units[-1])
    kwargs.setdefault("model_family", "spikformer")
    kwargs.setdefault("loss_fn", lambda out, tgt: snn_sequence_cross_entropy(out.transpose(0, 1), tgt))
    a = _pipeline_arguments(device, n_microbatches, pp_schedule, pp_virtual_stages, pp_layout, pp_delay_wgrad, stage_index, group, kwargs)
    return configure_snn_pipeline(units, example_input, a.pop("n_microbatches"), pre=add_time, glue={len(units) - 1: pool}, **a)


def configure_cifar10dvs_vgg_pipeline(module: nn.Module, example_input: torch.Tensor, device=None, n_microbatches: Optional[int] = None,
                                      pp_schedule: str = "auto", pp_virtual_stages: int = 1, pp_layout=None, pp_delay_wgrad: bool = False,
                                      stage_index: Optional[int] = None, group=None, **kwargs) -> SNNPipelineRuntime:
    """Units: the children of ``module.features`` and of ``module.classifier`` (flatten in between)."""
    if not (hasattr(module, "features") and hasattr(module, "classifier")):
        raise TypeError("Expected a VGG-like module with features and classifier.")
    feats, cls = list(module.features.children()), list(module.classifier.children())
    kwargs.setdefault("model_family", "cifar10dvs_vgg")
    a = _pipeline_arguments(device, n_microbatches, pp_schedule, pp_virtual_stages, pp_layout, pp_delay_wgrad, stage_index, group, kwargs)
    return configure_snn_pipeline(feats + cls, example_input, a.pop("n_microbatches"), glue={len(feats): lambda x: torch.flatten(x, 1)}, **a)


# ----------------------------------------------------------------------------- memopt per stage
def recommend_pipeline_memopt_stages(stage_costs: Sequence[float], stage_budget_ratio: float = 0.5) -> Tuple[int, ...]:
    """Indices of the most expensive ``round(ratio * n)`` (at least one) stages, ascending."""
    if not stage_costs:
        return ()
    if not math.isfinite(stage_budget_ratio) or stage_budget_ratio <= 0.0 or stage_budget_ratio > 1.0:
        raise ValueError(f"stage_budget_ratio must be a finite number in (0, 1], but got {stage_budget_ratio}.")
    n = len(stage_costs)
    k = max(1, min(n, int(round(n * stage_budget_ratio))))
    ranked = sorted(range(n), key=lambda i: (float(stage_costs[i]), -i), reverse=True)
    return tuple(sorted(ranked[:k]))


def apply_pipeline_stage_memopt(runtime: SNNPipelineRuntime, *, memopt_level: int, compress_x: bool = False,
                                stage_budget_ratio: float = 0.5, use_plan_cache: bool = True, target_types: Optional[tuple] = None):
    """Run ``memory_optimization`` on the local stages that are among the costliest ones.
    Returns ``(runtime, optimisation time in ms, whether anything was applied)``."""
    if memopt_level <= 0:
        runtime.memopt_selected_stage_indices = ()
        return runtime, 0.0, False
    if target_types is None:
        if runtime.model_family == "spikformer":
            from ..activation_based.layer.attention import SpikingSelfAttention
            from ..models.spikformer import SpikformerConv2dBNLIF, SpikformerMLP
            target_types = (SpikformerConv2dBNLIF, SpikingSelfAttention, SpikformerMLP)
        else:
            raise ValueError(f"Unsupported pipeline model_family='{runtime.model_family}' for memopt; pass target_types.")
    selected = recommend_pipeline_memopt_stages(runtime.stage_costs, stage_budget_ratio)
    if dist.is_initialized() and dist.get_world_size(runtime.group) > 1:
        t = torch.tensor(selected, dtype=torch.int64, device=runtime.device if runtime.device.type == "cuda" else "cpu")
        dist.broadcast(t, src=dist.get_global_rank(runtime.group, 0) if runtime.group is not None else 0, group=runtime.group)
        selected = tuple(t.tolist())
    runtime.memopt_selected_stage_indices = selected
    todo = [(wrapper, example) for wrapper, example, idx in zip(runtime.stage_modules, runtime.stage_input_examples,
                                                                runtime.local_stage_indices) if idx in selected]
    if not todo:
        return runtime, 0.0, False
    from ..activation_based.memopt import memory_optimization
    t0 = time.time()
    for wrapper, example in todo:
        if example is None:
            raise RuntimeError("Pipeline memopt requires a stage input example.")
        wrapper.inner = memory_optimization(wrapper.inner.to(runtime.device), target_types, dummy_input=(example.to(runtime.device),),
                                            compress_x=compress_x, level=memopt_level).to(runtime.device)
        wrapper.refresh_reset_modules()
    ms = (time.time() - t0) * 1e3
    logger.info("distributed_pipeline_memopt_summary model_family=%s applied=True memopt_level=%s selected_stage_indices=%s "
                "optimize_ms=%.3f compress_x=%s", runtime.model_family, memopt_level, selected, ms, compress_x)
    return runtime, ms, True
