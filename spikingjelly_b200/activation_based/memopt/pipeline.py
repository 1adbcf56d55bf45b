"""Automatic placement of compressed-input gradient checkpointing.

``memory_optimization(net, instance, dummy_input, level=...)`` rewrites ``net`` in four stages of
increasing cost:

1. wrap every (or the budgeted subset of) ``instance`` module in a ``GCContainer``; inputs that a
   probe finds to be binary are stored bit-packed;
2. split the container with the largest training footprint *spatially* (into its sub-blocks, or
   the blocks its ``__spatial_split__()`` returns) while that lowers the peak;
3. split the heaviest container *temporally* (``TCGCContainer``, chunk count doubled per step)
   while that lowers the peak;
4. remove containers (slowest forward first) whose removal does not raise the peak.

Presets: ``profile`` in ``MEMOPT_PROFILES`` picks a level and search limits, ``checkpoint_budget``
limits how many modules stage 1 wraps, ``prefer`` picks both.  The outcome is described by a
``MemOptSummary``.

Peak memory is measured *in this process* on a deep copy of the network with the profiler's
meter: the CUDA caching allocator on a GPU, the bytes autograd saves for backward elsewhere.
All kernels of this package are compiled ahead of time, so no worker process is needed to keep
just-in-time compilation out of the measurement; ``warmup_in_profile_workers`` only controls an
untimed warm-up step before each measurement.

Parity: ``spikingjelly/activation_based/memopt/pipeline.py:23-1763``.
"""
from __future__ import annotations

import copy
import os
import time
from dataclasses import dataclass, field
from math import ceil
from typing import Callable, Dict, Optional, Tuple, Union

import torch
import torch.distributed as dist
import torch.nn as nn

from ...logger import logger
from .. import functional, neuron
from ..profiler import LayerWiseFPCUDATimeProfiler, LayerWiseMemoryProfiler, make_meter
from . import compress
from .checkpointing import GCContainer, TCGCContainer
from .compress import BitSpikeCompressor, NullSpikeCompressor

__all__ = ["MEMOPT_CHECKPOINT_BUDGETS", "MEMOPT_PREFERENCES", "MEMOPT_PROFILES", "MemOptSummary", "apply_gc",
           "get_module_and_parent", "memory_optimization", "resolve_device"]

TCGC_FORBIDDEN_MODULES = [neuron.PSN, neuron.MaskedPSN, neuron.SlidingPSN]   # need the whole sequence at once
MEMOPT_PROFILES = ("safe", "balanced", "memory", "exhaustive")
MEMOPT_CHECKPOINT_BUDGETS = ("speed", "balanced", "memory")
MEMOPT_PREFERENCES = ("speed", "balanced", "memory")

_PROFILE_PRESETS = {
    #              level compress rounds cands  warm_main warm_workers expensive
    "safe":       (1, True, 0, 0, False, False, False),
    "balanced":   (2, True, 1, 1, False, False, False),
    "memory":     (3, True, 2, 2, False, True, True),
    "exhaustive": (4, True, None, None, True, True, True),
}
_OPTION_NAMES = ("level", "compress_x", "max_split_rounds", "max_candidates_per_round", "warmup_in_main_process",
                 "warmup_in_profile_workers", "allow_expensive_profiling")
_BUDGET_RATIOS = {"speed": 0.5, "balanced": 0.75, "memory": 1.0}
_PREFERENCE_DEFAULTS = {"speed": ("safe", "speed"), "balanced": ("balanced", "balanced"), "memory": ("memory", "memory")}


@dataclass
class MemOptSummary:
    """What ``memory_optimization`` decided and did (counts of wraps, splits, unwraps, the selected
    modules and a human-readable recommendation)."""
    profile: Optional[str]
    checkpoint_budget: Optional[str]
    prefer: Optional[str]
    device: str
    requested_level: int
    applied_level: int
    compress_x: bool
    allow_expensive_profiling: bool
    applied_steps: list = field(default_factory=list)
    skipped_steps: list = field(default_factory=list)
    notes: list = field(default_factory=list)
    gc_wrap_count: int = 0
    manual_compressor_count: int = 0
    bit_compressor_count: int = 0
    null_compressor_count: int = 0
    spatial_split_count: int = 0
    temporal_split_count: int = 0
    unwrap_count: int = 0
    gc_container_count: int = 0
    tcgc_container_count: int = 0
    options: dict = field(default_factory=dict)
    gc_candidate_count: int = 0
    gc_selected_count: int = 0
    gc_selection_policy: str = "all_candidates"
    gc_selected_modules: list = field(default_factory=list)
    gc_selection_explanation: str = ""
    recommendation: str = ""


# ---------------------------------------------------------------------------------------------
# small helpers
# ---------------------------------------------------------------------------------------------
def _compressor_from_spec(spec):
    if isinstance(spec, str):
        if not hasattr(compress, spec):
            known = ", ".join(n for n in dir(compress) if n.endswith("Compressor") and not n.startswith("_"))
            raise ValueError(f"Unknown compressor spec {spec!r}. Available compressor classes: {known}.")
        return getattr(compress, spec)()
    return copy.deepcopy(spec)


def resolve_device() -> str:
    """``"cpu"`` without CUDA; else the device of this process' local rank (``LOCAL_RANK``,
    ``SLURM_LOCALID``, ``OMPI_COMM_WORLD_LOCAL_RANK``, ``MV2_COMM_WORLD_LOCAL_RANK``), else
    ``rank % device_count`` of an initialised process group, else the current device."""
    if not torch.cuda.is_available():
        return "cpu"
    n_gpu = torch.cuda.device_count()
    for key in ("LOCAL_RANK", "SLURM_LOCALID", "OMPI_COMM_WORLD_LOCAL_RANK", "MV2_COMM_WORLD_LOCAL_RANK"):
        value = os.environ.get(key)
        if value is None:
            continue
        try:
            rank = int(value)
        except ValueError as e:
            raise ValueError(f"{key} must be an integer, got {value!r}") from e
        if not 0 <= rank < n_gpu:
            raise ValueError(f"{key} must be in [0, {n_gpu}), got {rank}")
        return f"cuda:{rank}"
    if dist.is_available() and dist.is_initialized() and n_gpu > 0:
        return f"cuda:{dist.get_rank() % n_gpu}"
    return f"cuda:{torch.cuda.current_device()}"


def _tree_map(fn: Callable, obj):
    if isinstance(obj, torch.Tensor):
        return fn(obj)
    if isinstance(obj, (tuple, list)):
        return type(obj)(_tree_map(fn, o) for o in obj)
    if isinstance(obj, dict):
        return {k: _tree_map(fn, v) for k, v in obj.items()}
    return obj


def _to_device(obj, device):
    return _tree_map(lambda t: t.to(device), obj)


def _random_like(obj):
    """A fresh input of the same structure: floats become N(0,1), U(-5,5) or Bernoulli(0.5)."""
    def one(x: torch.Tensor):
        if x.dtype == torch.bool:
            return torch.rand_like(x, dtype=torch.float32) > 0.5
        if x.is_floating_point():
            kind = int(torch.randint(0, 3, ()))
            if kind == 0:
                return torch.randn_like(x)
            if kind == 1:
                return torch.empty_like(x).uniform_(-5, 5)
            return torch.empty_like(x).bernoulli_(0.5)
        if x.dtype in (torch.uint8, torch.int8, torch.int16, torch.int32, torch.int64):
            return torch.randint(0, 3, x.shape, device=x.device, dtype=x.dtype)
        return x.clone()
    return _tree_map(one, obj)


class _eval_no_grad:
    def __init__(self, net):
        self.net = net

    def __enter__(self):
        self.was_training = self.net.training
        self.net.eval()
        self.ng = torch.no_grad()
        self.ng.__enter__()

    def __exit__(self, *exc):
        self.ng.__exit__(*exc)
        self.net.train(self.was_training)
        return False


def _probe_binary_inputs(net, targets, dummy_input, n_trials: int = 5) -> Dict[nn.Module, bool]:
    """For each target: did every first positional input seen over ``n_trials`` forwards (the given
    input, then random ones) consist of zeros and ones only?"""
    verdict = {m: True for m in targets}

    def hook(m, inputs):
        x = inputs[0]
        verdict[m] = verdict[m] and bool(torch.all((x == 0) | (x == 1)))

    handles = [m.register_forward_pre_hook(hook) for m in targets]
    try:
        with _eval_no_grad(net):
            for trial in range(n_trials):
                net(*(dummy_input if trial == 0 else _random_like(dummy_input)))
                functional.reset_net(net)
                if targets and not any(verdict.values()):
                    break
    finally:
        for h in handles:
            h.remove()
    return verdict


def _input_bytes(net, targets, dummy_input) -> Dict[nn.Module, int]:
    sizes = {m: 0 for m in targets}

    def hook(m, inputs):
        if inputs and isinstance(inputs[0], torch.Tensor):
            sizes[m] = max(sizes[m], inputs[0].numel() * inputs[0].element_size())

    handles = [m.register_forward_pre_hook(hook) for m in targets]
    try:
        with _eval_no_grad(net):
            net(*dummy_input)
            functional.reset_net(net)
    finally:
        for h in handles:
            h.remove()
    return sizes


def _select_targets(net, instance, dummy_input, device, max_modules, ratio):
    """-> (selected or None for "all", n_candidates, n_selected, policy)"""
    candidates = [m for m in net.modules() if isinstance(m, instance)]
    n = len(candidates)
    if n == 0:
        return None, 0, 0, "no_candidates"
    limits = []
    if max_modules is not None:
        if max_modules <= 0:
            return tuple(), n, 0, "explicit_zero_budget"
        limits.append(min(max_modules, n))
    if ratio is not None:
        if ratio <= 0:
            return tuple(), n, 0, "zero_ratio_budget"
        limits.append(max(1, min(n, ceil(n * ratio))))
    if not limits:
        return None, n, n, "all_candidates"
    k = min(limits)
    if k >= n:
        return None, n, n, "budget_covers_all"
    if dummy_input is None:
        return tuple(candidates[:k]), n, k, "fallback_module_order"
    net.to(device)
    sizes = _input_bytes(net, tuple(candidates), _to_device(dummy_input, device))
    order = sorted(range(n), key=lambda i: (-sizes[candidates[i]], i))
    return tuple(candidates[i] for i in order[:k]), n, k, "largest_input_activations"


def _selection_explanation(n, k, policy, checkpoint_budget, max_modules, ratio) -> str:
    if n == 0:
        return "No matching modules were found for checkpoint wrapping."
    if k == n:
        if checkpoint_budget is not None:
            return (f'Checkpoint budget "{checkpoint_budget}" covered all {n} matching modules, '
                    "so no module-level filtering was applied.")
        return f"All {n} matching modules were selected for checkpoint wrapping."
    if policy == "largest_input_activations":
        text = f"Selected {k} of {n} matching modules with the largest observed input activations."
        if checkpoint_budget is not None:
            text += f' This was driven by checkpoint budget "{checkpoint_budget}".'
        elif max_modules is not None or ratio is not None:
            text += " This was driven by the explicit selective-checkpoint budget."
        return text
    if policy == "fallback_module_order":
        return (f"Selected the first {k} of {n} matching modules by module order "
                "because no dummy_input was available to score activation sizes.")
    if policy == "explicit_zero_budget":
        return "Selective checkpointing budget was set to zero, so no modules were wrapped."
    if policy == "zero_ratio_budget":
        return "Selective checkpointing ratio budget was non-positive, so no modules were wrapped."
    return f'Selected {k} of {n} matching modules under policy "{policy}".'


def _recommendation(s: MemOptSummary) -> str:
    if s.gc_candidate_count == 0:
        return "No matching modules were found. Consider passing a different target instance tuple."
    by_prefer = {
        "speed": "Current settings favor training speed. If you need more memory reduction, try "
                 '`prefer="balanced"` or increase `gc_target_budget_ratio`.',
        "memory": "Current settings favor memory reduction. If optimization latency or training slowdown is too high, "
                  'try `prefer="balanced"` or `checkpoint_budget="speed"`.',
        "balanced": 'Current settings aim for a middle ground. Move to `prefer="speed"` for lower overhead or '
                    '`prefer="memory"` for more aggressive memory savings.',
    }
    if s.prefer in by_prefer:
        return by_prefer[s.prefer]
    if s.checkpoint_budget == "speed":
        return ("Checkpoint coverage is intentionally conservative. Increase to "
                '`checkpoint_budget="balanced"` or `"memory"` if you want more memory savings.')
    if s.checkpoint_budget == "memory":
        return ("Checkpoint coverage is already aggressive. To reduce optimization or training cost, "
                'drop to `checkpoint_budget="balanced"` or `"speed"`.')
    if s.profile == "safe":
        return ("You are using the conservative `safe` profile. If this does not save enough memory, "
                'try `profile="balanced"` or `prefer="balanced"`.')
    if s.profile == "exhaustive":
        return ("You are using the most expensive search mode. Keep it for offline tuning; for routine use, "
                'consider `profile="balanced"` or `prefer="balanced"`.')
    return ("Review `summary.gc_selected_count`, split counts, and skipped steps to decide whether to bias "
            "future runs toward speed or memory.")


def _resolve_options(level, profile, dummy_input, **given):
    if profile is not None and profile not in MEMOPT_PROFILES:
        raise ValueError(f"Unsupported memopt profile {profile!r}. Expected one of {MEMOPT_PROFILES}.")
    given = dict(level=level, **given)
    if profile is None:
        fallback = dict(level=0, compress_x=True, max_split_rounds=None, max_candidates_per_round=None,
                        warmup_in_main_process=True, warmup_in_profile_workers=True, allow_expensive_profiling=True)
        notes = []
    else:
        fallback = dict(zip(_OPTION_NAMES, _PROFILE_PRESETS[profile]))
        notes = [f"profile:{profile}"]
    # for an explicit profile None means "use the preset"; without a profile the two search limits stay None (= unlimited)
    opts = {k: (fallback[k] if given.get(k) is None else given[k]) for k in _OPTION_NAMES}
    if not opts["allow_expensive_profiling"] and opts["level"] > 1:
        opts.update(max_split_rounds=1, max_candidates_per_round=1, warmup_in_profile_workers=False)
    if dummy_input is None and opts["level"] > 1:
        if profile is None:
            raise ValueError("dummy_input must be provided for memory profiling.")
        notes.append("fallback:level>1_requires_dummy_input")
        opts.update(level=1, max_split_rounds=0, max_candidates_per_round=0, warmup_in_profile_workers=False)
    return opts, notes


def _resolve_preference(prefer, profile, checkpoint_budget):
    if prefer is not None and prefer not in MEMOPT_PREFERENCES:
        raise ValueError(f"Unsupported prefer {prefer!r}. Expected one of {MEMOPT_PREFERENCES}.")
    notes = []
    if prefer is not None:
        d_profile, d_budget = _PREFERENCE_DEFAULTS[prefer]
        if profile is None:
            profile = d_profile
            notes.append(f"prefer:profile={d_profile}")
        if checkpoint_budget is None:
            checkpoint_budget = d_budget
            notes.append(f"prefer:checkpoint_budget={d_budget}")
    return profile, checkpoint_budget, notes


def _resolve_budget(checkpoint_budget, max_modules, ratio):
    if checkpoint_budget is not None and checkpoint_budget not in MEMOPT_CHECKPOINT_BUDGETS:
        raise ValueError(f"Unsupported checkpoint_budget {checkpoint_budget!r}. Expected one of {MEMOPT_CHECKPOINT_BUDGETS}.")
    notes = []
    if checkpoint_budget is not None and ratio is None and max_modules is None:
        ratio = _BUDGET_RATIOS[checkpoint_budget]
        notes.append(f"checkpoint_budget:{checkpoint_budget}")
    return max_modules, ratio, notes


# ---------------------------------------------------------------------------------------------
# stage 1
# ---------------------------------------------------------------------------------------------
def apply_gc(net: nn.Module, instance, dummy_input: Optional[tuple] = None, compress_x: Optional[bool] = True,
             device: str = "cuda", checkpoint_budget: Optional[str] = None, max_gc_wrapped_modules: Optional[int] = None,
             gc_target_budget_ratio: Optional[float] = None, return_summary: bool = False):
    """Wrap modules of type ``instance`` in ``GCContainer``.

    Compressor per module: its ``x_compressor`` attribute if it has one (a compressor object or
    the name of a class in ``memopt.compress``); else ``BitSpikeCompressor`` when ``compress_x`` and
    the probe with ``dummy_input`` saw only binary inputs; else ``NullSpikeCompressor``.  A budget
    (``checkpoint_budget`` name, module count or ratio) keeps only the modules with the largest
    input activations.
    """
    info = dict(gc_wrap_count=0, manual_compressor_count=0, bit_compressor_count=0, null_compressor_count=0)
    candidates = [m for m in net.modules() if isinstance(m, instance)]
    max_modules, ratio, budget_notes = _resolve_budget(checkpoint_budget, max_gc_wrapped_modules, gc_target_budget_ratio)
    selected, n, k, policy = _select_targets(net, instance, dummy_input, device, max_modules, ratio)
    chosen = candidates if selected is None else list(selected)
    chosen_ids = {id(m) for m in chosen}
    paths = {id(m): name for name, m in net.named_modules() if name}
    info.update(gc_candidate_count=n, gc_selected_count=k, gc_selection_policy=policy, checkpoint_budget=checkpoint_budget,
                budget_notes=budget_notes, gc_selected_modules=[paths.get(id(m), "<root>") for m in chosen],
                gc_selection_explanation=_selection_explanation(n, k, policy, checkpoint_budget, max_modules, ratio))

    binary = {}
    if compress_x and dummy_input is not None:
        to_probe = tuple(m for m in chosen if getattr(m, "x_compressor", None) is None)
        if to_probe:
            net = net.to(device)
            binary = _probe_binary_inputs(net, to_probe, _to_device(dummy_input, device))

    def compressor_for(module):
        spec = getattr(module, "x_compressor", None)
        if not compress_x:
            info["null_compressor_count"] += 1
            return NullSpikeCompressor()
        if spec is not None:
            info["manual_compressor_count"] += 1
            return _compressor_from_spec(spec)
        if binary.get(module, False):
            info["bit_compressor_count"] += 1
            return BitSpikeCompressor()
        info["null_compressor_count"] += 1
        return NullSpikeCompressor()

    def rewrite(parent):
        for name, child in list(parent.named_children()):
            if isinstance(child, instance) and id(child) in chosen_ids:
                setattr(parent, name, GCContainer(compressor_for(child), child))
                info["gc_wrap_count"] += 1
            elif not isinstance(child, GCContainer):
                rewrite(child)

    rewrite(net)
    return (net, info) if return_summary else net


# ---------------------------------------------------------------------------------------------
# measurement
# ---------------------------------------------------------------------------------------------
def _bn_snapshot(net):
    return [(m, {k: (None if getattr(m, k) is None else getattr(m, k).clone())
                 for k in ("running_mean", "running_var", "num_batches_tracked")})
            for m in net.modules() if isinstance(m, nn.modules.batchnorm._BatchNorm)]


def _bn_restore(snapshot):
    with torch.no_grad():
        for m, state in snapshot:
            for k, v in state.items():
                if v is not None:
                    getattr(m, k).copy_(v)


def _dummy_train_step(net, dummy_input, restore_bn: bool = False):
    """forward + backward of ``sum(outputs)`` in training mode, then reset; gradients are dropped."""
    net.train()
    net.zero_grad(set_to_none=True)
    snapshot = _bn_snapshot(net) if restore_bn else None
    inputs = _tree_map(lambda t: t.clone().detach().requires_grad_(t.is_floating_point()), dummy_input)
    out = net(*inputs)

    def total(o):
        if isinstance(o, torch.Tensor):
            return o.sum()
        if isinstance(o, (tuple, list)):
            return sum(total(t) for t in o)
        if isinstance(o, dict):
            return sum(total(t) for t in o.values())
        return 0.0

    total(out).backward()
    net.zero_grad(set_to_none=True)
    functional.reset_net(net)
    if snapshot is not None:
        _bn_restore(snapshot)


class _Bench:
    """Measures a candidate network on ``device`` (on a private deep copy, so the caller's weights,
    BN statistics and neuron state are untouched)."""

    def __init__(self, dummy_input, device: str, warmup: bool):
        self.device, self.warmup = device, warmup
        self.dummy_input = _to_device(dummy_input, device)

    def _clone(self, net):
        return copy.deepcopy(net).to(self.device)

    def peak(self, net) -> int:
        probe = self._clone(net)
        if self.warmup:
            _dummy_train_step(probe, self.dummy_input)
        with make_meter(self.device, (probe,)) as meter:
            meter.reset_peak()
            _dummy_train_step(probe, self.dummy_input)
            meter.settle()
            return meter.peak()

    def memory_ranking(self, net):
        """Paths of the GCContainers, largest training footprint first."""
        probe = self._clone(net)
        if self.warmup:
            _dummy_train_step(probe, self.dummy_input)
        with LayerWiseMemoryProfiler((probe,), ("net",), ("submodules",), (GCContainer,), device=self.device,
                                     log_path=os.devnull, data_path=os.devnull) as prof:
            _dummy_train_step(probe, self.dummy_input)
            rows = prof.export(output=False)
        return [r[0].split(" ")[-1] for r in rows]

    def forward_time_ranking(self, net, repeats: int = 50):
        probe = self._clone(net).eval()
        with torch.no_grad(), LayerWiseFPCUDATimeProfiler((probe,), ("net",), ("submodules",), (GCContainer,),
                                                          log_path=os.devnull) as prof:
            for _ in range(repeats):
                probe(*self.dummy_input)
                functional.reset_net(probe)
            rows = prof.export(output=False)
        return [r[0].split(" ")[-1] for r in rows]


def get_module_and_parent(net: nn.Module, module_name: str) -> Tuple[nn.Module, nn.Module, str]:
    """``"net's a.b.2"`` or ``"a.b.2"`` -> (module, its parent, ``"2"``)."""
    parts = module_name.split(" ")[-1].split(".")
    parent = net
    for p in parts[:-1]:
        parent = getattr(parent, p)
    return getattr(parent, parts[-1]), parent, parts[-1]


# ---------------------------------------------------------------------------------------------
# container surgery
# ---------------------------------------------------------------------------------------------
def _spatial_pieces(block: GCContainer):
    if len(block) > 1:
        return list(block)
    if len(block) == 1 and hasattr(block[0], "__spatial_split__"):
        return list(block[0].__spatial_split__())
    return None


def _split_spatially(block: GCContainer, compress_x: bool = True):
    """One container per sub-block; only the first keeps the original input compressor (the input
    of the others is an intermediate activation of unknown range)."""
    pieces = _spatial_pieces(block)
    if pieces is None:
        return None
    wrapped = []
    for i, piece in enumerate(pieces):
        spec = getattr(piece, "x_compressor", None)
        if not compress_x:
            c = NullSpikeCompressor()
        elif spec is not None:
            c = _compressor_from_spec(spec)
        else:
            c = copy.deepcopy(block.x_compressor) if i == 0 else NullSpikeCompressor()
        wrapped.append(GCContainer(c, piece))
    return nn.Sequential(*wrapped)


def _temporal_ok(block: GCContainer) -> bool:
    return not any(isinstance(m, tuple(TCGC_FORBIDDEN_MODULES)) for m in block.modules())


def _split_temporally(block: GCContainer, factor: int = 2):
    if not _temporal_ok(block):
        return None
    return TCGCContainer(block.x_compressor, *block, n_chunk=getattr(block, "n_chunk", 1) * factor,
                         n_seq_inputs=getattr(block[0], "n_seq_inputs", 1), n_outputs=getattr(block[-1], "n_outputs", 1))


def _unwrap(block: GCContainer) -> nn.Module:
    return block[0] if len(block) == 1 else nn.Sequential(*block)


def _containers(net):
    return [m for m in net.modules() if isinstance(m, GCContainer)]


def _greedy_split(net, bench: _Bench, peak: int, can_split, split, max_rounds, max_candidates, tag: str, summary, counter: str):
    """Rounds of: rank containers by footprint, try the top candidates, keep the first split that
    lowers the peak.  Stops when a round brings no improvement."""
    rounds, blocked = 0, set()
    while True:
        if max_rounds is not None and rounds >= max_rounds:
            break
        if not any(can_split(c) for c in _containers(net)):
            break
        rounds += 1
        ranking = [p for p in bench.memory_ranking(net) if p not in blocked]
        if max_candidates is not None:
            ranking = ranking[:max(max_candidates, 0)]
        if not ranking:
            break
        improved = False
        for path in ranking:
            block, parent, child = get_module_and_parent(net, path)
            replacement = split(block)
            if replacement is None:
                blocked.add(path)
                continue
            setattr(parent, child, replacement)
            new_peak = bench.peak(net)
            if new_peak >= peak:
                logger.debug("\t%s: no reduction in memory, revert (%s -> %s)", path, peak, new_peak)
                setattr(parent, child, block)
                blocked.add(path)
                continue
            logger.debug("\t%s: split (%s -> %s)", path, peak, new_peak)
            peak = new_peak
            setattr(summary, counter, getattr(summary, counter) + 1)
            improved = True
            blocked.clear()
            break
        if not improved:
            summary.skipped_steps.append(f"{tag}:no_improving_candidate")
            break
    return peak


# ---------------------------------------------------------------------------------------------
# entry point
# ---------------------------------------------------------------------------------------------
def memory_optimization(net: nn.Module, instance, dummy_input: Optional[tuple] = None, compress_x: Optional[bool] = None,
                        level: Optional[int] = None, temporal_split_factor: int = 2, max_split_rounds: Optional[int] = None,
                        max_candidates_per_round: Optional[int] = None, warmup_in_main_process: Optional[bool] = None,
                        warmup_in_profile_workers: Optional[bool] = None, prefer: Optional[str] = None,
                        profile: Optional[str] = None, allow_expensive_profiling: Optional[bool] = None,
                        checkpoint_budget: Optional[str] = None, max_gc_wrapped_modules: Optional[int] = None,
                        gc_target_budget_ratio: Optional[float] = None, return_summary: bool = False):
    """Rewrite ``net`` for lower training memory (stages 1-4, see the module docstring).  Returns the
    network **on the CPU** (and the ``MemOptSummary`` when ``return_summary``)."""
    t0 = time.time()
    device = resolve_device()
    profile, checkpoint_budget, notes = _resolve_preference(prefer, profile, checkpoint_budget)
    requested_level = level if level is not None else {"safe": 1, "balanced": 2, "memory": 3, "exhaustive": 4}.get(profile, 0)
    opts, more_notes = _resolve_options(level, profile, dummy_input, compress_x=compress_x, max_split_rounds=max_split_rounds,
                                        max_candidates_per_round=max_candidates_per_round,
                                        warmup_in_main_process=warmup_in_main_process,
                                        warmup_in_profile_workers=warmup_in_profile_workers,
                                        allow_expensive_profiling=allow_expensive_profiling)
    level, compress_x = opts["level"], opts["compress_x"]
    summary = MemOptSummary(profile=profile, checkpoint_budget=checkpoint_budget, prefer=prefer, device=device,
                            requested_level=requested_level, applied_level=level, compress_x=compress_x,
                            allow_expensive_profiling=opts["allow_expensive_profiling"], notes=notes + more_notes,
                            options=dict(prefer=prefer, temporal_split_factor=temporal_split_factor,
                                         max_split_rounds=opts["max_split_rounds"],
                                         max_candidates_per_round=opts["max_candidates_per_round"],
                                         warmup_in_main_process=opts["warmup_in_main_process"],
                                         warmup_in_profile_workers=opts["warmup_in_profile_workers"],
                                         checkpoint_budget=checkpoint_budget, max_gc_wrapped_modules=max_gc_wrapped_modules,
                                         gc_target_budget_ratio=gc_target_budget_ratio))
    bench = _Bench(dummy_input, device, opts["warmup_in_profile_workers"]) if dummy_input is not None else None
    peak = -1

    if level > 0:
        net, info = apply_gc(net, instance, dummy_input, compress_x, device, checkpoint_budget=checkpoint_budget,
                             max_gc_wrapped_modules=max_gc_wrapped_modules, gc_target_budget_ratio=gc_target_budget_ratio,
                             return_summary=True)
        summary.applied_steps.append("level1_gc")
        summary.notes.extend(info.pop("budget_notes"))
        info.pop("checkpoint_budget")
        for k, v in info.items():
            setattr(summary, k, v)

    if level > 1:
        if not _containers(net):
            summary.skipped_steps.append("level2:no_gccontainers")
        elif not any(_spatial_pieces(c) is not None for c in _containers(net)):
            summary.skipped_steps.append("level2:no_spatial_candidates")
        else:
            summary.applied_steps.append("level2_spatial_split")
            peak = bench.peak(net)
            peak = _greedy_split(net, bench, peak, lambda c: _spatial_pieces(c) is not None,
                                 lambda c: _split_spatially(c, compress_x), opts["max_split_rounds"],
                                 opts["max_candidates_per_round"], "level2", summary, "spatial_split_count")

    if level > 2:
        if not _containers(net):
            summary.skipped_steps.append("level3:no_gccontainers")
        elif not any(_temporal_ok(c) for c in _containers(net)):
            summary.skipped_steps.append("level3:no_temporal_candidates")
        else:
            summary.applied_steps.append("level3_temporal_split")
            if peak < 0:
                peak = bench.peak(net)
            peak = _greedy_split(net, bench, peak, _temporal_ok, lambda c: _split_temporally(c, temporal_split_factor),
                                 opts["max_split_rounds"], opts["max_candidates_per_round"], "level3", summary,
                                 "temporal_split_count")

    if level > 3:
        if not _containers(net):
            summary.skipped_steps.append("level4:no_gccontainers")
        else:
            summary.applied_steps.append("level4_greedy_unwrap")
            if peak < 0:
                peak = bench.peak(net)
            for path in bench.forward_time_ranking(net):
                try:
                    block, parent, child = get_module_and_parent(net, path)
                except AttributeError:
                    continue          # an enclosing container was already removed
                if not isinstance(block, GCContainer):
                    continue
                setattr(parent, child, _unwrap(block))
                new_peak = bench.peak(net)
                if new_peak > peak:
                    setattr(parent, child, block)
                else:
                    peak = new_peak
                    summary.unwrap_count += 1

    if opts["warmup_in_main_process"] and dummy_input is not None:
        net = net.to(device)
        _dummy_train_step(net, _to_device(dummy_input, device), restore_bn=True)

    net = net.cpu()
    summary.gc_container_count = len(_containers(net))
    summary.tcgc_container_count = sum(isinstance(m, TCGCContainer) for m in net.modules())
    summary.recommendation = _recommendation(summary)
    logger.debug("memory_optimization took %.2fs", time.time() - t0)
    logger.info("Memory optimization completed: device=%s profile=%s requested_level=%s applied_level=%s "
                "applied_steps=%s skipped_steps=%s", summary.device, summary.profile, summary.requested_level,
                summary.applied_level, len(summary.applied_steps), len(summary.skipped_steps),
                extra={"event": "memopt_profile_summary", "device": summary.device, "profile": summary.profile,
                       "requested_level": summary.requested_level, "applied_level": summary.applied_level,
                       "gc_candidate_count": summary.gc_candidate_count, "gc_selected_count": summary.gc_selected_count})
    return (net, summary) if return_summary else net
