"""Run-time energy of a training or inference step on the NeuroMC-like accelerator model
(``op_counter/neuromc/core.py:1-2234`` of the reference).

The profiler watches a real step.  Forward and backward hooks on the layers the model knows (Conv1d/2d, Linear,
BatchNorm1d/2d/3d, spiking neurons) turn every call into a *fragment*: a loop nest ``B, T, C, K, OY, OX, FY, FX`` with a
core type, operand sizes and precisions.  A fragment's energy is the sum of

* its multiply-accumulates at the core's MAC cost (a core fed by spikes selects and adds: add + 1/16 mux; a dense core
  multiplies and adds),
* the *base* traffic of a contraction: both operands read from, and the result written to, the core's own SRAM macros
  and registers (a weight tile that fits its macro is fetched once for repeated batch / time tiles),
* the *extra* work of what surrounds the contraction - the soma (integrate, compare, reset, surrogate gradient), batch
  norm (statistics, normalisation and its closed-form backward), the optimizer update - as primitive operations
  (add / mul / comp / mux / sqrt) and as the named intermediate variables they stream through the shared buffers.

Which traffic counts is decided by :class:`MemoryHierarchyConfig`.  ATen operators executed outside the hooked layers
(activation functions, losses, reshapes ...) are listed in ``report.warnings`` (or raise with ``strict=True``): the
model has no core for them.  Stage names select the phase (``"backward"`` / ``"optimizer"`` / ``"update"`` in the name,
otherwise forward), tiling position (``b<i>`` / ``t<j>`` tokens, e.g. ``"forward_b1_t0"``) and ``without_bp_bn``.
"""
from __future__ import annotations

import re
from collections import defaultdict
from contextlib import contextmanager
from dataclasses import dataclass, field
from math import prod
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
from torch.overrides import resolve_name
from torch.utils._python_dispatch import TorchDispatchMode

from ..base import call_model
from .config import MemoryHierarchyConfig, MemoryInstanceSpec
from .counters import is_spike

__all__ = ["MemoryHierarchyConfig", "NeuroMCEnergyProfiler", "NeuroMCRuntimeEnergyReport", "estimate_neuromc_runtime_energy"]

CORE_TYPES = frozenset({"fp_soma", "fp_bn", "bp_grad", "bp_bn", "bp_grad_opt", "wg", "ann_fe", "ann_be", "ann_we", "ann_bn", "ann_bn_bp"})
_ADD, _MUL, _MUX = 0.548, 0.812, 0.548 / 16.0
OP_COST_PJ = {"mux": _MUX, "add": _ADD, "mul": _MUL, "comp": 0.056, "sqrt": 0.514}
MAC_COST_PJ = {"fp_soma": _ADD + _MUX, "wg": _ADD + _MUX, "bp_grad": _ADD + _MUL, "ann_fe": _ADD + _MUL, "ann_be": _ADD + _MUL, "ann_we": _ADD + _MUL}

#: core type -> (register of operand 1, operand 2, result), (SRAM of operand 1, operand 2, result)
_CORE_MEMORIES = {
    "fp_soma": (("reg_1b", "reg_16b", "reg_16b"), ("sram_fp_conv_in_s", "sram_fp_conv_in_w", "sram_fp_conv_out_xi")),
    "ann_fe": (("reg_16b",) * 3, ("sram_fp_conv_in_w", "sram_fp_conv_in_w", "sram_fp_conv_out_xi")),
    "bp_grad": (("reg_16b",) * 3, ("sram_bp_conv_in_du", "sram_bp_conv_in_w", "sram_bp_conv_out_res")),
    "ann_be": (("reg_16b",) * 3, ("sram_bp_conv_in_du", "sram_bp_conv_in_w", "sram_bp_conv_out_res")),
    "ann_we": (("reg_16b",) * 3, ("sram_wg_conv_in_du", "sram_wg_conv_in_du", "sram_wg_conv_out_dw")),
    "wg": (("reg_1b", "reg_16b", "reg_16b"), ("sram_wg_conv_in_s", "sram_wg_conv_in_du", "sram_wg_conv_out_dw")),
}
_W16 = ("reg_16b", "sram_2MB")
_W32 = ("reg_32b", "sram_6MB")
#: (process key, phase) -> intermediate variables: name -> (size key, bits, register, SRAM)
_EXTRA_VARIABLES = {
    ("with_sg", "forward"): {"fp_yi1": ("OYOXKBT", 16, "reg_16b", "sram_fp_conv_out_xi"), "fp_u_l": ("OYOXKBT", 16, "reg_16b", "sram_fp_soma_u"),
                             "fp_s_l": ("OYOXKBT", 1, "reg_1b", "sram_fp_soma_s"), "fp_smask_l": ("OYOXKBT", 1, "reg_1b", "sram_fp_soma_smask")},
    ("with_sg", "backward"): {"bp_conv_res": ("OYOXCBT", 16, "reg_16b", "sram_bp_conv_out_res"), "bp_u_l_pre": ("OYOXCBT", 16, "reg_16b", "sram_bp_grad_in_u"),
                              "bp_s_l_pre": ("OYOXCBT", 1, "reg_1b", "sram_bp_grad_in_s"), "bp_smask_l_pre": ("OYOXCBT", 1, "reg_1b", "sram_bp_grad_in_smask"),
                              "bp_du_l_pre": ("OYOXCBT", 16, "reg_16b", "sram_bp_grad_out_du")},
    ("with_bn", "forward"): {n: (k, 16, *_W16) for n, k in (("fp_bn_mean_v", "KT"), ("fp_bn_variance", "KT"), ("fp_bn_n", "OYOXKBT"), ("fp_bn_sqrt", "KT"),
                                                             ("fp_bn_xi_", "OYOXKBT"), ("fp_bn_y", "KT"), ("fp_bn_b", "KT"))},
    ("with_bn", "backward"): {n: (k, 16, *_W16) for n, k in (("bp_bn_du_l_pre1", "OYOXCBT"), ("bp_bn_sqrt", "CT"), ("bp_bn_y", "CT"), ("bp_bn_m", "OYOXCBT"),
                                                              ("bp_bn_n", "OYOXCBT"), ("bp_bn_sigma_m", "CT"), ("bp_bn_sigma_n", "CT"), ("bp_bn_sigma_mn", "CT"),
                                                              ("bp_bn_dy", "CT"), ("bp_bn_db", "CT"), ("bp_bn_du_l_pre2", "OYOXCBT"))},
    # Adam / AdamW: parameter, gradient, both moments, both bias-corrected moments, updated parameter (fp32 master copies)
    ("with_opt", "optimizer"): {f"opt_{n}": ("P", 32, *_W32) for n in ("w", "dw", "v", "s", "vbc", "sbc", "w_updated")},
}
_VIEW_PREFIXES = ("aten.detach", "aten.view", "aten.t.default", "aten.transpose", "aten.permute", "aten.expand", "aten.slice", "aten.select",
                  "aten.alias", "aten._unsafe_view", "aten.as_strided", "aten.clone", "aten.copy_", "aten.reshape", "aten.unsqueeze", "aten.squeeze",
                  "aten.empty", "aten.zeros", "aten.ones", "aten.full", "aten.new_", "aten.lift_fresh", "aten._to_copy", "aten._local_scalar_dense",
                  "aten.unbind", "aten.stack", "aten.cat", "aten.split", "aten.flatten", "aten.unflatten", "profiler.")


@dataclass
class NeuroMCRuntimeEnergyReport:
    """All energies in pJ.  ``energy_total = energy_compute + energy_memory``; ``energy_compute = energy_mac +
    energy_extra_compute``; ``energy_memory = energy_base_memory + energy_extra_memory``."""
    energy_total_pj: float = 0.0
    energy_compute_pj: float = 0.0
    energy_memory_pj: float = 0.0
    energy_by_stage: Dict[str, float] = field(default_factory=dict)
    energy_by_op: Dict[str, float] = field(default_factory=dict)
    primitive_counts: Dict[str, Any] = field(default_factory=dict)
    memory_bits_by_level: Dict[str, Any] = field(default_factory=dict)
    warnings: List[str] = field(default_factory=list)
    energy_mac_pj: float = 0.0
    energy_base_memory_pj: float = 0.0
    energy_extra_memory_pj: float = 0.0
    energy_extra_compute_pj: float = 0.0
    energy_by_core_type: Dict[str, float] = field(default_factory=dict)
    energy_by_process_key: Dict[str, float] = field(default_factory=dict)
    energy_by_memory_level_dir: Dict[str, Dict[str, float]] = field(default_factory=dict)
    counts_by_core_type: Dict[str, Dict[str, int]] = field(default_factory=dict)
    counts_by_process_key: Dict[str, Dict[str, int]] = field(default_factory=dict)
    mapping_summary: List[Dict[str, Any]] = field(default_factory=list)

    def summary(self) -> str:
        lines = [f"total {self.energy_total_pj / 1e6:.4f} uJ  (compute {self.energy_compute_pj / 1e6:.4f}, memory {self.energy_memory_pj / 1e6:.4f})"]
        lines += [f"  {stage}: {e / 1e6:.4f} uJ" for stage, e in self.energy_by_stage.items()]
        lines += [f"  warning: {w}" for w in self.warnings]
        return "\n".join(lines)


@dataclass
class _Fragment:
    stage: str
    phase: str
    op_name: str
    core_type: str
    process_key: str
    loop_dims: Dict[str, int]
    bits: Tuple[int, int, int]              # operand 1, operand 2 (weight), result
    numel: Tuple[int, int, int]
    mac_count: int
    conv_type: str = "--"
    b_type: int = 0
    t_type: int = 0
    optimizer: Dict[str, bool] = field(default_factory=dict)
    source: str = "module"                  # "module": seen by a layer hook; "trace": recovered from the operator trace


def _layout(x, module) -> Tuple[int, int, int, Tuple[int, ...]]:
    """``(T, B, C, spatial)`` of an activation; a leading time axis is recognised from the module's step mode."""
    if not torch.is_tensor(x):
        return 1, 1, 1, ()
    shape = tuple(x.shape)
    if getattr(module, "step_mode", "s") == "m" and len(shape) >= 3:
        return shape[0], shape[1], shape[2], shape[3:]
    if len(shape) == 1:
        return 1, 1, shape[0], ()
    return 1, shape[0], shape[1], shape[2:]


def _dims(B, T, C, K, OY=1, OX=1, FY=1, FX=1) -> Dict[str, int]:
    return {k: max(int(v), 1) for k, v in dict(B=B, T=T, C=C, K=K, OY=OY, OX=OX, FY=FY, FX=FX).items()}


def _first(x):
    while isinstance(x, (tuple, list)) and x:
        x = x[0]
    return x


class _Watch(TorchDispatchMode):
    """Notes the ATen operators that run while no hooked layer is active."""

    def __init__(self, owner):
        super().__init__()
        self.owner = owner

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        out = func(*args, **(kwargs or {}))
        self.owner._saw(resolve_name(func))
        return out


_AUXILIARY = re.compile(r"aten\.(add|sub|rsub|mul|div|where|eq|ne|lt|le|gt|ge|logical_\w+|sum|mean|sigmoid|sqrt|rsqrt|all|index|mse_loss\w*|"
                        r"ones_like|zeros_like|full_like)_?\.")


class NeuroMCEnergyProfiler:
    """``with profiler: with profiler.stage("forward"): ...`` around a real step of a bound model; then :meth:`get_report`.
    ``core_type`` names the accelerator core the run is mapped to (kept in the report; the per-layer core types follow from
    whether a layer's input is binary)."""

    def __init__(self, *, core_type: str = "fp_soma", memory_config: Optional[MemoryHierarchyConfig] = None, strict: bool = False,
                 extra_ignore_modules: Optional[list] = None):
        if core_type not in CORE_TYPES:
            raise ValueError(f"core_type must be one of {sorted(CORE_TYPES)}, got {core_type!r}.")
        self.core_type = core_type
        self.memory_config = (memory_config or MemoryHierarchyConfig.neuromc_like_v1()).copy()
        self.memory_config.validate()
        self.strict = strict
        self.extra_ignore_modules = list(extra_ignore_modules or [])
        self._stage: List[str] = []
        self._fragments: List[_Fragment] = []
        self._outside: Dict[str, int] = defaultdict(int)
        self._inside = 0
        self._active = self._suspended = False
        self._model: Optional[nn.Module] = None
        self._optimizer = None
        self._handles: list = []
        self._watch = _Watch(self)

    # -- binding ------------------------------------------------------------------------------------------------------
    def bind_model(self, model: nn.Module) -> None:
        if self._model is not None:
            if self._model is model:
                return
            raise RuntimeError("NeuroMCEnergyProfiler is already bound to a different model.")
        from ...neuron.base_node import BaseNode
        kinds = (nn.Conv1d, nn.Conv2d, nn.Linear, nn.BatchNorm1d, nn.BatchNorm2d, nn.BatchNorm3d, BaseNode)
        mods = [m for m in model.modules() if m not in self.extra_ignore_modules]
        if any(isinstance(m, nn.Conv3d) for m in mods):
            raise ValueError("Exact NeuroMC runtime does not support nn.Conv3d yet.")
        self._model = model
        for m in mods:
            if isinstance(m, kinds):
                self._handles += [m.register_forward_pre_hook(self._enter_layer), m.register_forward_hook(self._forward_hook),
                                  m.register_full_backward_hook(self._backward_hook)]

    def bind_optimizer(self, optimizer) -> None:
        self._optimizer = optimizer

    def __enter__(self):
        self._watch.__enter__()
        self._active = True
        return self

    def __exit__(self, exc_type, exc, tb):
        self._active = False
        for h in self._handles:
            h.remove()
        self._handles.clear()
        if self._model is not None:
            for m in self._model.modules():
                m.__dict__.pop("_neuromc_last_input", None)
        self._model = None
        return self._watch.__exit__(exc_type, exc, tb)

    @contextmanager
    def stage(self, name: str):
        if not self._active:
            raise RuntimeError("stage() can only be used inside active profiler context.")
        if self._stage:
            raise RuntimeError("Nested stage() is not supported in NeuroMC v2.")
        self._stage.append(name)
        try:
            yield self
        finally:
            self._stage.pop()

    @contextmanager
    def suspend(self):
        old, self._suspended = self._suspended, True
        try:
            yield self
        finally:
            self._suspended = old

    # -- stage names --------------------------------------------------------------------------------------------------
    def _current_stage(self) -> str:
        return self._stage[-1] if self._stage else "unlabeled"

    def _phase(self, stage: Optional[str] = None) -> str:
        name = (stage or self._current_stage()).lower()
        return "backward" if "backward" in name else "optimizer" if ("optimizer" in name or "update" in name) else "forward"

    def _position(self, stage: str) -> Tuple[int, int]:
        find = lambda letter: re.search(rf"(?:^|[^a-z0-9]){letter}(\d+)(?:[^a-z0-9]|$)", stage.lower())
        b, t = find("b"), find("t")
        return (int(b.group(1)) if b else 0, int(t.group(1)) if t else 0)

    # -- what runs ----------------------------------------------------------------------------------------------------
    def _saw(self, op: str) -> None:
        if self._active and not self._suspended and self._inside == 0 and self._phase() == "forward":
            if not op.startswith(_VIEW_PREFIXES) and not _AUXILIARY.match(op):
                self._outside[op] += 1

    def _enter_layer(self, module, args):
        self._inside += 1

    def _forward_hook(self, module, args, out):
        self._inside = max(self._inside - 1, 0)
        if not self._active or self._suspended:
            return
        from ...neuron.base_node import BaseNode
        x = _first(args)
        stage = self._current_stage()
        with self.suspend():                          # the profiler's own tensor inspections are not part of the run
            module.__dict__["_neuromc_last_input"] = x.detach() if torch.is_tensor(x) else None
            if isinstance(module, (nn.Conv1d, nn.Conv2d, nn.Linear)):
                self._fragments.append(self._contraction(stage, "forward", module, x, _first(out)))
            elif isinstance(module, (nn.BatchNorm1d, nn.BatchNorm2d, nn.BatchNorm3d)):
                self._fragments.append(self._pointwise(stage, "forward", "bn", module, x, _first(out)))
            elif isinstance(module, BaseNode):
                self._fragments.append(self._pointwise(stage, "forward", "soma", module, x, _first(out)))

    def _backward_hook(self, module, grad_input, grad_output):
        if not self._active or self._suspended:
            return
        from ...neuron.base_node import BaseNode
        stage = self._current_stage()
        x, gy, gx = module.__dict__.get("_neuromc_last_input"), _first(grad_output), _first(grad_input)
        with self.suspend():
            if isinstance(module, (nn.Conv1d, nn.Conv2d, nn.Linear)):
                if torch.is_tensor(gx):
                    self._fragments.append(self._contraction(stage, "backward", module, gy, gx, role="grad_input", layer_input=x))
                if module.weight.requires_grad:
                    self._fragments.append(self._contraction(stage, "backward", module, x, gy, role="grad_weight", layer_input=x))
            elif isinstance(module, (nn.BatchNorm1d, nn.BatchNorm2d, nn.BatchNorm3d)):
                self._fragments.append(self._pointwise(stage, "backward", "bn", module, gy, gx if torch.is_tensor(gx) else gy))
            elif isinstance(module, BaseNode):
                self._fragments.append(self._pointwise(stage, "backward", "soma", module, gy, gx if torch.is_tensor(gx) else gy))

    # -- fragments ----------------------------------------------------------------------------------------------------
    def _contraction(self, stage, phase, module, a, b, role: str = "forward", layer_input=None) -> _Fragment:
        """Forward: ``a`` = input, ``b`` = output.  ``grad_input``: ``a`` = output gradient, ``b`` = input gradient.
        ``grad_weight``: ``a`` = layer input, ``b`` = output gradient."""
        act_out = b if role == "forward" else (a if role == "grad_input" else b)
        T, B, _, spatial = _layout(act_out, module)
        if isinstance(module, nn.Linear):
            C, K, oy, ox, fy, fx = module.in_features, module.out_features, 1, 1, 1, 1
            if torch.is_tensor(act_out) and act_out.dim() > 2 and getattr(module, "step_mode", "s") != "m":
                B = prod(act_out.shape[:-1])                      # tokens of a [B, L, C] activation are batch
                T = 1
        else:
            k = tuple(module.kernel_size) + (1,) * (2 - len(module.kernel_size))
            sp = tuple(spatial) + (1,) * (2 - len(spatial)) if len(spatial) < 2 else tuple(spatial[:2])
            C, K, oy, ox, fy, fx = module.in_channels // module.groups, module.out_channels, sp[0], sp[1], k[0], k[1]
        dims = _dims(B, T, C, K, oy, ox, fy, fx)
        spikes_in = is_spike(layer_input if layer_input is not None else a)
        if role == "forward":
            core, name, bits = ("fp_soma" if spikes_in else "ann_fe"), "forward", (1 if spikes_in else 16, 16, 16)
            numel = (a.numel(), module.weight.numel(), b.numel())
        elif role == "grad_input":
            core, name, bits = ("bp_grad" if spikes_in else "ann_be"), "backward.grad_input", (16, 16, 16)
            numel = (a.numel(), module.weight.numel(), b.numel())
        else:
            core, name, bits = ("wg" if spikes_in else "ann_we"), "backward.grad_weight", (1 if spikes_in else 16, 16, 16)
            numel = (a.numel() if torch.is_tensor(a) else 0, b.numel(), module.weight.numel())
        kind = "linear" if isinstance(module, nn.Linear) else "conv"
        bt, tt = self._position(stage)
        return _Fragment(stage, phase, f"{kind}.{name}", core, "with_nothing", dims, bits, numel, prod(dims.values()), b_type=bt, t_type=tt)

    def _pointwise(self, stage, phase, kind, module, a, b) -> _Fragment:
        ref = b if (kind == "soma" and phase == "forward") else a
        T, B, C, spatial = _layout(ref, module)
        dims = _dims(B, T, C, C, max(prod(spatial), 1) if spatial else 1)
        bt, tt = self._position(stage)
        if kind == "bn":
            spikes = is_spike(a) if phase == "forward" else False
            core = {("forward", True): "fp_bn", ("forward", False): "ann_bn", ("backward", True): "bp_bn", ("backward", False): "ann_bn_bp"}[(phase, spikes)]
            conv_type = "without_bp_bn" if "without_bp_bn" in stage.lower() else "--"
            return _Fragment(stage, phase, f"bn.{phase}", core, "with_bn", dims, (16, 16, 16), (a.numel(), 2 * C, b.numel()), 0, conv_type=conv_type)
        core = "fp_soma" if phase == "forward" else "bp_grad"
        out_bits = 1 if phase == "forward" else 16
        return _Fragment(stage, phase, f"soma.{phase}", core, "with_sg", dims, (16, 16, out_bits), (a.numel(), 0, b.numel()), 0, b_type=bt, t_type=tt)

    def record_optimizer_step(self, stage: str = "optimizer") -> None:
        """Adam / AdamW: one fragment for the whole update.  SGD: one fragment per (momentum, weight decay, momentum buffer
        present, vector or matrix) bucket.  ``K`` of the loop dimensions holds the element count of the vector parameters (biases,
        normalisation scales and shifts), ``FX`` the element count of all others."""
        opt = self._optimizer
        if opt is None:
            return
        kind = type(opt).__name__.lower()
        if kind not in ("sgd", "adam", "adamw"):
            raise ValueError(f"NeuroMC models SGD, Adam and AdamW updates, got {type(opt).__name__}.")
        buckets: Dict[Tuple[bool, bool, bool, str], int] = defaultdict(int)
        for group in opt.param_groups:
            if kind == "sgd" and (group.get("nesterov") or group.get("dampening", 0) != 0 or group.get("maximize")):
                raise ValueError("NeuroMC SGD model supports plain / momentum / weight-decay SGD only (no nesterov, dampening or maximize).")
            momentum, decay = kind == "sgd" and float(group.get("momentum", 0.0)) > 0, kind == "sgd" and float(group.get("weight_decay", 0.0)) > 0
            for p in group["params"]:
                if p.grad is None:
                    continue
                has_buffer = momentum and "momentum_buffer" in opt.state.get(p, {})
                key = (momentum, decay, has_buffer) if kind == "sgd" else (False, False, False)
                buckets[key + ("vector" if p.dim() <= 1 else "matrix",)] += int(p.numel())
        groups: Dict[Tuple[bool, bool, bool], Dict[str, int]] = defaultdict(lambda: {"vector": 0, "matrix": 0})
        for (m, d, buf, shape), count in buckets.items():
            groups[(m, d, buf)][shape] += count
        for (m, d, buf), sizes in groups.items():
            # SGD keeps vectors and matrices in fragments of their own, Adam puts both in one
            parts = [(sizes["vector"], sizes["matrix"])] if kind != "sgd" else [(sizes["vector"], 0), (0, sizes["matrix"])]
            for vec, mat in parts:
                if vec + mat == 0:
                    continue
                dims = _dims(1, 1, 1, vec, 1, 1, 1, mat)
                dims["K"], dims["FX"] = vec, mat                              # either may be zero
                self._fragments.append(_Fragment(stage, "optimizer", kind, "bp_grad_opt", "with_opt", dims, (32, 32, 32), (vec, mat, vec + mat), 0,
                                                 optimizer={"momentum": m, "weight_decay": d, "momentum_buffer": buf}, source="optimizer"))

    # -- accounting ---------------------------------------------------------------------------------------------------
    def _charge(self, bits_out, energy_out, level: str, direction: str, bits: int, spec: MemoryInstanceSpec, word: int, read: bool) -> None:
        cfg = self.memory_config
        if bits <= 0 or word <= 0:
            return
        if (level == "dram" and cfg.zero_dram_in_paper_energy) or (level == "noc" and cfg.zero_noc_in_paper_energy):
            return
        if level == "sram" and cfg.zero_sram_high_directions and direction in ("rl2h", "wh2l"):
            return
        port, cost = (spec.r_bw, spec.r_cost) if read else (spec.w_bw, spec.w_cost)
        if port <= 0:
            return
        bits_out[level][direction] += bits
        energy_out[level][direction] += (bits / word) * cost / (port / word)      # elements x energy per element

    def _base_memory(self, f: _Fragment):
        bits, energy = defaultdict(lambda: defaultdict(int)), defaultdict(lambda: defaultdict(float))
        if f.core_type not in _CORE_MEMORIES or f.mac_count == 0:
            return bits, energy
        inst = self.memory_config.memory_instances
        regs, srams = _CORE_MEMORIES[f.core_type]
        operand_bits = [n * b for n, b in zip(f.numel, f.bits)]
        weight_stays = (f.b_type > 0 or f.t_type > 0) and operand_bits[1] <= inst[srams[1]].size_bits
        for i, (direction, read) in enumerate((("rh2l", True), ("rh2l", True), ("wl2h", False))):
            if i == 1 and weight_stays:
                continue
            self._charge(bits, energy, "reg", direction, operand_bits[i], inst[regs[i]], f.bits[i], read)
            self._charge(bits, energy, "sram", direction, operand_bits[i], inst[srams[i]], f.bits[i], read)
        return bits, energy

    @staticmethod
    def _sizes(f: _Fragment) -> Dict[str, int]:
        d = f.loop_dims
        plane = d["OY"] * d["OX"] * d["B"] * d["T"]
        sizes = {"OYOXKBT": plane * d["K"], "OYOXCBT": plane * d["C"], "KT": d["K"] * d["T"], "CT": d["C"] * d["T"]}
        if f.process_key == "with_opt":
            # Adam's update model carries a scale and a shift vector of K elements each beside the FX weight elements
            sizes["P"] = (2 if f.op_name in ("adam", "adamw") else 1) * d["K"] + d["FX"] * d["FY"] * d["C"]
        return sizes

    def _extra_counts(self, f: _Fragment) -> Dict[str, int]:
        c = {"mux": 0, "add": 0, "mul": 0, "comp": 0, "sqrt": 0}
        n = self._sizes(f)
        if f.process_key == "with_sg":
            if f.phase == "forward":          # integrate, compare with threshold, reset select, spike mask
                c.update(mux=n["OYOXKBT"], add=n["OYOXKBT"], mul=n["OYOXKBT"], comp=3 * n["OYOXKBT"])
            else:                              # surrogate gradient and the recurrence of the potential gradient
                c.update(mux=n["OYOXCBT"], add=2 * n["OYOXCBT"], mul=4 * n["OYOXCBT"])
        elif f.process_key == "with_bn":
            if f.phase == "forward":
                c.update(add=3 * n["OYOXKBT"] + 2 * n["KT"], mul=3 * n["OYOXKBT"] + 4 * n["KT"], sqrt=n["KT"])
            elif f.conv_type != "without_bp_bn":
                c.update(add=7 * n["OYOXCBT"], mul=3 * n["OYOXCBT"] + 22 * n["CT"])
        elif f.process_key == "with_opt":
            P = n["P"]
            if f.op_name in ("adam", "adamw"):
                c.update(add=4 * P, mul=11 * P, sqrt=P)
            else:
                extra = int(f.optimizer.get("weight_decay", False)) + int(f.optimizer.get("momentum", False) and f.optimizer.get("momentum_buffer", False))
                c.update(add=P * (1 + extra), mul=P * (1 + extra))
        return c

    def _extra_memory(self, f: _Fragment):
        bits, energy = defaultdict(lambda: defaultdict(int)), defaultdict(lambda: defaultdict(float))
        if f.process_key == "with_nothing":
            return bits, energy
        inst, n = self.memory_config.memory_instances, self._sizes(f)
        if f.process_key == "with_opt" and f.op_name == "sgd":
            total, spec = n["P"] * 32, inst["sram_6MB"]
            reads = 2 + int(f.optimizer.get("momentum", False) and f.optimizer.get("momentum_buffer", False))     # parameter, gradient, buffer
            writes = 1 + int(f.optimizer.get("momentum", False))
            for _ in range(reads):
                self._charge(bits, energy, "sram", "rh2l", total, spec, 32, True)
            for _ in range(writes):
                self._charge(bits, energy, "sram", "wl2h", total, spec, 32, False)
            return bits, energy
        for size_key, word, reg, sram in _EXTRA_VARIABLES.get((f.process_key, f.phase), {}).values():
            total = n[size_key] * word
            # every intermediate is written to its SRAM once and read back once (the register file is charged for the
            # contraction operands only)
            for direction, read in (("wl2h", False), ("rh2l", True)):
                self._charge(bits, energy, "sram", direction, total, inst[sram], word, read)
        return bits, energy

    def _unsupported_ops(self) -> List[str]:
        return sorted(self._outside)

    def get_report(self) -> NeuroMCRuntimeEnergyReport:
        if self.strict and self._outside:
            raise RuntimeError(f"NeuroMC has no core for these operators: {self._unsupported_ops()}")
        rep = NeuroMCRuntimeEnergyReport()
        rep.warnings = [f"no NeuroMC core for {op} ({n} call{'s' if n > 1 else ''}); its energy is not included" for op, n in sorted(self._outside.items())]
        by_stage, by_op, by_core, by_key = (defaultdict(float) for _ in range(4))
        level_dir = defaultdict(lambda: defaultdict(float))
        bits_level = defaultdict(lambda: defaultdict(int))
        counts_core, counts_key = defaultdict(lambda: defaultdict(int)), defaultdict(lambda: defaultdict(int))
        prim = defaultdict(int)
        prim_stage, prim_op = defaultdict(lambda: defaultdict(int)), defaultdict(lambda: defaultdict(int))
        for f in self._fragments:
            mac_e = f.mac_count * MAC_COST_PJ.get(f.core_type, 0.0)
            extra = self._extra_counts(f)
            extra_e = sum(extra[k] * OP_COST_PJ[k] for k in extra)
            base_bits, base_en = self._base_memory(f)
            more_bits, more_en = self._extra_memory(f)
            base_e = sum(v for d in base_en.values() for v in d.values())
            more_e = sum(v for d in more_en.values() for v in d.values())
            total = mac_e + extra_e + base_e + more_e
            rep.energy_mac_pj += mac_e
            rep.energy_extra_compute_pj += extra_e
            rep.energy_base_memory_pj += base_e
            rep.energy_extra_memory_pj += more_e
            by_stage[f.stage] += total
            by_op[f.op_name] += total
            by_core[f.core_type] += total
            by_key[f.process_key] += total
            for src_bits, src_en in ((base_bits, base_en), (more_bits, more_en)):
                for level, dirs in src_en.items():
                    for direction, e in dirs.items():
                        level_dir[level][direction] += e
                        bits_level[level][direction] += src_bits[level][direction]
            prim["mac"] += f.mac_count
            for table, key in ((counts_core, f.core_type), (counts_key, f.process_key)):
                table[key]["fragments"] += 1
                table[key]["mac"] += f.mac_count
            for k, v in extra.items():
                prim[k] += v
                prim_stage[f.stage][k] += v
                prim_op[f.op_name][k] += v
                counts_core[f.core_type][k] += v
                counts_key[f.process_key][k] += v
            rep.mapping_summary.append({
                "stage": f.stage, "phase": f.phase, "op_name": f.op_name, "core_type": f.core_type, "process_key": f.process_key,
                "input_precision_bits": f.bits[0], "weight_precision_bits": f.bits[1], "output_precision_bits": f.bits[2],
                "loop_dims": dict(f.loop_dims), "b_type": f.b_type, "t_type": f.t_type, "mac_count": f.mac_count, "source": f.source,
                "optimizer_has_momentum": bool(f.optimizer.get("momentum", False)),
                "optimizer_has_weight_decay": bool(f.optimizer.get("weight_decay", False)),
                "optimizer_has_momentum_buffer": bool(f.optimizer.get("momentum_buffer", False)), "energy_pj": total})
        rep.energy_compute_pj = rep.energy_mac_pj + rep.energy_extra_compute_pj
        rep.energy_memory_pj = rep.energy_base_memory_pj + rep.energy_extra_memory_pj
        rep.energy_total_pj = rep.energy_compute_pj + rep.energy_memory_pj
        rep.energy_by_stage, rep.energy_by_op = dict(by_stage), dict(by_op)
        rep.energy_by_core_type, rep.energy_by_process_key = dict(by_core), dict(by_key)
        rep.energy_by_memory_level_dir = {k: dict(v) for k, v in level_dir.items()}
        rep.memory_bits_by_level = {"preset_name": self.memory_config.preset_name,
                                    "totals": {level: int(sum(d.values())) for level, d in bits_level.items()},
                                    "by_level_dir": {k: dict(v) for k, v in bits_level.items()}}
        rep.primitive_counts = {"totals": {k: int(prim[k]) for k in ("mux", "add", "mul", "comp", "sqrt", "mac")},
                                "by_stage": {k: dict(v) for k, v in prim_stage.items()}, "by_op": {k: dict(v) for k, v in prim_op.items()},
                                "core_type": self.core_type}
        rep.counts_by_core_type = {k: dict(v) for k, v in counts_core.items()}
        rep.counts_by_process_key = {k: dict(v) for k, v in counts_key.items()}
        return rep

    def get_total(self) -> float:
        return self.get_report().energy_total_pj

    def get_counts(self) -> Dict[str, Any]:
        rep = self.get_report()
        return {"primitive_counts": rep.primitive_counts, "counts_by_core_type": rep.counts_by_core_type,
                "counts_by_process_key": rep.counts_by_process_key, "fragments": len(self._fragments)}


def estimate_neuromc_runtime_energy(model: nn.Module, inputs, *, target: Optional[torch.Tensor] = None, loss_fn: Optional[Callable] = None,
                                    optimizer=None, core_type: str = "fp_soma", memory_config: Optional[MemoryHierarchyConfig] = None,
                                    strict: bool = False, extra_ignore_modules: Optional[list] = None) -> NeuroMCRuntimeEnergyReport:
    """One forward (and, with ``loss_fn`` and ``target``, backward and optimizer) step of ``model`` on ``inputs`` under the
    profiler; the loss itself and ``optimizer.step()`` run unobserved (the update is modelled, not traced)."""
    if optimizer is not None and loss_fn is None:
        raise ValueError("Exact NeuroMC optimizer modeling requires loss_fn and target; optimizer.step() without backward is unsupported.")
    if loss_fn is not None and target is None:
        raise ValueError("target is required when loss_fn is provided")
    prof = NeuroMCEnergyProfiler(core_type=core_type, memory_config=memory_config, strict=strict, extra_ignore_modules=extra_ignore_modules)
    prof.bind_model(model)
    prof.bind_optimizer(optimizer)
    for p in model.parameters():
        p.grad = None
    with prof:
        with prof.stage("forward"):
            out = call_model(model, inputs)
        if loss_fn is not None:
            with prof.suspend():
                loss = loss_fn(out, target)
            with prof.stage("backward"):
                loss.backward()
            if optimizer is not None:
                with prof.stage("optimizer"):
                    prof.record_optimizer_step("optimizer")
                    with prof.suspend():
                        optimizer.step()
                        optimizer.zero_grad(set_to_none=True)
        report = prof.get_report()
    return report
