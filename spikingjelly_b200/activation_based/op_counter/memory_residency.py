"""Where operands live: a three-level inclusive memory hierarchy (register file inside SRAM inside DRAM) with LRU
replacement, driven by the tensors each ATen operator reads and writes.  It reports the bits read / written at every
level and the bits moved along every edge (``dram->sram``, ``sram->reg``, ``reg->sram``, ...), per operator too.

Rules of the model (``op_counter/memory_residency.py:147-459`` of the reference):

* a tensor is identified by device, dtype and storage address, so views share residency;
* a read brings the tensor as close to the compute as it fits (DRAM -> SRAM -> registers), charging a read at each level
  it passes and a write at each level it lands in; a tensor larger than a level skips that level;
* a write lands in the register file if it fits, else in SRAM, else in DRAM, without reading anything;
* eviction is LRU; a line evicted from registers goes to SRAM if SRAM can take it, else to DRAM; a line evicted from SRAM
  takes its register copy with it (inclusion).  Evictions are charged as a read at the source and a write at the target.
Default capacities: 256 KiB of registers, 38 MiB of SRAM.
"""
from __future__ import annotations

from collections import OrderedDict, defaultdict
from typing import Any, Callable, Dict, List, Optional

import torch
import torch.nn as nn
from torch.overrides import resolve_name

from .base import BaseCounter, _collect_tensors, _tensor_bits

aten = torch.ops.aten

__all__ = ["MemoryResidencySimulator", "MemoryResidencyCounter", "_access_convolution_backward"]

_DEFAULT_CAPACITY_BITS = {"reg": float(256 * 1024 * 8), "sram": float(38 * 1024 * 1024 * 8), "dram": float("inf")}


# ---- which tensors an operator reads / writes -----------------------------------------------------
def _tensors(xs) -> List[torch.Tensor]:
    return [x for x in xs if torch.is_tensor(x)]


def _access_matmul(args, kwargs, out):
    return list(args[:2]), [out]


def _access_add_matmul(args, kwargs, out):
    bias, x, y = args[:3]
    return ([x, y, bias] if kwargs.get("beta", 1.0) != 0 else [x, y]), [out]


def _access_convolution(args, kwargs, out):
    x, w, bias = args[:3]
    return ([x, w] if bias is None else [x, w, bias]), [out]


def _access_convolution_backward(args, kwargs, out):
    grad_out, x, w = args[0], args[1], args[2]
    mask = args[-1]
    if not isinstance(out, (tuple, list)) or len(out) < 3:
        return [grad_out], _collect_tensors(out)
    reads = [grad_out] + ([w] if mask[0] else []) + ([x] if mask[1] else [])
    return reads, [o for o, m in zip(out[:3], mask[:3]) if m and torch.is_tensor(o)]


def _access_native_batch_norm(args, kwargs, out):
    reads = [args[0]] + _tensors(args[1:5])
    return reads, ([out[0], out[1], out[2]] if args[5] else [out[0]])


def _access_native_batch_norm_backward(args, kwargs, out):
    return _tensors(args[:7]), _collect_tensors(out)


def _access_binary(args, kwargs, out):
    return _tensors(args[:2]), [out]


def _access_unary(args, kwargs, out):
    return [args[0]], [out]


def _access_where(args, kwargs, out):
    return list(args[:3]), [out]


_RESIDENCY_ACCESS_RULES: Dict[Any, Callable] = {
    aten.mm.default: _access_matmul, aten.bmm.default: _access_matmul,
    aten.addmm.default: _access_add_matmul, aten.baddbmm.default: _access_add_matmul,
    aten.convolution.default: _access_convolution, aten.convolution_backward.default: _access_convolution_backward,
    aten.native_batch_norm.default: _access_native_batch_norm,
    aten.native_batch_norm_backward.default: _access_native_batch_norm_backward,
    aten.sqrt.default: _access_unary, aten.sqrt_.default: _access_unary, aten.rsqrt.default: _access_unary,
    aten.sum.default: _access_unary, aten.sum.dim_IntList: _access_unary, aten.mean.dim: _access_unary,
    aten.where.self: _access_where, aten.where.ScalarOther: _access_where, aten.where.ScalarSelf: _access_where,
}
for _name in ("add", "add_", "sub", "sub_", "mul", "mul_", "div", "div_"):
    for _ov in ("Tensor", "Scalar"):
        _RESIDENCY_ACCESS_RULES[getattr(getattr(aten, _name), _ov)] = _access_binary
_RESIDENCY_ACCESS_RULES[aten.rsub.Tensor] = _access_binary
_RESIDENCY_ACCESS_RULES[aten.rsub.Scalar] = _access_binary


def _rw() -> Dict[str, int]:
    return {"read_bits": 0, "write_bits": 0, "total_bits": 0}


class MemoryResidencySimulator:
    def __init__(self, config: Any = None, *, capacity_bits: Optional[Dict[str, float]] = None):
        if capacity_bits is None:
            capacity_bits = getattr(config, "capacity_bits", None) if config is not None else None
            if capacity_bits is None:
                capacity_bits = dict(_DEFAULT_CAPACITY_BITS)
        self.capacity_bits = {lv: float(capacity_bits.get(lv, float("inf"))) for lv in ("reg", "sram", "dram")}
        self.reg_cache: "OrderedDict[str, int]" = OrderedDict()
        self.sram_cache: "OrderedDict[str, int]" = OrderedDict()
        self.reset()

    def reset(self):
        self.reg_cache.clear()
        self.sram_cache.clear()
        self.usage_bits = {"reg": 0, "sram": 0}
        self.level_rw_bits = defaultdict(_rw)
        self.op_level_rw_bits = defaultdict(lambda: defaultdict(_rw))
        self.move_bits_by_edge = defaultdict(int)
        self.move_bits_by_op = defaultdict(lambda: defaultdict(int))

    # ---- bookkeeping
    def _charge(self, level: str, rw: str, bits: int, op: str):
        if bits > 0:
            for table in (self.level_rw_bits[level], self.op_level_rw_bits[op][level]):
                table[rw] += bits
                table["total_bits"] += bits

    def _move(self, src: str, dst: str, bits: int, op: str):
        if bits > 0:
            self.move_bits_by_edge[f"{src}->{dst}"] += bits
            self.move_bits_by_op[op][f"{src}->{dst}"] += bits
            self._charge(dst, "write_bits", bits, op)

    def _drop_reg_copy(self, key: str, op: str):
        bits = self.reg_cache.pop(key, None)
        if bits is not None:
            self.usage_bits["reg"] -= bits
            self._charge("reg", "read_bits", bits, op)
            self._move("reg", "dram", bits, op)

    def _make_room(self, level: str, bits: int, op: str):
        cache = self.reg_cache if level == "reg" else self.sram_cache
        while cache and self.usage_bits[level] + bits > self.capacity_bits[level]:
            victim, vbits = cache.popitem(last=False)
            self.usage_bits[level] -= vbits
            self._charge(level, "read_bits", vbits, op)
            if level == "reg":
                self._move("reg", "sram" if self._insert("sram", victim, vbits, op) else "dram", vbits, op)
            else:
                self._move("sram", "dram", vbits, op)
                self._drop_reg_copy(victim, op)

    def _insert(self, level: str, key: str, bits: int, op: str) -> bool:
        cache = self.reg_cache if level == "reg" else self.sram_cache
        if bits > self.capacity_bits[level]:
            return False
        grown = key in cache
        if grown:
            if bits <= cache[key]:
                cache.move_to_end(key)
                return True
            self.usage_bits[level] -= cache.pop(key)
            if level == "sram":
                self._drop_reg_copy(key, op)
        self._make_room(level, bits, op)
        if self.usage_bits[level] + bits > self.capacity_bits[level]:
            return False
        cache[key] = bits
        self.usage_bits[level] += bits
        return True

    def _touch_inclusive_levels(self, key: str):
        for cache in (self.reg_cache, self.sram_cache):
            if key in cache:
                cache.move_to_end(key)

    def _tensor_key(self, tensor: torch.Tensor) -> str:
        storage = tensor.untyped_storage()
        ptr = int(storage.data_ptr())
        return f"{tensor.device}:{tensor.dtype}:" + (f"id={id(storage)}" if ptr == 0 else f"ptr={ptr}")

    # ---- events
    def on_tensor_read(self, tensor: torch.Tensor, op_name: str):
        bits = _tensor_bits(tensor)
        if bits <= 0:
            return
        key = self._tensor_key(tensor)
        if key in self.reg_cache:
            self._touch_inclusive_levels(key)
            return self._charge("reg", "read_bits", bits, op_name)
        in_sram = key in self.sram_cache
        if in_sram:
            self.sram_cache.move_to_end(key)
        elif self._insert("sram", key, bits, op_name):
            self._charge("dram", "read_bits", bits, op_name)
            self._move("dram", "sram", bits, op_name)
            in_sram = True
        if in_sram:
            self._charge("sram", "read_bits", bits, op_name) if not self._insert("reg", key, bits, op_name) else self._sram_to_reg(bits, op_name, "read_bits")
            return
        if self._insert("reg", key, bits, op_name):                    # too large for SRAM but fits the register file
            self._charge("dram", "read_bits", bits, op_name)
            self._move("dram", "reg", bits, op_name)
            return self._charge("reg", "read_bits", bits, op_name)
        self._charge("dram", "read_bits", bits, op_name)

    def _sram_to_reg(self, bits: int, op: str, final: str):
        self._charge("sram", "read_bits", bits, op)
        self._move("sram", "reg", bits, op)
        self._charge("reg", final, bits, op)

    def on_tensor_write(self, tensor: torch.Tensor, op_name: str):
        bits = _tensor_bits(tensor)
        if bits <= 0:
            return
        key = self._tensor_key(tensor)
        if key in self.reg_cache:
            self._touch_inclusive_levels(key)
            return self._charge("reg", "write_bits", bits, op_name)
        if key in self.sram_cache:
            self.sram_cache.move_to_end(key)
            if self._insert("reg", key, bits, op_name):
                return self._sram_to_reg(bits, op_name, "write_bits")
            return self._charge("sram", "write_bits", bits, op_name)
        for level in ("reg", "sram"):
            if self._insert(level, key, bits, op_name):
                return self._charge(level, "write_bits", bits, op_name)
        self._charge("dram", "write_bits", bits, op_name)

    # ---- results
    def get_level_rw_bits(self):
        return {k: dict(v) for k, v in self.level_rw_bits.items()}

    def get_op_level_rw_bits(self):
        return {op: {lv: dict(info) for lv, info in d.items()} for op, d in self.op_level_rw_bits.items()}

    def get_move_bits_by_edge(self):
        return dict(self.move_bits_by_edge)

    def get_move_bits_by_op(self):
        return {op: dict(d) for op, d in self.move_bits_by_op.items()}


class MemoryResidencyCounter(BaseCounter):
    """Feeds every counted operator's reads and writes to a :class:`MemoryResidencySimulator`; the counter's own value is
    the number of bits the operator touches."""

    def __init__(self, *, config: Any = None, capacity_bits: Optional[Dict[str, float]] = None,
                 extra_rules: Optional[Dict[Any, Callable]] = None, extra_ignore_modules: Optional[List[type]] = None):
        super().__init__()
        self.rules = dict(_RESIDENCY_ACCESS_RULES)
        self.rules.update(extra_rules or {})
        self.ignore_modules = list(extra_ignore_modules or [])
        self.simulator = MemoryResidencySimulator(config, capacity_bits=capacity_bits)

    def reset(self):
        self.records.clear()
        self.simulator.reset()

    def count(self, func, args, kwargs, out, active_modules=None, parent_names=None) -> int:
        rule = self.rules.get(func)
        if rule is None:
            return 0
        op = resolve_name(func)
        reads, writes = rule(args, kwargs, out)
        for t in reads:
            self.simulator.on_tensor_read(t, op)
        for t in writes:
            self.simulator.on_tensor_write(t, op)
        return sum(_tensor_bits(t) for t in (*reads, *writes))

    def get_level_bits(self) -> Dict[str, int]:
        return {lv: v["total_bits"] for lv, v in self.simulator.get_level_rw_bits().items()}

    def get_level_rw_bits(self):
        return self.simulator.get_level_rw_bits()

    def get_op_level_bits(self):
        return {op: {lv: v["total_bits"] for lv, v in levels.items()} for op, levels in self.simulator.get_op_level_rw_bits().items()}

    def get_move_bits_by_edge(self):
        return self.simulator.get_move_bits_by_edge()

    def get_move_bits_by_op(self):
        return self.simulator.get_move_bits_by_op()
