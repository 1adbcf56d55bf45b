"""The fp8 policy of this package: every convertible linear map (step-mode ``Linear``, ``nn.Linear``,
1x1 ``Conv1d``; optionally ``LayerNorm -> Linear`` and ``LayerNorm -> Linear -> GELU -> Linear``
blocks as one module) runs its three matrix products on the e4m3 / e5m2 tensor-core kernel of
``ops/fp8.py``; everything else runs under bf16 autocast.  Two per-tensor scaling recipes: ``"delayed"`` (the
default behind ``"auto"``: each tensor is scaled by the maximum its role showed in the previous call and read once)
and ``"current"`` (scaled by its own maximum, read twice).  ``"block"`` and ``"mxfp8"`` are accepted names that
resolve to ``"delayed"``: block-scaled operands are not implemented, and the capability report says so.

Parameters stay in their original dtype and under their original names, so optimisers and
checkpoints are unaffected by the conversion.

``Float8TorchAOPolicy`` (mode ``"fp8-torchao"``) and ``Float8TransformerEnginePolicy`` (``"fp8-te"``)
are the names the reference gives to its two vendor-library policies
(``spikingjelly/activation_based/precision/float8_torchao.py:76-146``, ``float8_te.py:424-595``); here
they are the same native policy (the second one also fuses the LayerNorm patterns, as TE does).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import layer
from .float8_base import _Float8StepModule, wrap_float8_linear_module
from .float8_conv import is_supported_pointwise_conv1d, make_linear_from_pointwise_conv1d, wrap_float8_pointwise_conv1d_module
from .policy import PrecisionPolicy

__all__ = ["Float8Linear", "Float8LayerNormLinear", "Float8LayerNormMLP", "Float8NativePolicy", "Float8TorchAOPolicy",
           "Float8TransformerEnginePolicy", "Float8TELayerNormLinearModule", "Float8TELayerNormMLPModule"]

_SUPPORTED_RECIPES = {"auto", "delayed", "current", "block", "mxfp8"}


def _fp8_linear(x, weight, bias, scaling=None):
    from ...ops import fp8
    return fp8.linear(x, weight, bias, scaling)


class _RecipeMixin:
    """Scaling recipe of a converted module: ``n`` products, each with its own delayed-scaling state (kept outside
    the state dict: it is rebuilt from the first call after a resume)."""
    _n_products = 1

    def set_recipe(self, recipe: str) -> None:
        from ...ops import fp8
        if recipe not in ("current", "delayed"):
            raise ValueError(f"recipe must be 'current' or 'delayed', got {recipe!r}")
        self.__dict__["fp8_recipe"] = recipe
        self.__dict__["_scalings"] = [fp8.LinearScaling(delayed=recipe == "delayed") for _ in range(self._n_products)]

    def _scaling(self, i: int = 0):
        sc = self.__dict__.get("_scalings")
        return None if sc is None else sc[i]


class Float8Linear(_RecipeMixin, nn.Linear):
    """``nn.Linear`` whose products run in fp8 (same parameters, same state dict)."""

    @classmethod
    def from_float(cls, source: nn.Linear) -> "Float8Linear":
        new = cls.__new__(cls)
        nn.Module.__init__(new)
        new.in_features, new.out_features = source.in_features, source.out_features
        new.weight = source.weight
        new.bias = source.bias
        return new

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _fp8_linear(x, self.weight, self.bias, self._scaling())


class Float8LayerNormLinear(_RecipeMixin, nn.Module):
    """``Linear(LayerNorm(x))`` with the product in fp8."""

    def __init__(self, norm: nn.LayerNorm, linear: nn.Linear):
        super().__init__()
        self.eps, self.normalized_shape = norm.eps, tuple(norm.normalized_shape)
        self.layer_norm_weight, self.layer_norm_bias = norm.weight, norm.bias
        self.weight, self.bias = linear.weight, linear.bias

    def forward(self, x):
        return _fp8_linear(F.layer_norm(x, self.normalized_shape, self.layer_norm_weight, self.layer_norm_bias, self.eps),
                           self.weight, self.bias, self._scaling())


class Float8LayerNormMLP(_RecipeMixin, nn.Module):
    """``fc2(GELU(fc1(LayerNorm(x))))`` with both products in fp8."""
    _n_products = 2

    def __init__(self, norm: nn.LayerNorm, fc1: nn.Linear, fc2: nn.Linear):
        super().__init__()
        self.eps, self.normalized_shape = norm.eps, tuple(norm.normalized_shape)
        self.layer_norm_weight, self.layer_norm_bias = norm.weight, norm.bias
        self.fc1_weight, self.fc1_bias = fc1.weight, fc1.bias
        self.fc2_weight, self.fc2_bias = fc2.weight, fc2.bias

    def forward(self, x):
        h = F.layer_norm(x, self.normalized_shape, self.layer_norm_weight, self.layer_norm_bias, self.eps)
        return _fp8_linear(F.gelu(_fp8_linear(h, self.fc1_weight, self.fc1_bias, self._scaling(0))), self.fc2_weight, self.fc2_bias,
                           self._scaling(1))


class _PatternModule(_Float8StepModule):
    """Wrapper of a fused block that keeps the *original* ``nn.Sequential`` state-dict keys
    (``0.weight``, ``1.weight`` ...) through ``state_key_map``: public key -> attribute of ``wrapped``."""

    def __init__(self, wrapped: nn.Module, state_key_map: Dict[str, str], step_mode: str = "s"):
        super().__init__(wrapped, step_mode)
        self._state_key_map = state_key_map

    def forward(self, x):
        out = self.wrapped(x)
        return out[0] if isinstance(out, tuple) else out

    def state_dict(self, *args, destination=None, prefix="", keep_vars=False):
        destination = {} if destination is None else destination
        inner = self.wrapped.state_dict(keep_vars=keep_vars)
        mapped = set(self._state_key_map.values())
        for public, key in self._state_key_map.items():
            if key in inner:
                destination[prefix + public] = inner[key]
        for key, value in inner.items():
            if key not in mapped:
                destination[prefix + "wrapped." + key] = value
        return destination

    def _save_to_state_dict(self, destination, prefix, keep_vars):
        self.state_dict(destination=destination, prefix=prefix, keep_vars=keep_vars)

    def _load_from_state_dict(self, state_dict, prefix, *rest):
        for public, key in self._state_key_map.items():
            if prefix + public in state_dict:
                state_dict[prefix + "wrapped." + key] = state_dict.pop(prefix + public)


class Float8TELayerNormLinearModule(_PatternModule):
    pass


class Float8TELayerNormMLPModule(_PatternModule):
    pass


def _affine_ln(m) -> bool:
    return (isinstance(m, nn.LayerNorm) and m.elementwise_affine and m.weight is not None and m.bias is not None
            and len(tuple(m.normalized_shape)) == 1)


def _fuse_pattern(module: nn.Module):
    """``nn.Sequential(LayerNorm, Linear)`` or ``nn.Sequential(LayerNorm, Linear, GELU(exact), Linear)``."""
    if not isinstance(module, nn.Sequential):
        return None
    ch = list(module.children())
    lin = (nn.Linear, layer.Linear)
    if len(ch) == 4 and _affine_ln(ch[0]) and isinstance(ch[1], lin) and isinstance(ch[2], nn.GELU) \
            and getattr(ch[2], "approximate", "none") in (None, "none") and isinstance(ch[3], lin):
        h = int(ch[0].normalized_shape[0])
        if ch[1].in_features == h and ch[3].in_features == ch[1].out_features and ch[3].out_features == h \
                and (ch[1].bias is None) == (ch[3].bias is None):
            keys = {"0.weight": "layer_norm_weight", "0.bias": "layer_norm_bias", "1.weight": "fc1_weight", "1.bias": "fc1_bias",
                    "3.weight": "fc2_weight", "3.bias": "fc2_bias"}
            return Float8TELayerNormMLPModule(Float8LayerNormMLP(ch[0], ch[1], ch[3]), keys, getattr(ch[1], "step_mode", "s")), "LayerNormMLP"
    if len(ch) == 2 and _affine_ln(ch[0]) and isinstance(ch[1], lin) and ch[1].in_features == int(ch[0].normalized_shape[0]):
        keys = {"0.weight": "layer_norm_weight", "0.bias": "layer_norm_bias", "1.weight": "weight", "1.bias": "bias"}
        return Float8TELayerNormLinearModule(Float8LayerNormLinear(ch[0], ch[1]), keys, getattr(ch[1], "step_mode", "s")), "LayerNormLinear"
    return None


def _replace_child(parent: nn.Module, name: str, new: nn.Module) -> None:
    if isinstance(parent, nn.ModuleDict):
        parent[name] = new
    elif isinstance(parent, (nn.ModuleList, nn.Sequential)) and name.isdigit():
        parent[int(name)] = new
    else:
        setattr(parent, name, new)


def _convert_leaf(m: nn.Module) -> Optional[nn.Module]:
    if is_supported_pointwise_conv1d(m):
        return wrap_float8_pointwise_conv1d_module(m, Float8Linear.from_float(make_linear_from_pointwise_conv1d(m)))
    if isinstance(m, (nn.Linear, layer.Linear)) and not isinstance(m, Float8Linear):
        return wrap_float8_linear_module(m, Float8Linear.from_float(m))
    return None


class Float8NativePolicy(PrecisionPolicy):
    name = "fp8"
    fuse_layer_norm_patterns = False

    def __init__(self, device_type: str = "cuda", fp8_recipe: str = "auto"):
        super().__init__()
        self.device_type = device_type
        self.fp8_recipe = str(fp8_recipe or "auto").lower()
        self._resolved_recipe_name: Optional[str] = None

    def describe(self) -> dict:
        return {"name": self.name, "backend": "sjb200", "device_type": self.device_type, "fp8_recipe": self.fp8_recipe,
                "resolved_fp8_recipe": self._resolved_recipe_name, "autocast": True, "autocast_dtype": "torch.bfloat16",
                "grad_scaler": False}

    def check_capability(self, model, device) -> None:
        super().check_capability(model, device)
        report = self._capability
        report["te_recipe_requested"] = self.fp8_recipe
        if self.fp8_recipe not in _SUPPORTED_RECIPES:
            report["te_recipe_fallback_reason"] = f"unsupported fp8 recipe {self.fp8_recipe!r}"
            raise RuntimeError(f"Failed to resolve FP8 recipe: unsupported fp8 recipe {self.fp8_recipe!r}")
        # two per-tensor schemes: "current" recomputes every scale from the tensor itself, "delayed" takes it from
        # the previous call of the same role; the block-scaled names resolve to "delayed"
        self._resolved_recipe_name = "current" if self.fp8_recipe == "current" else "delayed"
        report["te_recipe_resolved"] = self._resolved_recipe_name
        if self.fp8_recipe in ("block", "mxfp8"):
            report["te_recipe_fallback_reason"] = f"recipe {self.fp8_recipe!r} is served by per-tensor delayed scaling"
        target = torch.device(device)
        if target.type == "cuda" and target.index is None and torch.cuda.is_available():
            target = torch.device("cuda", torch.cuda.current_device())
        devices = {p.device for p in model.parameters()}
        if devices and any(d != target for d in devices):
            raise RuntimeError(f"All model parameters must be moved to the target CUDA device '{target}' (e.g. model.to('{target}')) "
                               f"before calling prepare_model_for_precision() for {self.name!r}.")

    def autocast_context(self):
        return torch.amp.autocast(self.device_type, dtype=torch.bfloat16)

    def _convert_modules(self, model, report):
        out = self._convert_tree(model, report)
        recipe = self._resolved_recipe_name or ("current" if self.fp8_recipe == "current" else "delayed")
        for m in out.modules():
            if isinstance(m, _RecipeMixin):
                m.set_recipe(recipe)
        return out

    def _convert_tree(self, model, report):
        root = _convert_leaf(model)
        if root is not None:
            report.converted_modules.append("<root>")
            return root
        memo, visited = {}, set()

        def walk(parent, prefix):
            for name, child in list(parent._modules.items()):
                if child is None:
                    continue
                fqn = f"{prefix}.{name}" if prefix else name
                if child in memo:
                    _replace_child(parent, name, memo[child])
                    report.converted_modules.append(fqn)
                    continue
                fused = _fuse_pattern(child) if self.fuse_layer_norm_patterns else None
                if fused is not None:
                    memo[child] = fused[0]
                    _replace_child(parent, name, fused[0])
                    report.converted_modules.append(fqn)
                    report.converted_patterns.append({"module": fqn, "pattern": fused[1], "backend": "sjb200"})
                    continue
                new = _convert_leaf(child)
                if new is not None:
                    memo[child] = new
                    _replace_child(parent, name, new)
                    report.converted_modules.append(fqn)
                    continue
                if next(child.children(), None) is None:
                    report.skipped_modules.append(fqn)
                if id(child) not in visited:
                    visited.add(id(child))
                    walk(child, fqn)
        walk(model, "")
        return model


class Float8TorchAOPolicy(Float8NativePolicy):
    name = "fp8-torchao"


class Float8TransformerEnginePolicy(Float8NativePolicy):
    name = "fp8-te"
    supports_layer_norm_conversion = True
    fuse_layer_norm_patterns = True
