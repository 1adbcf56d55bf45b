"""Model-family adapters: which roots get tensor parallelism / FSDP2 for a known architecture.
Parity: ``spikingjelly/activation_based/distributed/adapters/{__init__,base,spikformer,cifar10dvs_vgg}.py``."""
from __future__ import annotations

from typing import Dict, Optional, Protocol, runtime_checkable

import torch.nn as nn

from .analysis import SNNDistributedAnalysis, analyze_snn_distributed_capability
from .config import SNNDistributedConfig
from .execution import configure_snn_distributed
from .planner import SNNDistributedPlan
from .runtime import SNNDistributedRuntime

__all__ = ["SNNDistributedAdapter", "SpikformerAdapter", "CIFAR10DVSVGGAdapter", "build_distributed_runtime", "get_adapter",
           "infer_model_family", "list_adapters", "resolve_adapter"]


def build_distributed_runtime(model: nn.Module, plan: SNNDistributedPlan, *, device_type: str = "cuda", device_mesh=None,
                              **config_overrides) -> SNNDistributedRuntime:
    if plan.mode == "pp":
        raise ValueError("Pipeline plans require the pipeline-specific runtime builder, not build_distributed_runtime().")
    kw = dict(mode=plan.mode, device_type=device_type, mesh_shape=plan.mesh_shape, device_mesh=device_mesh, tp_mesh_dim=plan.tp_mesh_dim,
              dp_mesh_dim=plan.dp_mesh_dim, tensor_parallel_plan=plan.tensor_parallel_plan,
              auto_tensor_parallel=plan.mode in ("tp", "fsdp2_tp") and plan.tensor_parallel_plan is None)
    kw.update(config_overrides)
    configured, mesh, analysis = configure_snn_distributed(model, SNNDistributedConfig(**kw))
    return SNNDistributedRuntime(model=configured, mesh=mesh, analysis=analysis, plan=plan)


@runtime_checkable
class SNNDistributedAdapter(Protocol):
    name: str

    def analyze(self, model: nn.Module) -> SNNDistributedAnalysis: ...

    def apply(self, model: nn.Module, plan: SNNDistributedPlan, *, device_type: str = "cuda", device_mesh=None) -> SNNDistributedRuntime: ...


class SpikformerAdapter:
    """Head tensor-parallel by default; blocks and patch stem when the plan's feature set allows it;
    FSDP2 wraps the patch stem and every block separately."""
    name = "spikformer"

    def analyze(self, model):
        return analyze_snn_distributed_capability(model, tensor_parallel_roots=["head"])

    def apply(self, model, plan, *, device_type="cuda", device_mesh=None):
        tp = plan.mode in ("tp", "fsdp2_tp")
        blocks_tp = tp and plan.experimental_features.allow_experimental_spikformer_tp
        block_roots = ("patch_embed",) + tuple(f"blocks.{i}" for i in range(len(model.blocks)))
        fsdp_roots, shard_root = None, True
        if plan.mode == "fsdp2":
            fsdp_roots = block_roots + ("head",)
        elif plan.mode == "fsdp2_tp":
            fsdp_roots, shard_root = block_roots, False
        return build_distributed_runtime(model, plan, device_type=device_type, device_mesh=device_mesh,
                                         tensor_parallel_roots=("head",) if tp else None,
                                         spikformer_tensor_parallel_roots=("blocks",) if blocks_tp else None,
                                         spikformer_patch_stem_tensor_parallel_roots=("patch_embed",) if blocks_tp else None,
                                         fsdp_shard_roots=fsdp_roots, fsdp_shard_module_root=shard_root)


class CIFAR10DVSVGGAdapter:
    """Classifier tensor-parallel; feature convolutions channel-sharded when allowed."""
    name = "cifar10dvs_vgg"

    def analyze(self, model):
        return analyze_snn_distributed_capability(model, tensor_parallel_roots=["classifier"])

    def apply(self, model, plan, *, device_type="cuda", device_mesh=None):
        tp = plan.mode in ("tp", "fsdp2_tp")
        roots = tuple(plan.tensor_parallel_roots) if plan.tensor_parallel_roots is not None else ("classifier",)
        fsdp_roots, shard_root = None, True
        if plan.mode == "fsdp2":
            fsdp_roots = ("features", "classifier")
        elif plan.mode == "fsdp2_tp":
            fsdp_roots, shard_root = ("features",), False
        return build_distributed_runtime(model, plan, device_type=device_type, device_mesh=device_mesh,
                                         tensor_parallel_roots=roots if tp else None,
                                         conv_tensor_parallel_roots=("features",) if tp and plan.experimental_features.allow_experimental_conv_tp else None,
                                         fsdp_shard_roots=fsdp_roots, fsdp_shard_module_root=shard_root)


_REGISTRY: Dict[str, SNNDistributedAdapter] = {"cifar10dvs_vgg": CIFAR10DVSVGGAdapter(), "spikformer": SpikformerAdapter()}
_PATTERNS = {"spikformer": "spikformer", "cifar10dvsvgg": "cifar10dvs_vgg"}


def infer_model_family(model: nn.Module) -> Optional[str]:
    inner = getattr(model, "module", None)
    name = type(inner if isinstance(inner, nn.Module) else model).__name__.lower()
    return next((family for pattern, family in _PATTERNS.items() if pattern in name), None)


def get_adapter(name: str) -> SNNDistributedAdapter:
    if name not in _REGISTRY:
        raise KeyError(f"Unknown distributed adapter '{name}'.")
    return _REGISTRY[name]


def resolve_adapter(model, model_family: Optional[str] = None) -> Optional[SNNDistributedAdapter]:
    family = (model_family if model_family != "generic" else None) or infer_model_family(model)
    return None if family is None else _REGISTRY.get(family)


def list_adapters():
    return tuple(sorted(_REGISTRY))
