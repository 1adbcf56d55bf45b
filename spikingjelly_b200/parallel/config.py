"""``SNNDistributedConfig``: the eager configuration of a distributed run (mode, mesh, roots).
Parity: ``spikingjelly/activation_based/distributed/config.py:12-114``."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Sequence, Tuple, Union

import torch

__all__ = ["SNNDistributedConfig", "VALID_MODES"]

VALID_MODES = ("none", "dp", "tp", "fsdp2", "fsdp2_tp")


@dataclass
class SNNDistributedConfig:
    """``mode``: ``none | dp | tp | fsdp2 | fsdp2_tp``.  ``mesh_shape`` / ``device_mesh`` describe the
    rank grid, ``tp_mesh_dim`` / ``dp_mesh_dim`` which of its axes carry tensor / data parallelism.
    ``tensor_parallel_roots`` restricts where linear layers are sharded; ``tensor_parallel_plan`` maps
    module paths to styles (``colwise``, ``colwise_local_output``, ``rowwise``) explicitly.
    ``conv_tensor_parallel_roots`` / ``spikformer_*_roots`` enable channel sharding of convolution
    stacks and Spikformer blocks.  The ``fsdp_*`` fields are passed to FSDP2."""
    mode: str = "none"
    device_type: str = "cuda"
    mesh_shape: Optional[Tuple[int, ...]] = None
    device_mesh: Optional[Any] = None
    tp_mesh_dim: int = 0
    dp_mesh_dim: Optional[int] = None
    tensor_parallel_roots: Optional[Sequence[str]] = None
    tensor_parallel_plan: Optional[Mapping[str, Union[str, Any]]] = None
    auto_tensor_parallel: bool = True
    conv_tensor_parallel_roots: Optional[Sequence[str]] = None
    spikformer_tensor_parallel_roots: Optional[Sequence[str]] = None
    spikformer_patch_stem_tensor_parallel_roots: Optional[Sequence[str]] = None
    broadcast_buffers: bool = False
    find_unused_parameters: bool = False
    static_graph: bool = False
    fsdp_shard_roots: Optional[Sequence[str]] = None
    fsdp_shard_module_root: bool = True
    fsdp_root_reshard_after_forward: bool = False
    fsdp_param_dtype: Optional[torch.dtype] = None
    fsdp_reduce_dtype: Optional[torch.dtype] = None
    fsdp_output_dtype: Optional[torch.dtype] = None

    def __post_init__(self) -> None:
        self.mode = self.mode.lower()
        if self.mode not in VALID_MODES:
            raise ValueError(f"Unsupported mode={self.mode!r}; expected one of {VALID_MODES}.")
