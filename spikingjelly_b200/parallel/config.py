"""``SNNDistributedConfig``: the explicit description of one distributed set-up (mode, mesh, which parts of the model get
which treatment).  Field names and defaults are those of ``spikingjelly/activation_based/distributed/config.py:12-62`` so
that configurations written for the reference construct unchanged; the axis checks that the reference keeps in its
execution module live here, next to the fields they concern."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Sequence, Tuple, Union

import torch

from . import _schema

__all__ = ["SNNDistributedConfig", "VALID_MODES"]

VALID_MODES = ("none", "dp", "tp", "fsdp2", "fsdp2_tp")


@dataclass
class SNNDistributedConfig:
    """``mode`` selects the parallelism (``none | dp | tp | fsdp2 | fsdp2_tp``).

    Mesh: either ``device_mesh`` (used as is) or ``mesh_shape`` (a mesh is created); ``tp_mesh_dim`` / ``dp_mesh_dim`` name the
    axes that carry tensor and data parallelism.  Tensor parallelism: ``tensor_parallel_plan`` maps module paths to a style
    (``colwise``, ``colwise_local_output``, ``rowwise``); without one, linear layers under ``tensor_parallel_roots`` are planned
    automatically (``auto_tensor_parallel``).  ``conv_tensor_parallel_roots`` and the two ``spikformer_*`` fields switch on
    channel sharding of convolution stacks / Spikformer blocks.  The ``fsdp_*`` fields go to FSDP2, the three booleans after
    them to the data-parallel wrapper."""
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
        self.mode = _schema.one_of(self.mode, VALID_MODES, "mode")

    # ------------------------------------------------------------------ what the mode implies
    @property
    def uses_tensor_parallel(self) -> bool:
        return self.mode in ("tp", "fsdp2_tp")

    @property
    def uses_fsdp(self) -> bool:
        return self.mode in ("fsdp2", "fsdp2_tp")

    @property
    def uses_data_parallel(self) -> bool:
        return self.mode == "dp"

    @property
    def shards_the_batch(self) -> bool:
        return self.mode in ("dp", "fsdp2", "fsdp2_tp")

    # ------------------------------------------------------------------ mesh axes
    def check_axes(self, ndim: int) -> None:
        """Raise unless ``tp_mesh_dim`` / ``dp_mesh_dim`` are usable on a mesh with ``ndim`` axes for this mode."""
        if self.shards_the_batch and ndim > 1 and self.dp_mesh_dim is None:
            raise ValueError(f"dp_mesh_dim: mode {self.mode!r} on a {ndim}-axis mesh needs to know which axis splits the batch")
        _schema.axis_index(self.tp_mesh_dim, ndim, "tp_mesh_dim")
        _schema.axis_index(self.dp_mesh_dim, ndim, "dp_mesh_dim", optional=True)
        if self.uses_tensor_parallel and self.dp_mesh_dim == self.tp_mesh_dim:
            raise ValueError(f"tp_mesh_dim and dp_mesh_dim both name axis {self.tp_mesh_dim}; tensor and data parallelism need "
                             "different axes")

    def axis_names(self, ndim: int) -> Optional[Tuple[str, ...]]:
        """Names for a new mesh: ``tp`` / ``dp`` at their axes, ``axis<i>`` elsewhere; one-axis meshes stay unnamed."""
        if ndim <= 1:
            return None
        names = [f"axis{i}" for i in range(ndim)]
        names[self.tp_mesh_dim] = "tp"
        if self.dp_mesh_dim is not None:
            names[self.dp_mesh_dim] = "dp"
        return tuple(names)
