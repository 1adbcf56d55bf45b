"""Process-group bootstrap and device-mesh queries.

The public helpers keep the names of ``spikingjelly/activation_based/distributed/mesh.py:21-168``; every question about a
mesh (shape, this rank's coordinate, the group or sub-mesh of one axis) is answered by one small view class,
:class:`MeshView`, which also accepts a plain process group or ``None`` so that callers need no special cases."""
from __future__ import annotations

import inspect
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..logger import logger
from . import _schema

try:
    from torch.distributed.device_mesh import DeviceMesh, init_device_mesh
    DTENSOR_AVAILABLE = True
except ImportError:                                       # pragma: no cover
    DeviceMesh = None
    init_device_mesh = None
    DTENSOR_AVAILABLE = False

__all__ = ["DTENSOR_AVAILABLE", "MeshView", "ensure_distributed_initialized", "build_device_mesh", "resolve_data_parallel_partition",
           "resolve_tensor_parallel_group_size"]


class MeshView:
    """Read-only answers about a ``DeviceMesh`` (or the default process group when there is no mesh tensor)."""

    def __init__(self, mesh):
        self.mesh = mesh
        grid = getattr(mesh, "mesh", None)
        self.shape: Optional[Tuple[int, ...]] = None if grid is None else tuple(int(s) for s in grid.shape)

    @property
    def ndim(self) -> int:
        return 1 if self.shape is None else len(self.shape)

    def extent(self, axis: int, field: str) -> int:
        if self.shape is None:
            return dist.get_world_size() if dist.is_initialized() else 1
        return self.shape[_schema.axis_index(axis, len(self.shape), field)]

    def coordinate(self) -> Optional[Tuple[int, ...]]:
        if self.shape is None:
            return (dist.get_rank(),) if dist.is_initialized() else (0,)
        where = self.mesh.get_coordinate() if hasattr(self.mesh, "get_coordinate") else None
        return None if where is None else tuple(int(c) for c in where)

    def axis_group(self, axis: int):
        groups = self.mesh.get_all_groups() if hasattr(self.mesh, "get_all_groups") else self.mesh.get_dim_groups()
        return groups[_schema.axis_index(axis, len(groups), "mesh axis")]

    def axis_submesh(self, axis: int):
        if getattr(self.mesh, "ndim", 1) == 1:
            return self.mesh
        names = getattr(self.mesh, "mesh_dim_names", None)
        if not names:
            raise ValueError("a mesh with several axes must carry axis names before one axis can be sliced out of it")
        return self.mesh[names[axis]]


def ensure_distributed_initialized(backend: Optional[str] = None, init_method: Optional[str] = None, rank: Optional[int] = None,
                                   world_size: Optional[int] = None) -> bool:
    """Create the default process group if there is none yet and say whether this call created it.  The backend defaults
    to NCCL on a machine with CUDA (bound to the current device, which lets NCCL set up eagerly) and to gloo elsewhere."""
    if not dist.is_available():
        raise RuntimeError("this PyTorch build has no torch.distributed")
    if dist.is_initialized():
        return False
    chosen = backend or ("nccl" if torch.cuda.is_available() else "gloo")
    options = {}
    if init_method is not None:
        options["init_method"] = init_method
    if rank is not None:
        options["rank"] = rank
    if world_size is not None:
        options["world_size"] = world_size
    accepts_device = "device_id" in inspect.signature(dist.init_process_group).parameters
    if chosen == "nccl" and accepts_device and torch.cuda.is_available():
        options["device_id"] = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group(backend=chosen, **options)
    logger.info("process group ready: backend=%s rank=%d/%d", chosen, dist.get_rank(), dist.get_world_size())
    return True


def build_device_mesh(device_type: str = "cuda", mesh_shape: Optional[Tuple[int, ...]] = None,
                      mesh_dim_names: Optional[Tuple[str, ...]] = None):
    """``init_device_mesh`` over the whole job; ``mesh_shape`` defaults to one axis of ``world_size`` ranks."""
    if not DTENSOR_AVAILABLE:
        raise RuntimeError("this PyTorch build has no torch.distributed.device_mesh")
    if not dist.is_initialized():
        raise RuntimeError("no process group yet: call ensure_distributed_initialized() before building a mesh")
    world = dist.get_world_size()
    shape = (world,) if mesh_shape is None else tuple(_schema.positive(s, "mesh_shape entry") for s in mesh_shape)
    covered = 1
    for extent in shape:
        covered *= extent
    if covered != world:
        raise ValueError(f"mesh_shape {shape} covers {covered} rank(s) but the job has {world}")
    mesh = init_device_mesh(device_type, shape, mesh_dim_names=mesh_dim_names)
    logger.info("device mesh ready: %s %s names=%s", device_type, shape, mesh_dim_names)
    return mesh


# The three helpers below are what the tensor-parallel, FSDP and execution modules import.
def _resolve_mesh_submesh(device_mesh, mesh_dim: int):
    return MeshView(device_mesh).axis_submesh(mesh_dim)


def _resolve_mesh_dim_group(device_mesh, mesh_dim: int):
    return MeshView(device_mesh).axis_group(mesh_dim)


def _resolve_dp_group_from_mesh(device_mesh, dp_mesh_dim: Optional[int]):
    return None if dp_mesh_dim is None else MeshView(device_mesh).axis_group(dp_mesh_dim)


def resolve_data_parallel_partition(device_mesh, dp_mesh_dim: Optional[int], sharded_by_data_parallel: bool) -> Tuple[int, int]:
    """``(replicas, index of this rank's replica)`` — what a distributed sampler needs.  Ranks that only differ along a
    tensor-parallel axis belong to the same replica and must read the same samples."""
    if device_mesh is None or not sharded_by_data_parallel:
        return 1, 0
    view = MeshView(device_mesh)
    if view.shape is None:
        return view.extent(0, "dp_mesh_dim"), view.coordinate()[0]
    if dp_mesh_dim is None:
        if view.ndim != 1:
            raise ValueError("dp_mesh_dim: a mesh with several axes needs to be told which axis splits the batch")
        dp_mesh_dim = 0
    replicas = view.extent(dp_mesh_dim, "dp_mesh_dim")
    where = view.coordinate()
    if where is None:
        raise ValueError("this rank is not part of the given mesh, so it has no data-parallel index")
    return replicas, where[dp_mesh_dim]


def resolve_tensor_parallel_group_size(device_mesh, tp_mesh_dim: int, tensor_parallel_enabled: bool) -> int:
    if device_mesh is None or not tensor_parallel_enabled:
        return 1
    return MeshView(device_mesh).extent(tp_mesh_dim, "tp_mesh_dim")
