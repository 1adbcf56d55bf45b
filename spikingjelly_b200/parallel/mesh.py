"""Process-group and device-mesh helpers.
Parity: ``spikingjelly/activation_based/distributed/mesh.py:21-259``."""
from __future__ import annotations

import inspect
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..logger import logger

try:
    from torch.distributed.device_mesh import DeviceMesh, init_device_mesh
    DTENSOR_AVAILABLE = True
except ImportError:                                       # pragma: no cover
    DeviceMesh = None
    init_device_mesh = None
    DTENSOR_AVAILABLE = False

__all__ = ["DTENSOR_AVAILABLE", "ensure_distributed_initialized", "build_device_mesh", "resolve_data_parallel_partition",
           "resolve_tensor_parallel_group_size"]


def ensure_distributed_initialized(backend: Optional[str] = None, init_method: Optional[str] = None, rank: Optional[int] = None,
                                   world_size: Optional[int] = None) -> bool:
    """Initialise the default process group unless it exists; returns whether this call did it.
    Default backend: NCCL with CUDA (bound to the current device), gloo otherwise."""
    if dist.is_available() and dist.is_initialized():
        return False
    if not dist.is_available():
        raise RuntimeError("torch.distributed is not available in the current PyTorch build.")
    backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
    kwargs = {k: v for k, v in (("init_method", init_method), ("rank", rank), ("world_size", world_size)) if v is not None}
    if backend == "nccl" and torch.cuda.is_available() and "device_id" in inspect.signature(dist.init_process_group).parameters:
        kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group(backend=backend, **kwargs)
    logger.info("distributed_process_group_initialized backend=%s rank=%s world_size=%s", backend, dist.get_rank(), dist.get_world_size())
    return True


def build_device_mesh(device_type: str = "cuda", mesh_shape: Optional[Tuple[int, ...]] = None,
                      mesh_dim_names: Optional[Tuple[str, ...]] = None):
    if not DTENSOR_AVAILABLE:
        raise RuntimeError("DeviceMesh is unavailable in this PyTorch build.")
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed is not initialized. Call ensure_distributed_initialized() first.")
    world = dist.get_world_size()
    mesh_shape = (world,) if mesh_shape is None else tuple(mesh_shape)
    volume = 1
    for s in mesh_shape:
        volume *= s
    if volume != world:
        raise ValueError(f"mesh_shape={mesh_shape} uses {volume} ranks, but world_size={world}.")
    mesh = init_device_mesh(device_type, mesh_shape, mesh_dim_names=mesh_dim_names)
    logger.info("distributed_device_mesh_created device_type=%s mesh_shape=%s mesh_dim_names=%s world_size=%s", device_type,
                mesh_shape, mesh_dim_names, world)
    return mesh


def _resolve_mesh_submesh(device_mesh, mesh_dim: int):
    if getattr(device_mesh, "ndim", 1) == 1:
        return device_mesh
    if getattr(device_mesh, "mesh_dim_names", None):
        return device_mesh[device_mesh.mesh_dim_names[mesh_dim]]
    raise ValueError("A multi-dimensional DeviceMesh requires mesh_dim_names to derive a 1D submesh.")


def _resolve_mesh_dim_group(device_mesh, mesh_dim: int):
    groups = device_mesh.get_all_groups() if hasattr(device_mesh, "get_all_groups") else device_mesh.get_dim_groups()
    if mesh_dim < 0 or mesh_dim >= len(groups):
        raise ValueError(f"mesh_dim={mesh_dim} is out of range for a mesh with {len(groups)} dimensions.")
    return groups[mesh_dim]


def _resolve_dp_group_from_mesh(device_mesh, dp_mesh_dim: Optional[int]):
    return None if dp_mesh_dim is None else _resolve_mesh_dim_group(device_mesh, dp_mesh_dim)


def resolve_data_parallel_partition(device_mesh, dp_mesh_dim: Optional[int], sharded_by_data_parallel: bool) -> Tuple[int, int]:
    """``(number of data replicas, index of this rank's replica)`` for a sampler."""
    if not sharded_by_data_parallel or device_mesh is None:
        return 1, 0
    mesh_tensor = getattr(device_mesh, "mesh", None)
    if mesh_tensor is None:
        return (dist.get_world_size(), dist.get_rank()) if dist.is_initialized() else (1, 0)
    shape = tuple(int(v) for v in mesh_tensor.shape)
    coord = device_mesh.get_coordinate() if hasattr(device_mesh, "get_coordinate") else None
    coord = tuple(int(v) for v in coord) if coord is not None else None
    if dp_mesh_dim is None:
        if len(shape) != 1:
            raise ValueError("dp_mesh_dim must be specified for data-parallel sharding on a multi-dimensional mesh.")
        dp_mesh_dim = 0
    elif dp_mesh_dim < 0 or dp_mesh_dim >= len(shape):
        raise ValueError(f"dp_mesh_dim={dp_mesh_dim} is out of range for a mesh with shape {shape}.")
    if coord is None:
        raise ValueError("Current rank does not belong to the supplied DeviceMesh; cannot derive a data-parallel partition index.")
    return shape[dp_mesh_dim], coord[dp_mesh_dim]


def resolve_tensor_parallel_group_size(device_mesh, tp_mesh_dim: int, tensor_parallel_enabled: bool) -> int:
    if not tensor_parallel_enabled or device_mesh is None:
        return 1
    mesh_tensor = getattr(device_mesh, "mesh", None)
    if mesh_tensor is None:
        return dist.get_world_size() if dist.is_initialized() else 1
    shape = tuple(int(v) for v in mesh_tensor.shape)
    if tp_mesh_dim < 0 or tp_mesh_dim >= len(shape):
        raise ValueError(f"tp_mesh_dim={tp_mesh_dim} is out of range for a mesh with shape {shape}.")
    return shape[tp_mesh_dim]
