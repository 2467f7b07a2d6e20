"""Process-group bootstrap and the 2-D (data-parallel x tensor-parallel) rank mesh.

Rank layout follows the reference (models/tp.py:422-483): world ranks are laid out row-major as
``[dp, tp]``; tensor-parallel groups are runs of contiguous ranks (NVLink neighbours), the
data-parallel groups are the strided columns. Unlike the reference, a missing process group is
not an error: a single process is a 1x1 mesh, so every trainer also runs on one GPU (or on CPU),
and the backend is NCCL when CUDA is present and gloo otherwise.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class _Mesh:
    tp_group: Optional[dist.ProcessGroup] = None
    dp_group: Optional[dist.ProcessGroup] = None
    tp_size: int = 1
    dp_size: int = 1
    tp_rank: int = 0
    dp_rank: int = 0
    tp_ranks: tuple = (0,)
    dp_ranks: tuple = (0,)
    initialized: bool = False


_MESH = _Mesh()


def _env_int(name: str, default: int) -> int:
    return int(os.environ.get(name, default))


def maybe_init_dist(backend: Optional[str] = None, timeout_s: float = 1800.0) -> Optional[int]:
    """Create the world process group from torchrun's environment. Returns the rank, or None
    when the job is a single process (then every parallel helper degrades to a no-op)."""
    world = _env_int("WORLD_SIZE", 1)
    if world < 2:
        return None
    rank, local_rank = _env_int("RANK", 0), _env_int("LOCAL_RANK", 0)
    if dist.is_initialized():
        return dist.get_rank()
    use_cuda = torch.cuda.is_available()
    if backend is None:
        backend = "nccl" if use_cuda else "gloo"
    kwargs = {}
    if use_cuda:
        torch.cuda.set_device(local_rank)
        if backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", local_rank)
    dist.init_process_group(backend=backend, rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    return rank


def initialize_model_parallel(model_parallel_size: int, *,
                              model_parallel_backend: Optional[str] = None,
                              ddp_backend: Optional[str] = None) -> None:
    """Build the TP groups (contiguous ranks) and DP groups (strided ranks)."""
    global _MESH
    if not dist.is_initialized():
        _MESH = _Mesh(initialized=True)
        return
    world, rank = dist.get_world_size(), dist.get_rank()
    tp = int(min(model_parallel_size, world))
    assert world % tp == 0, f"world size {world} is not divisible by tensor-parallel size {tp}"
    dp = world // tp
    my_dp, my_tp = divmod(rank, tp)
    mesh = _Mesh(tp_size=tp, dp_size=dp, tp_rank=my_tp, dp_rank=my_dp, initialized=True)
    for k in range(tp):  # every rank must take part in every new_group call, in the same order
        ranks = tuple(i * tp + k for i in range(dp))
        g = dist.new_group(list(ranks), backend=ddp_backend)
        if k == my_tp:
            mesh.dp_group, mesh.dp_ranks = g, ranks
    for i in range(dp):
        ranks = tuple(i * tp + k for k in range(tp))
        g = dist.new_group(list(ranks), backend=model_parallel_backend)
        if i == my_dp:
            mesh.tp_group, mesh.tp_ranks = g, ranks
    _MESH = mesh


def destroy_model_parallel() -> None:
    global _MESH, _ROLLOUT
    _MESH = _Mesh()
    _ROLLOUT = None


_ROLLOUT = None     # (group, ranks, size, rank in group) of the rollout tensor-parallel group


def initialize_rollout_parallel(rollout_tp: int) -> None:
    """Tensor-parallel groups of the PPO rollout engine when generation runs at a wider degree
    than training (``--rollout_tensor_parallel_size``): runs of ``rollout_tp`` contiguous ranks,
    each the union of ``rollout_tp / tp`` neighbouring training tensor-parallel groups.
    Collective over the world (every rank creates every group, in the same order)."""
    global _ROLLOUT
    if not dist.is_initialized() or rollout_tp <= 1:
        _ROLLOUT = None
        return
    world, rank = dist.get_world_size(), dist.get_rank()
    assert world % rollout_tp == 0 and rollout_tp % _MESH.tp_size == 0, \
        f"rollout TP {rollout_tp} must divide the world ({world}) and be a multiple of the " \
        f"training TP ({_MESH.tp_size})"
    if rollout_tp == _MESH.tp_size:
        _ROLLOUT = (_MESH.tp_group, _MESH.tp_ranks, _MESH.tp_size, _MESH.tp_rank)
        return
    for first in range(0, world, rollout_tp):
        ranks = tuple(range(first, first + rollout_tp))
        g = dist.new_group(list(ranks))
        if first <= rank < first + rollout_tp:
            _ROLLOUT = (g, ranks, rollout_tp, rank - first)


def get_rollout_parallel():
    """(group, ranks, size, rank) of this rank's rollout tensor-parallel group; the training
    tensor-parallel group when no separate rollout degree was set up."""
    if _ROLLOUT is not None:
        return _ROLLOUT
    return (_MESH.tp_group, _MESH.tp_ranks, _MESH.tp_size, _MESH.tp_rank)


class model_parallel_as:
    """Context in which the tensor-parallel accessors name another group (the rollout group),
    for code that runs a model sharded over that group through the module path."""

    def __init__(self, group, ranks, size, rank):
        self.new = (group, tuple(ranks), size, rank)

    def __enter__(self):
        m = _MESH
        self.old = (m.tp_group, m.tp_ranks, m.tp_size, m.tp_rank)
        m.tp_group, m.tp_ranks, m.tp_size, m.tp_rank = self.new
        return self

    def __exit__(self, *exc):
        m = _MESH
        m.tp_group, m.tp_ranks, m.tp_size, m.tp_rank = self.old
        return False


def model_parallel_is_initialized() -> bool:
    return _MESH.initialized


def get_model_parallel_group():
    return _MESH.tp_group


def get_data_parallel_group():
    return _MESH.dp_group


def get_model_parallel_world_size() -> int:
    return _MESH.tp_size


def get_model_parallel_rank() -> int:
    return _MESH.tp_rank


def get_data_parallel_world_size() -> int:
    return _MESH.dp_size


def get_data_parallel_rank() -> int:
    return _MESH.dp_rank


def get_model_parallel_ranks() -> tuple:
    return _MESH.tp_ranks


def get_data_parallel_ranks() -> tuple:
    return _MESH.dp_ranks


def get_model_parallel_src_rank() -> int:
    """World rank of the first member of this rank's tensor-parallel group."""
    return _MESH.tp_ranks[0]


def get_data_parallel_src_rank() -> int:
    return _MESH.dp_ranks[0]


def world_size() -> int:
    return dist.get_world_size() if dist.is_initialized() else 1


def world_rank() -> int:
    return dist.get_rank() if dist.is_initialized() else 0


def barrier() -> None:
    if dist.is_initialized():
        dist.barrier()
