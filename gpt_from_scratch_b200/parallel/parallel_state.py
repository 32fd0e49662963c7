"""Process-group registry for tensor (TP) and data (DP) parallelism.

Rank layout, as in the reference (core/parallel_state.py:43-62): world rank ``r`` has TP
rank ``r % P`` and DP rank ``r // P``; TP groups are contiguous rank ranges, DP groups are
strided. Everything also works without ``torch.distributed`` (one process, one GPU or CPU):
sizes are then 1 and the groups are ``None``.

Beyond the reference this module owns the per-process device choice (so the same model
code runs on CPU/gloo and CUDA/NCCL), the model-parallel RNG seed, and the switch between
the NCCL composition and the fused symmetric-memory communication kernels.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

_TP_GROUP = None
_DP_GROUP = None
_TP_RANK = 0
_TP_WORLD = 1
_DP_RANK = 0
_DP_WORLD = 1
_TP_RANKS: list[int] = [0]
_DP_RANKS: list[int] = [0]
_INITIALIZED = False
_DEVICE: torch.device | None = None
_SEED = 1234
_COMM_IMPL = "nccl"  # "nccl": torch.distributed collectives; "fused": symmetric-memory kernels


def initialize_parallel_state(tensor_model_parallel_size: int = 1) -> None:
    """Build the TP and DP groups. Collective: every rank must call it."""
    global _TP_GROUP, _DP_GROUP, _TP_RANK, _TP_WORLD, _DP_RANK, _DP_WORLD, _INITIALIZED, _TP_RANKS, _DP_RANKS
    P = int(tensor_model_parallel_size)
    if not (dist.is_available() and dist.is_initialized()):
        if P != 1:
            raise RuntimeError("tensor parallelism needs torch.distributed to be initialised")
        _TP_GROUP = _DP_GROUP = None
        _TP_RANK = _DP_RANK = 0
        _TP_WORLD = _DP_WORLD = 1
        _TP_RANKS, _DP_RANKS = [0], [0]
        _INITIALIZED = True
        return
    world = dist.get_world_size()
    rank = dist.get_rank()
    if P < 1 or world % P != 0:
        raise ValueError(f"world size {world} is not divisible by tensor parallel size {P}")
    dp = world // P
    for i in range(dp):
        ranks = list(range(i * P, (i + 1) * P))
        group = dist.new_group(ranks)
        if rank in ranks:
            _TP_GROUP, _TP_RANKS = group, ranks
    for i in range(P):
        ranks = list(range(i, world, P))
        group = dist.new_group(ranks)
        if rank in ranks:
            _DP_GROUP, _DP_RANKS = group, ranks
    _TP_RANK, _TP_WORLD = rank % P, P
    _DP_RANK, _DP_WORLD = rank // P, dp
    _INITIALIZED = True


def destroy_model_parallel() -> None:
    global _TP_GROUP, _DP_GROUP, _TP_RANK, _TP_WORLD, _DP_RANK, _DP_WORLD, _INITIALIZED, _TP_RANKS, _DP_RANKS
    _TP_GROUP = _DP_GROUP = None
    _TP_RANK = _DP_RANK = 0
    _TP_WORLD = _DP_WORLD = 1
    _TP_RANKS, _DP_RANKS = [0], [0]
    _INITIALIZED = False
    from . import symm
    symm.reset()


def model_parallel_is_initialized() -> bool:
    return _INITIALIZED


def get_tensor_model_parallel_group():
    return _TP_GROUP


def get_tensor_model_parallel_group_rank() -> int:
    return _TP_RANK


def get_tensor_model_parallel_world_size() -> int:
    return _TP_WORLD


def get_tensor_model_parallel_ranks() -> list[int]:
    return list(_TP_RANKS)


def get_data_parallel_group():
    return _DP_GROUP


def get_data_parallel_group_rank() -> int:
    return _DP_RANK


def get_data_parallel_world_size() -> int:
    return _DP_WORLD


def get_data_parallel_ranks() -> list[int]:
    return list(_DP_RANKS)


# -- device / seed / comm implementation ------------------------------------------------
def set_device(device) -> None:
    global _DEVICE
    _DEVICE = torch.device(device)


def get_device() -> torch.device:
    if _DEVICE is not None:
        return _DEVICE
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def set_seed(seed: int) -> None:
    global _SEED
    _SEED = int(seed)


def get_seed() -> int:
    return _SEED


def sharded_param_generator(device: torch.device, salt: int = 0) -> torch.Generator:
    """Generator for a TP-sharded parameter: differs across TP ranks, equal across DP ranks."""
    g = torch.Generator(device=device)
    g.manual_seed(_SEED + 2718 * (_TP_RANK + 1) + 7919 * salt)
    return g


def set_comm_impl(impl: str) -> None:
    global _COMM_IMPL
    if impl not in ("nccl", "fused"):
        raise ValueError(impl)
    _COMM_IMPL = impl


def get_comm_impl() -> str:
    return _COMM_IMPL
