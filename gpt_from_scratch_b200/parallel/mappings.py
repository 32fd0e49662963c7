"""Sequence-parallel <-> tensor-parallel region mappings (collectives on dim 0).

Same three operator pairs as the reference (core/tensor_parallel/mappings.py:51-107):
gather/reduce-scatter, reduce-scatter/gather, split/gather. They are the identity when the
TP size is 1. These are the *composition* path (torch.distributed over NCCL or gloo); the
fused kernels in ``fused_comm.py`` replace gather+GEMM and GEMM+reduce-scatter pairs when
``--comm-impl fused`` is active.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import parallel_state as ps


def _backend_is_gloo(group) -> bool:
    try:
        return dist.get_backend(group) == "gloo"
    except Exception:
        return False


def all_gather_dim0(x: torch.Tensor, group=None, world: int | None = None) -> torch.Tensor:
    group = ps.get_tensor_model_parallel_group() if group is None else group
    world = ps.get_tensor_model_parallel_world_size() if world is None else world
    if world == 1:
        return x
    x = x.contiguous()
    out = torch.empty((x.shape[0] * world, *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=group)
    return out


def reduce_scatter_dim0(x: torch.Tensor, group=None, world: int | None = None, rank: int | None = None) -> torch.Tensor:
    group = ps.get_tensor_model_parallel_group() if group is None else group
    world = ps.get_tensor_model_parallel_world_size() if world is None else world
    rank = ps.get_tensor_model_parallel_group_rank() if rank is None else rank
    if world == 1:
        return x
    x = x.contiguous()
    assert x.shape[0] % world == 0, "dim 0 must be divisible by the group size"
    n = x.shape[0] // world
    if _backend_is_gloo(group):  # gloo has no reduce_scatter: all-reduce a copy and keep our slice
        tmp = x.clone()
        dist.all_reduce(tmp, group=group)
        return tmp[rank * n:(rank + 1) * n].contiguous()
    out = torch.empty((n, *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x, group=group)
    return out


def split_dim0(x: torch.Tensor) -> torch.Tensor:
    world = ps.get_tensor_model_parallel_world_size()
    if world == 1:
        return x
    rank = ps.get_tensor_model_parallel_group_rank()
    n = x.shape[0] // world
    return x[rank * n:(rank + 1) * n].contiguous()


class _GatherFromSequenceParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return all_gather_dim0(x)

    @staticmethod
    def backward(ctx, g):
        return reduce_scatter_dim0(g)


class _ReduceScatterToSequenceParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return reduce_scatter_dim0(x)

    @staticmethod
    def backward(ctx, g):
        return all_gather_dim0(g)


class _ScatterToSequenceParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return split_dim0(x)

    @staticmethod
    def backward(ctx, g):
        return all_gather_dim0(g)


def gather_from_sequence_parallel_region(x: torch.Tensor) -> torch.Tensor:
    """[S/P, ...] -> [S, ...]; backward reduce-scatters."""
    return _GatherFromSequenceParallelRegion.apply(x)


def reduce_scatter_to_sequence_parallel_region(x: torch.Tensor) -> torch.Tensor:
    """[S, ...] partial sums -> [S/P, ...]; backward all-gathers."""
    return _ReduceScatterToSequenceParallelRegion.apply(x)


def scatter_to_sequence_parallel_region(x: torch.Tensor) -> torch.Tensor:
    """[S, ...] replicated -> this rank's [S/P, ...] slice; backward all-gathers."""
    return _ScatterToSequenceParallelRegion.apply(x)
