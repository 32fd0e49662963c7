"""Vocab-parallel cross entropy kernels (csrc/loss_optim.cu).

Forward reads the local logits once (online max / sum-exp / target logit per row, fp32);
backward overwrites the logits buffer in place with ``(softmax - onehot) * grad`` so no
extra ``[tokens, V/P]`` tensor is ever allocated. The reference materialises two such
tensors (core/tensor_parallel/loss.py:16,19) and does its math in bf16.
"""
from __future__ import annotations

import torch

from . import _lib


def ce_local_stats(logits2d: torch.Tensor, target: torch.Tensor, vocab_start: int, single_rank: bool):
    """Returns (stats [M,3] = {max, sumexp, target logit}, lse [M], loss [M]); lse/loss valid iff single_rank."""
    M, Vp = logits2d.shape
    dev = logits2d.device
    stats = torch.empty((M, 3), dtype=torch.float32, device=dev)
    lse = torch.empty(M, dtype=torch.float32, device=dev)
    loss = torch.empty(M, dtype=torch.float32, device=dev)
    rc = _lib.lib().gfs_ce_fwd(logits2d.data_ptr(), target.data_ptr(), stats.data_ptr(), lse.data_ptr(),
                               loss.data_ptr(), M, Vp, logits2d.stride(0), vocab_start, 1 if single_rank else 0,
                               _lib.stream_ptr())
    _lib.check(rc, "gfs_ce_fwd")
    return stats, lse, loss


def ce_stats_from_partials(partials: torch.Tensor, logits2d: torch.Tensor, target: torch.Tensor, vocab_start: int,
                           single_rank: bool):
    """Same outputs as :func:`ce_local_stats`, from the per-slice statistics the LM-head GEMM epilogue
    produced (``partials`` fp32 ``[parts, M, 2]``): no pass over the logits."""
    M, Vp = logits2d.shape
    dev = logits2d.device
    stats = torch.empty((M, 3), dtype=torch.float32, device=dev)
    lse = torch.empty(M, dtype=torch.float32, device=dev)
    loss = torch.empty(M, dtype=torch.float32, device=dev)
    rc = _lib.lib().gfs_ce_from_partials(partials.data_ptr(), logits2d.data_ptr(), target.data_ptr(), stats.data_ptr(),
                                         lse.data_ptr(), loss.data_ptr(), partials.shape[0], M, Vp,
                                         logits2d.stride(0), vocab_start, 1 if single_rank else 0, _lib.stream_ptr())
    _lib.check(rc, "gfs_ce_from_partials")
    return stats, lse, loss


def ce_combine(stats_all: torch.Tensor):
    """stats_all: [world, M, 3] -> (lse [M], loss [M])."""
    world, M, _ = stats_all.shape
    lse = torch.empty(M, dtype=torch.float32, device=stats_all.device)
    loss = torch.empty(M, dtype=torch.float32, device=stats_all.device)
    rc = _lib.lib().gfs_ce_combine(stats_all.data_ptr(), lse.data_ptr(), loss.data_ptr(), M, world,
                                   _lib.stream_ptr())
    _lib.check(rc, "gfs_ce_combine")
    return lse, loss


def ce_backward_inplace(logits2d: torch.Tensor, lse: torch.Tensor, target: torch.Tensor, grad_rows: torch.Tensor,
                        vocab_start: int) -> torch.Tensor:
    M, Vp = logits2d.shape
    rc = _lib.lib().gfs_ce_bwd(logits2d.data_ptr(), lse.data_ptr(), target.data_ptr(), grad_rows.data_ptr(), M, Vp,
                               logits2d.stride(0), vocab_start, _lib.stream_ptr())
    _lib.check(rc, "gfs_ce_bwd")
    return logits2d
