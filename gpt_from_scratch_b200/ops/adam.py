"""Fused optimizer kernels (csrc/loss_optim.cu): deterministic sum of squares and
clip + AdamW + bf16 cast in one pass, with the clip decision made on the device.

Reference counterpart: core/optimizer.py:84-104 (bf16->fp32 cast, square, sum, sqrt, a
host-synchronising ``if norm > clip``, in-place scale, cast, torch AdamW, cast).
"""
from __future__ import annotations

import math

import torch

from . import _lib

_scratch: dict[int, torch.Tensor] = {}


def _sumsq_scratch(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _scratch.get(idx)
    if t is None:
        t = torch.zeros(_lib.lib().gfs_sumsq_scratch_bytes() // 4, dtype=torch.float32, device=device)
        _scratch[idx] = t
    return t


def sumsq_bf16(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[0] = sum(x.float()**2); x is a contiguous bf16 vector, out a 1-element fp32 tensor."""
    rc = _lib.lib().gfs_sumsq_bf16(x.data_ptr(), x.numel(), out.data_ptr(), _sumsq_scratch(x.device).data_ptr(),
                                   _lib.stream_ptr())
    _lib.check(rc, "gfs_sumsq_bf16")
    return out


def adamw_step(grad: torch.Tensor, master: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor,
               param_out: torch.Tensor, *, step: int, lr: float, beta1: float, beta2: float, eps: float,
               weight_decay: float, sumsq: torch.Tensor | None, clip: float, grad_scale: float = 1.0,
               norm_out: torch.Tensor | None = None, step_dev: torch.Tensor | None = None) -> None:
    """``step_dev``: optional device float with the step count; the kernel then derives the bias
    corrections from it instead of from ``step`` (for launches captured in a CUDA graph)."""
    bc1 = 1.0 - beta1 ** step
    bc2_sqrt = math.sqrt(1.0 - beta2 ** step)
    rc = _lib.lib().gfs_adamw_step(grad.data_ptr(), master.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(),
                                   param_out.data_ptr(), grad.numel(), _lib.ptr(sumsq), _lib.ptr(norm_out),
                                   lr, beta1, beta2, eps, weight_decay, bc1, bc2_sqrt, clip, grad_scale,
                                   _lib.ptr(step_dev), _lib.stream_ptr())
    _lib.check(rc, "gfs_adamw_step")
