"""SwiGLU activation on the packed ``[M, 2I]`` gate|up projection (csrc/elementwise.cu).

``act = silu(gate) * up`` with gate = first I columns, up = last I columns, the
reference's local layout (core/mlp.py:25-28).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib


def swiglu_reference(gu: torch.Tensor) -> torch.Tensor:
    gate, up = gu.chunk(2, dim=-1)
    return F.silu(gate) * up


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        M, I2 = gu.shape
        act = torch.empty((M, I2 // 2), dtype=gu.dtype, device=gu.device)
        rc = _lib.lib().gfs_swiglu_fwd(gu.data_ptr(), act.data_ptr(), M, I2 // 2, _lib.stream_ptr())
        _lib.check(rc, "gfs_swiglu_fwd")
        ctx.save_for_backward(gu)
        return act

    @staticmethod
    def backward(ctx, dact):
        (gu,) = ctx.saved_tensors
        M, I2 = gu.shape
        dgu = torch.empty_like(gu)
        rc = _lib.lib().gfs_swiglu_bwd(dact.contiguous().data_ptr(), gu.data_ptr(), dgu.data_ptr(), M, I2 // 2,
                                       _lib.stream_ptr())
        _lib.check(rc, "gfs_swiglu_bwd")
        return dgu


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    if gu.is_cuda and gu.dtype == torch.bfloat16 and gu.dim() == 2 and (gu.shape[1] // 2) % 8 == 0:
        return _SwiGLU.apply(gu.contiguous())
    return swiglu_reference(gu)
