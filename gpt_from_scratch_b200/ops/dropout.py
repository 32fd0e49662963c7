"""``residual + dropout(x)`` in one kernel (csrc/elementwise.cu).

The reference composes ``nn.Dropout`` with the residual add (core/transformer_layer.py:89,
97,103) and notes that it does no per-rank seed handling. Here the keep mask is a
counter-based function of ``(seed, element index)``: the backward regenerates it (no mask
tensor), every call draws a fresh seed from the framework's generator, and the realised
drop probability is ``round(p * 256) / 256``.
"""
from __future__ import annotations

import torch

from . import _lib


def _native(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and x.numel() % 8 == 0


class _DropoutAdd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, p, seed):
        x = x.contiguous()
        res = residual.contiguous() if residual is not None else None
        out = torch.empty_like(x)
        rc = _lib.lib().gfs_dropout_residual(x.data_ptr(), _lib.ptr(res), out.data_ptr(), x.numel(), p, seed, 0,
                                             _lib.stream_ptr())
        _lib.check(rc, "gfs_dropout_residual(fwd)")
        ctx.p, ctx.seed, ctx.has_res = p, seed, residual is not None
        return out

    @staticmethod
    def backward(ctx, dout):
        dout = dout.contiguous()
        dx = torch.empty_like(dout)
        rc = _lib.lib().gfs_dropout_residual(dout.data_ptr(), None, dx.data_ptr(), dout.numel(), ctx.p, ctx.seed, 1,
                                             _lib.stream_ptr())
        _lib.check(rc, "gfs_dropout_residual(bwd)")
        return dx, (dout if ctx.has_res else None), None, None


def dropout_add(x: torch.Tensor, residual: torch.Tensor | None, p: float, training: bool,
                generator: torch.Generator | None = None) -> torch.Tensor:
    """``residual + dropout(x, p)`` (``residual`` may be ``None``)."""
    if not training or p == 0.0:
        return x if residual is None else residual + x
    if _native(x) and (residual is None or (_native(residual) and residual.shape == x.shape)):
        seed = int(torch.randint(0, 2 ** 62, (1,), generator=generator).item())   # host generator: no device sync
        return _DropoutAdd.apply(x, residual, float(p), seed)
    y = torch.nn.functional.dropout(x, p, True)
    return y if residual is None else residual + y
