"""RMSNorm forward/backward (csrc/elementwise.cu) with the reference's rounding order:
normalise in fp32, round to the activation dtype, then multiply by the weight
(core/normalization.py:16-24). The backward can fold in the gradient that arrives on
the residual branch so the block's ``dx`` is produced by one kernel.
"""
from __future__ import annotations

import torch

from . import _lib


def rmsnorm_reference(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    x32 = x.float()
    n = x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + eps)
    return n.to(x.dtype) * w


def _parts(rows: int) -> int:
    return _lib.lib().gfs_rmsnorm_bwd_parts(rows)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, grad_sink, fork):
        H = x.shape[-1]
        x2 = x.contiguous().view(-1, H)
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        rc = _lib.lib().gfs_rmsnorm_fwd(x2.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, H, eps,
                                        _lib.stream_ptr())
        _lib.check(rc, "gfs_rmsnorm_fwd")
        ctx.save_for_backward(x2, w, rstd)
        ctx.grad_sink = grad_sink
        ctx.xshape = x.shape
        ctx.fork = fork
        if fork:
            # second output: the input itself, to be used as the residual branch, so that the
            # gradient arriving on that branch is added inside the backward kernel
            return y.view(x.shape), x
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dres=None):
        x2, w, rstd = ctx.saved_tensors
        rows, H = x2.shape
        dy2 = dy.contiguous().view(rows, H)
        dx = torch.empty_like(x2)
        parts = _parts(rows)
        partial = torch.empty(parts * H, dtype=torch.float32, device=x2.device)
        sink = ctx.grad_sink
        if sink is not None:
            dw, acc = sink.target(), sink.consume_accumulate()
        else:
            dw, acc = torch.empty_like(w), False
        dres_ptr = 0
        if dres is not None:
            dres = dres.contiguous().view(rows, H)
            dres_ptr = dres.data_ptr()
        rc = _lib.lib().gfs_rmsnorm_bwd(dy2.data_ptr(), x2.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres_ptr,
                                        dx.data_ptr(), dw.data_ptr(), partial.data_ptr(), rows, H, 1 if acc else 0,
                                        _lib.stream_ptr())
        _lib.check(rc, "gfs_rmsnorm_bwd")
        _lib.add_launches(1)
        return dx.view(ctx.xshape), (None if sink is not None else dw), None, None, None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, grad_sink=None, fork: bool = False):
    """``grad_sink``: optional :class:`GradSink` that receives the weight gradient in place.
    ``fork=True`` returns ``(y, x)``: use the second value as the residual-branch input and the
    backward kernel adds that branch's gradient to ``dx`` itself (no separate add kernel)."""
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        return _RMSNorm.apply(x, w, eps, grad_sink, fork)
    y = rmsnorm_reference(x, w, eps)
    return (y, x) if fork else y
