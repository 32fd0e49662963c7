"""RMSNorm forward/backward (csrc/elementwise.cu) with the reference's rounding order:
normalise in fp32, round to the activation dtype, then multiply by the weight
(core/normalization.py:16-24). The backward can fold in the gradient that arrives on
the residual branch so the block's ``dx`` is produced by one kernel.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def rmsnorm_reference(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    x32 = x.float()
    n = x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + eps)
    return n.to(x.dtype) * w


def _parts(rows: int) -> int:
    return _lib.lib().gfs_rmsnorm_bwd_parts(rows)


class _DwReduceQueue:
    """Weight-gradient reductions of the RMSNorm layers waiting for one batched launch.

    Each layer's backward leaves fp32 column partials; turning them into the bf16 weight
    gradient is a few-microsecond kernel per layer. Layers whose gradient goes to a gradient
    sink park (partial, destination) here; one launch handles up to 32 layers, at the end of
    the backward pass (autograd-engine callback) or at :func:`flush_dw_reductions`."""

    MAX = 32

    def __init__(self):
        self.items: list[tuple] = []
        self._callback_pending = False

    def _end_of_backward(self) -> None:
        self._callback_pending = False
        self.flush()

    def push(self, partial, dw, parts, accumulate, H, done_cb) -> None:
        if self.items and self.items[0][4] != H:
            self.flush()
        self.items.append((partial, dw, parts, accumulate, H, done_cb))
        if len(self.items) == self.MAX:
            self.flush()
        elif not self._callback_pending:
            try:
                torch.autograd.Variable._execution_engine.queue_callback(self._end_of_backward)
                self._callback_pending = True
            except RuntimeError:
                pass   # not inside a backward pass: the explicit flush will run it

    def flush(self) -> None:
        items, self.items = self.items, []
        if not items:
            return
        n = len(items)
        U, I = ctypes.c_ulonglong * n, ctypes.c_int * n
        rc = _lib.lib().gfs_rmsnorm_dw_reduce_multi(
            n, U(*[it[0].data_ptr() for it in items]), U(*[it[1].data_ptr() for it in items]),
            I(*[it[2] for it in items]), I(*[1 if it[3] else 0 for it in items]), items[0][4], _lib.stream_ptr())
        _lib.check(rc, "gfs_rmsnorm_dw_reduce_multi")
        for it in items:
            if it[5] is not None:
                it[5]()


_dw_queue = _DwReduceQueue()


def flush_dw_reductions() -> None:
    """Run every parked RMSNorm weight-gradient reduction (no-op when nothing is parked)."""
    _dw_queue.flush()


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
        defer = sink is not None and dw.is_contiguous()
        rc = _lib.lib().gfs_rmsnorm_bwd(dy2.data_ptr(), x2.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres_ptr,
                                        dx.data_ptr(), None if defer else dw.data_ptr(), partial.data_ptr(), rows, H,
                                        1 if acc else 0, _lib.stream_ptr())
        _lib.check(rc, "gfs_rmsnorm_bwd")
        if defer:
            _dw_queue.push(partial, dw, parts, acc, H, sink.done)
            sink.parked()
        else:
            _lib.add_launches(1)
            if sink is not None:
                sink.done()
        return dx.view(ctx.xshape), (None if sink is not None else dw), None, None, None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, grad_sink=None, fork: bool = False):
    """``grad_sink``: optional :class:`GradSink` that receives the weight gradient in place.
    ``fork=True`` returns ``(y, x)``: use the second value as the residual-branch input and the
    backward kernel adds that branch's gradient to ``dx`` itself (no separate add kernel)."""
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        return _RMSNorm.apply(x, w, eps, grad_sink, fork)
    y = rmsnorm_reference(x, w, eps)
    return (y, x) if fork else y
