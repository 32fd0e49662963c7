"""Where a backward kernel puts a weight gradient.

The distributed optimizer binds every parameter's ``.grad`` to a slice of one flat bf16
buffer (as the reference does, core/optimizer.py:54-60). Letting autograd *add* each new
weight gradient into that slice costs an extra read-modify-write per parameter per step
and forces a full-buffer memset in ``zero_grad``. Instead, backward kernels write (first
use in a step) or accumulate (later uses) straight into the slice through a
:class:`GradSink`, and return ``None`` to autograd.
"""
from __future__ import annotations

import torch


class GradSink:
    __slots__ = ("param",)

    def __init__(self, param: torch.nn.Parameter):
        self.param = param

    def target(self) -> torch.Tensor:
        return self.param.grad

    def consume_accumulate(self) -> bool:
        """True if the slice already holds this step's gradient (so the kernel must add)."""
        fresh = getattr(self.param, "_grad_fresh", False)
        self.param._grad_fresh = False
        return not fresh

    def done(self) -> None:
        """Tell the owner (optimizer bucket logic) that this parameter's gradient is final."""
        cb = getattr(self.param, "_grad_ready_cb", None)
        if cb is not None:
            cb(self.param)

    def parked(self) -> None:
        """Tell the owner that the kernel producing this gradient has been queued for a batched
        launch (so it can ask for the launch when nothing else is outstanding)."""
        cb = getattr(self.param, "_grad_parked_cb", None)
        if cb is not None:
            cb(self.param)

    @staticmethod
    def of(param: torch.nn.Parameter | None) -> "GradSink | None":
        if param is None or param.grad is None or not getattr(param, "_grad_sink_ok", False):
            return None
        return GradSink(param)
