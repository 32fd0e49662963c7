"""RMSNorm module (weight ``[H]`` of ones). Reference: core/normalization.py:6-25."""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops.grad_sink import GradSink
from ..ops.rmsnorm import rmsnorm
from ..parallel import parallel_state as ps


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size, device=ps.get_device(), dtype=torch.float32))
        # replicated across TP ranks: its gradient is summed over the TP group by the optimizer
        self.weight.tp_replicated = True

    def forward(self, x: torch.Tensor, fork: bool = False):
        return rmsnorm(x, self.weight, self.eps, GradSink.of(self.weight), fork)
