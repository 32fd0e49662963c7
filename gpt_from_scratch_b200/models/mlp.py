"""SwiGLU feed-forward block. Reference: core/mlp.py:9-33 (gate_up_proj column-parallel
``H -> 2I`` whose local rows are ``[gate_local | up_local]``, ``silu(gate) * up``,
down_proj row-parallel ``I -> H``)."""
from __future__ import annotations

import torch.nn as nn

from ..ops.grad_sink import GradSink
from ..ops.mlp_fused import _FusedMLP, fused_mlp_supported
from ..ops.swiglu import swiglu
from ..parallel import mappings
from ..parallel import parallel_state as ps
from ..parallel.layers import ColumnParallelLinear, RowParallelLinear
from .init import get_init_method


class ParallelMLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.hidden_size = config.hidden_size
        self.intermediate_size = getattr(config, "intermediate_size", None) or 4 * config.hidden_size
        bias = getattr(config, "bias", False)
        init_method = get_init_method(config)
        self.gate_up_proj = ColumnParallelLinear(self.hidden_size, 2 * self.intermediate_size, bias=bias,
                                                 init_method=init_method)
        self.down_proj = RowParallelLinear(self.intermediate_size, self.hidden_size, bias=bias,
                                           init_method=init_method)

    def forward(self, hidden_states, residual=None):
        world = ps.get_tensor_model_parallel_world_size()
        w_gu, w_down = self.gate_up_proj.weight, self.down_proj.weight
        fused_comm_active = world > 1 and ps.get_comm_impl() == "fused"
        if (self.gate_up_proj.bias is None and self.down_proj.bias is None and not fused_comm_active and
                fused_mlp_supported(hidden_states, w_gu, w_down)):
            # both GEMMs local: SwiGLU lives in their epilogues
            x = mappings.gather_from_sequence_parallel_region(hidden_states)
            out = _FusedMLP.apply(x, w_gu, w_down, residual if world == 1 else None, GradSink.of(w_gu),
                                  GradSink.of(w_down))
            if world > 1:
                out = mappings.reduce_scatter_to_sequence_parallel_region(out)
                if residual is not None:
                    out = out + residual
            return out
        if fused_comm_active and self.gate_up_proj.bias is None and self.down_proj.bias is None:
            from ..parallel import fused_comm
            if fused_comm.fused_mlp_eligible(hidden_states, w_gu, w_down):
                # gather -> gate|up GEMM + SwiGLU epilogue -> down GEMM -> reduce-scatter (+ residual)
                return fused_comm.swiglu_mlp(hidden_states, w_gu, w_down, residual)
        gu = self.gate_up_proj(hidden_states)              # [S, B, 2I/P]
        S, B, W = gu.shape
        act = swiglu(gu.reshape(S * B, W)).view(S, B, W // 2)
        return self.down_proj(act, residual)               # [S/P, B, H]
