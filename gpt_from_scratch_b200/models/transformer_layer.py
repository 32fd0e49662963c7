"""Pre-norm transformer block with tensor-parallel attention and SwiGLU MLP.

Structure and parameter names follow the reference (core/transformer_layer.py:14-105):
``x + drop(attn(norm1(x)))`` then ``x + drop(mlp(norm2(x)))`` on ``[S/P, B, H]``
activations. The attention path keeps the projection output packed as
``[S, B, 3, nh/P, D]`` and hands it to the fused RoPE + flash-attention operator, so none
of the reference's permute/contiguous copies exist; with dropout disabled (the only value
the reference's CLI can reach) the residual adds run inside the row-parallel GEMMs.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops.attention import attention_reference, fused_rope_attention
from ..ops.dropout import dropout_add
from ..ops.rope import rope_reference
from ..parallel import parallel_state as ps
from ..parallel.layers import ColumnParallelLinear, RowParallelLinear
from .init import get_init_method
from .mlp import ParallelMLP
from .normalization import RMSNorm
from .position_embeddings import RotaryEmbedding


class ParallelAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.hidden_size = config.hidden_size
        self.num_attention_heads = config.num_attention_heads
        self.head_dim = self.hidden_size // self.num_attention_heads
        world = ps.get_tensor_model_parallel_world_size()
        assert self.num_attention_heads % world == 0, "heads must be divisible by the TP size"
        self.num_heads_per_partition = self.num_attention_heads // world
        bias = getattr(config, "bias", False)
        init_method = get_init_method(config)
        self.qkv_proj = ColumnParallelLinear(self.hidden_size, 3 * self.hidden_size, bias=bias,
                                             init_method=init_method)
        self.out_proj = RowParallelLinear(self.hidden_size, self.hidden_size, bias=bias, init_method=init_method)
        self.rotary_emb = RotaryEmbedding(self.head_dim, config.max_position_embeddings,
                                          getattr(config, "rope_base", 10000.0),
                                          round_to_activation_dtype=getattr(config, "reference_quirks", False))
        self.attention_impl = getattr(config, "attention_impl", "fused")

    def forward(self, hidden_states, residual=None):
        nh, D = self.num_heads_per_partition, self.head_dim
        world = ps.get_tensor_model_parallel_world_size()
        S_full, B_ = hidden_states.shape[0] * world, hidden_states.shape[1]
        w = self.qkv_proj.weight
        rope_in_gemm = (self.attention_impl == "fused" and w.is_cuda and w.dtype == hidden_states.dtype ==
                        torch.bfloat16 and D in (64, 128) and self.qkv_proj.bias is None)
        if rope_in_gemm:
            # q and k are rotated by the projection GEMM's epilogue
            cos, sin = self.rotary_emb(hidden_states, S_full)
            qkv = self.qkv_proj(hidden_states, rope=(cos, sin, 2 * nh * D, D, B_))
        else:
            qkv = self.qkv_proj(hidden_states)             # [S, B, 3H/P]
        S, B, W = qkv.shape
        if not rope_in_gemm:
            cos, sin = self.rotary_emb(qkv, S)
        if self.attention_impl == "fused":
            ctx = fused_rope_attention(qkv.reshape(S * B, W), cos, sin, S, B, nh, D,
                                       pre_rotated=rope_in_gemm).view(S, B, nh * D)
        else:
            q, k, v = qkv.view(S, B, 3, nh, D).unbind(2)
            q, k = rope_reference(q, cos, sin), rope_reference(k, cos, sin)
            o = attention_reference(q.permute(1, 2, 0, 3), k.permute(1, 2, 0, 3), v.permute(1, 2, 0, 3), True)
            ctx = o.permute(2, 0, 1, 3).reshape(S, B, nh * D)
        return self.out_proj(ctx, residual)                # [S/P, B, H]


class TransformerLayer(nn.Module):
    def __init__(self, layer_id, config):
        super().__init__()
        self.layer_id = layer_id
        self.input_norm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.attention = ParallelAttention(config)
        self.post_attention_norm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.mlp = ParallelMLP(config)
        self.dropout_prob = getattr(config, "dropout_prob", 0.0)
        self.dropout = nn.Dropout(self.dropout_prob)

    def forward(self, hidden_states):
        if self.dropout_prob == 0.0 or not self.training:
            h, res = self.input_norm(hidden_states, fork=True)
            x = self.attention(h, residual=res)
            h, res = self.post_attention_norm(x, fork=True)
            return self.mlp(h, residual=res)
        # residual + dropout(x) in one kernel (regenerated mask in the backward)
        x = dropout_add(self.attention(self.input_norm(hidden_states)), hidden_states, self.dropout_prob, True)
        return dropout_add(self.mlp(self.post_attention_norm(x)), x, self.dropout_prob, True)
