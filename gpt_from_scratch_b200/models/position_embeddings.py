"""Rotary embedding tables. ``freqs = base^(-2i/D)`` is a persistent buffer (it appears in
``state_dict`` like in the reference, core/position_embeddings.py:19-23); the cos/sin
caches are non-persistent fp32 ``[max_pos, D/2]`` and grow on demand (the reference's
growth path raises a TypeError, core/position_embeddings.py:46-48)."""
from __future__ import annotations

import torch
import torch.nn as nn

from ..parallel import parallel_state as ps


class RotaryEmbedding(nn.Module):
    def __init__(self, head_dim: int, max_position_embeddings: int = 1024, base: float = 10000.0,
                 round_to_activation_dtype: bool = False):
        super().__init__()
        self.head_dim = head_dim
        self.base = base
        self.max_position_embeddings = max_position_embeddings
        self.round_to_activation_dtype = round_to_activation_dtype
        dev = ps.get_device()
        freqs = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=dev) / head_dim))
        self.register_buffer("freqs", freqs, persistent=True)
        self._rounded_for = None
        self._set_cos_sin_cache(max_position_embeddings)

    def _set_cos_sin_cache(self, seq_len: int) -> None:
        self.max_seq_len_cached = seq_len
        t = torch.arange(seq_len, dtype=torch.float32, device=self.freqs.device)
        ang = torch.outer(t, self.freqs.float())
        self.register_buffer("cos_cached", ang.cos().contiguous(), persistent=False)
        self.register_buffer("sin_cached", ang.sin().contiguous(), persistent=False)
        self._rounded_for = None

    def forward(self, x: torch.Tensor, seq_len: int):
        """Returns fp32 ``(cos, sin)`` of shape ``[seq_len, D/2]``."""
        if seq_len > self.max_seq_len_cached:
            self._set_cos_sin_cache(seq_len)
        if self.round_to_activation_dtype and x.dtype != torch.float32 and self._rounded_for != x.dtype:
            # the reference hands bf16 tables to its kernel (core/position_embeddings.py:51)
            self.cos_cached = self.cos_cached.to(x.dtype).float()
            self.sin_cached = self.sin_cached.to(x.dtype).float()
            self._rounded_for = x.dtype
        return self.cos_cached[:seq_len], self.sin_cached[:seq_len]
