"""Model configuration. Field names and defaults follow the reference's ``GPTConfig``
(train.py:15-26); the extra fields select implementation details that the reference
hard-codes."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class GPTConfig:
    vocab_size: int = 50304          # GPT-2's 50257 padded so every TP size divides it
    hidden_size: int = 768
    num_layers: int = 12
    num_attention_heads: int = 12
    max_position_embeddings: int = 1024
    intermediate_size: int = 3072
    rms_norm_eps: float = 1e-5
    bias: bool = False
    dropout_prob: float = 0.0
    # --- additions ---
    rope_base: float = 10000.0
    init_method: str = "xavier_uniform"   # or "normal"
    init_std: float = 0.02
    attention_impl: str = "fused"         # "fused": tcgen05 flash attention on CUDA; "torch": eager oracle
    reference_quirks: bool = False        # reproduce reference behaviours that were fixed by default

    def flops_per_token(self, seq_len: int) -> float:
        """Forward+backward matmul FLOPs per token (causal attention counted at half)."""
        H, I, L, V = self.hidden_size, self.intermediate_size, self.num_layers, self.vocab_size
        return 3.0 * (L * (2.0 * (4 * H * H + 3 * H * I) + 2.0 * seq_len * H) + 2.0 * H * V)

    def num_parameters(self) -> int:
        H, I, L, V = self.hidden_size, self.intermediate_size, self.num_layers, self.vocab_size
        return 2 * V * H + L * (4 * H * H + 3 * H * I + 2 * H) + H
