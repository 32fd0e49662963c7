"""GPT model assembly. Reference: core/models/gpt.py:10-35 - vocab-parallel embedding,
``num_layers`` transformer blocks, final RMSNorm, and an LM head that is a bias-free
ColumnParallelLinear **untied** from the embedding. ``forward(inputs[B, S])`` returns
vocab-parallel logits ``[S, B, V/P]``."""
from __future__ import annotations

import torch.nn as nn

from ..parallel.layers import ColumnParallelLinear, VocabParallelEmbedding, reset_init_salts
from .init import get_init_method
from .normalization import RMSNorm
from .transformer_layer import TransformerLayer


class GPTModel(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        reset_init_salts()
        init_method = get_init_method(config)
        self.embedding = VocabParallelEmbedding(config.vocab_size, config.hidden_size, init_method=init_method)
        self.layers = nn.ModuleList([TransformerLayer(i, config) for i in range(config.num_layers)])
        self.final_norm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.output = ColumnParallelLinear(config.hidden_size, config.vocab_size, bias=False,
                                           init_method=init_method)

    def forward(self, inputs, return_ce_stats: bool = False):
        """``return_ce_stats=True`` returns ``(logits, partials)``: the LM head's GEMM epilogue also
        emits the softmax statistics the loss needs (``None`` on paths without that epilogue)."""
        hidden = self.embedding(inputs)            # [S/P, B, H]
        for layer in self.layers:
            hidden = layer(hidden)
        hidden = self.final_norm(hidden)
        if return_ce_stats:
            return self.output(hidden, ce_stats=True)
        return self.output(hidden)                 # [S, B, V/P]
