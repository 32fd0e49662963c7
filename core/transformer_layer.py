from gpt_from_scratch_b200.models.transformer_layer import ParallelAttention, TransformerLayer  # noqa: F401
