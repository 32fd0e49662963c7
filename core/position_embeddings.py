from gpt_from_scratch_b200.models.position_embeddings import RotaryEmbedding  # noqa: F401
