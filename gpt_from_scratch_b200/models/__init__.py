from .gpt import GPTModel  # noqa: F401
from .mlp import ParallelMLP  # noqa: F401
from .normalization import RMSNorm  # noqa: F401
from .position_embeddings import RotaryEmbedding  # noqa: F401
from .transformer_layer import ParallelAttention, TransformerLayer  # noqa: F401
