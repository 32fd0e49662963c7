"""gpt_from_scratch_b200: a Blackwell-native GPT pre-training framework (TP + sequence
parallel + DP with a sharded optimizer) whose hot paths are hand-written sm_100a kernels."""
from .config import GPTConfig  # noqa: F401

__all__ = ["GPTConfig"]
__version__ = "0.1.0"
