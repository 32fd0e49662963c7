"""Parallel state, sequence/tensor-parallel mappings, TP layers and the vocab-parallel loss."""
from .layers import ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding, normal_init  # noqa: F401
from .loss import _VocabParallelCrossEntropy, vocab_parallel_cross_entropy  # noqa: F401
from .mappings import (gather_from_sequence_parallel_region, reduce_scatter_to_sequence_parallel_region,  # noqa: F401
                       scatter_to_sequence_parallel_region)
from .parallel_state import (destroy_model_parallel, get_data_parallel_group, get_data_parallel_group_rank,  # noqa: F401
                             get_data_parallel_world_size, get_tensor_model_parallel_group,
                             get_tensor_model_parallel_group_rank, get_tensor_model_parallel_world_size,
                             initialize_parallel_state)
