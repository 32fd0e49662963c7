from gpt_from_scratch_b200.parallel.layers import (ColumnParallelLinear, RowParallelLinear,  # noqa: F401
                                                   VocabParallelEmbedding)
