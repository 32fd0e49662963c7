from gpt_from_scratch_b200.parallel.mappings import (gather_from_sequence_parallel_region,  # noqa: F401
                                                     reduce_scatter_to_sequence_parallel_region,
                                                     scatter_to_sequence_parallel_region)
