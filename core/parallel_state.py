from gpt_from_scratch_b200.parallel.parallel_state import *  # noqa: F401,F403
from gpt_from_scratch_b200.parallel.parallel_state import (destroy_model_parallel, get_data_parallel_group,  # noqa: F401
                                                           get_data_parallel_group_rank,
                                                           get_data_parallel_world_size,
                                                           get_tensor_model_parallel_group,
                                                           get_tensor_model_parallel_group_rank,
                                                           get_tensor_model_parallel_world_size,
                                                           initialize_parallel_state)
