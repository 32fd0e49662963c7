"""Import aliases with the reference's module paths (``core.parallel_state``,
``core.tensor_parallel.layers`` ...), re-exporting ``gpt_from_scratch_b200``."""
