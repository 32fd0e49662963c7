from gpt_from_scratch_b200.models.mlp import ParallelMLP  # noqa: F401
