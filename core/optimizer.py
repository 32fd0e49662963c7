from gpt_from_scratch_b200.optimizer import DistributedOptimizer  # noqa: F401
