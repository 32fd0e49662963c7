from gpt_from_scratch_b200.data import DistributedDataset, create_distributed_dataloader  # noqa: F401
