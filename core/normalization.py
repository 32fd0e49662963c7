from gpt_from_scratch_b200.models.normalization import RMSNorm  # noqa: F401
