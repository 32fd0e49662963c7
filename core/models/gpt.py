from gpt_from_scratch_b200.models.gpt import GPTModel  # noqa: F401
