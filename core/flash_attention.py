from gpt_from_scratch_b200.ops.attention import apply_flash_attn  # noqa: F401
