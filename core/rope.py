from gpt_from_scratch_b200.ops.rope import apply_rope, apply_rope_qk  # noqa: F401
