"""Single-GPU operators: sm_100a kernels with PyTorch reference implementations for CPU."""
from .attention import apply_flash_attn, attention_reference, fused_rope_attention  # noqa: F401
from .gemm import gemm_bf16, linear_dgrad, linear_fwd, linear_wgrad  # noqa: F401
from .rmsnorm import rmsnorm, rmsnorm_reference  # noqa: F401
from .rope import apply_rope, apply_rope_qk, rope_reference  # noqa: F401
from .swiglu import swiglu, swiglu_reference  # noqa: F401
