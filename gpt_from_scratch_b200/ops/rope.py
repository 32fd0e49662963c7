"""Rotary position embedding on interleaved pairs (csrc/elementwise.cu: rope_kernel).

``x'[2i] = x[2i] cos - x[2i+1] sin``, ``x'[2i+1] = x[2i] sin + x[2i+1] cos``; the backward
is the inverse rotation. Same math as the reference's Triton kernel
(core/rope_triton.py:112-133), but q and k are rotated by one launch, in place,
inside the packed qkv buffer. cos/sin are fp32 ``[S, D/2]`` tables.
"""
from __future__ import annotations

import torch

from . import _lib


def rope_reference(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: ``[S, B, nh, D]``; cos, sin: ``[S, D/2]``."""
    S = x.shape[0]
    c = cos[:S].float()[:, None, None, :]
    s = sin[:S].float()[:, None, None, :]
    xe = x[..., 0::2].float()
    xo = x[..., 1::2].float()
    out = torch.stack((xe * c - xo * s, xe * s + xo * c), dim=-1).flatten(-2)
    return out.to(x.dtype)


def rope_inplace_native(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, S: int, B: int, nh: int, D: int,
                        parts: int, token_stride: int, backward: bool, s_offset: int = 0) -> None:
    assert cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
    assert cos.shape[0] >= S + s_offset and cos.shape[1] == D // 2
    rc = _lib.lib().gfs_rope(x.data_ptr(), cos.data_ptr(), sin.data_ptr(), S, B, nh, D, parts, token_stride,
                             1 if backward else 0, s_offset, _lib.stream_ptr())
    _lib.check(rc, "gfs_rope")


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        S, B, nh, D = x.shape
        out = x.contiguous().clone()
        rope_inplace_native(out, cos, sin, S, B, nh, D, 1, nh * D, False)
        ctx.save_for_backward(cos, sin)
        return out

    @staticmethod
    def backward(ctx, g):
        cos, sin = ctx.saved_tensors
        S, B, nh, D = g.shape
        dx = g.contiguous().clone()
        rope_inplace_native(dx, cos, sin, S, B, nh, D, 1, nh * D, True)
        return dx, None, None


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate ``x [S, B, nh, D]`` (reference API: core/rope_triton.py:144)."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        return _Rope.apply(x, cos.float().contiguous(), sin.float().contiguous())
    return rope_reference(x, cos, sin)


def apply_rope_qk(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    """Rotate q and k (reference API: core/rope_triton.py:147-148)."""
    return apply_rope(q, cos, sin), apply_rope(k, cos, sin)
