"""Causal flash attention (tcgen05 kernels in csrc/attention.cu) and its torch oracle.

Two entry points:

* :func:`apply_flash_attn` - the reference's public API (core/myFlashAttn.py:1321):
  ``q, k, v`` of shape ``[B, nh, S, D]`` -> ``[B, nh, S, D]``.
* :func:`fused_rope_attention` - what the model uses: takes the packed projection
  output ``[S*B, 3*nh*D]`` (row order ``[q|k|v] x heads x D``, the reference's layout,
  core/transformer_layer.py:42-44), rotates q and k in place, and runs attention
  straight out of that buffer, producing ``[S*B, nh*D]``. This removes the four
  permute/contiguous copies per layer that the reference pays
  (core/transformer_layer.py:52-61, core/myFlashAttn.py:206-208).
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _lib
from .rope import rope_inplace_native, rope_reference


def attention_reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
                        scale: float | None = None) -> torch.Tensor:
    """Eager attention on ``[B, nh, S, D]`` tensors (materialises the S x S matrix)."""
    D = q.shape[-1]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * scale
    if causal:
        S = q.shape[-2]
        mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, v.float()).to(q.dtype)


def _strides3(t: torch.Tensor) -> tuple[int, int, int]:
    assert t.dim() == 4 and t.stride(3) == 1, "need a [S,B,nh,D] view with contiguous head_dim"
    return t.stride(0), t.stride(1), t.stride(2)


def _pad128(S: int) -> int:
    return (S + 127) // 128 * 128


def flash_fwd_native(q, k, v, out, causal: bool, scale: float) -> torch.Tensor:
    """q, k, v, out: logical ``[S, B, nh, D]`` views (any strides, head_dim contiguous). Returns LSE."""
    S, B, nh, D = q.shape
    lse = torch.empty((B, nh, _pad128(S)), dtype=torch.float32, device=q.device)
    st = (ctypes.c_longlong * 12)(*_strides3(q), *_strides3(k), *_strides3(v), *_strides3(out))
    with _lib.nvtx("flash_attention_fwd"):
        rc = _lib.lib().gfs_flash_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                      S, B, nh, D, st, scale, 1 if causal else 0, _lib.stream_ptr())
    _lib.check(rc, "gfs_flash_fwd")
    return lse


def flash_bwd_native(q, k, v, out, dout, lse, dq, dk, dv, causal: bool, scale: float, rope=None) -> None:
    """``rope = (cos, sin)``: dq and dk are rotated back (inverse RoPE) as they are written."""
    S, B, nh, D = q.shape
    # scratch of the pre-pass: dvec = rowsum(dO * O), then a copy of lse scaled by log2(e)
    dvec = torch.empty((2,) + tuple(lse.shape), dtype=torch.float32, device=lse.device)
    st = (ctypes.c_longlong * 24)(*_strides3(q), *_strides3(k), *_strides3(v), *_strides3(out), *_strides3(dout),
                                  *_strides3(dq), *_strides3(dk), *_strides3(dv))
    rc = _lib.lib().gfs_flash_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(),
                                  lse.data_ptr(), dvec.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                  S, B, nh, D, st, scale, 1 if causal else 0,
                                  rope[0].data_ptr() if rope else 0, rope[1].data_ptr() if rope else 0,
                                  _lib.stream_ptr())
    _lib.check(rc, "gfs_flash_bwd")
    _lib.add_launches(2)  # pre-pass + two main kernels


def _native_ok(*ts: torch.Tensor) -> bool:
    return all(t.is_cuda and t.dtype == torch.bfloat16 for t in ts) and ts[0].shape[-1] in (64, 128)


class _FlashAttnBHSD(torch.autograd.Function):
    """[B, nh, S, D] API on the native kernels."""

    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        qv, kv, vv = (t.permute(2, 0, 1, 3) for t in (q, k, v))
        out = torch.empty_like(q)
        lse = flash_fwd_native(qv, kv, vv, out.permute(2, 0, 1, 3), causal, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal, ctx.scale = causal, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        if dout.stride(-1) != 1:
            dout = dout.contiguous()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        pm = lambda t: t.permute(2, 0, 1, 3)  # noqa: E731
        flash_bwd_native(pm(q), pm(k), pm(v), pm(out), pm(dout), lse, pm(dq), pm(dk), pm(dv), ctx.causal, ctx.scale)
        return dq, dk, dv, None, None


def apply_flash_attn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal_mask: bool = True) -> torch.Tensor:
    """Flash attention on ``[B, nh, S, D]`` tensors (reference API, core/myFlashAttn.py:1321)."""
    scale = 1.0 / math.sqrt(q.shape[-1])
    if (q.is_cuda and q.dtype == k.dtype == v.dtype == torch.float16 and q.shape[-1] in (64, 128)):
        # the kernels are bf16: fp16 inputs (the dtype of the reference's self-test,
        # core/myFlashAttn.py:28-32) are rounded to bf16, run natively and the result is cast back;
        # this keeps 8 of fp16's 11 significand bits, within the self-test's tolerances
        o = apply_flash_attn(q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16), causal_mask)
        return o.to(torch.float16)
    if q.is_cuda and q.dtype in (torch.float16, torch.bfloat16) and q.shape[-1] not in (64, 128):
        raise ValueError(f"apply_flash_attn: head_dim {q.shape[-1]} has no native kernel (64 and 128 do); "
                         "use attention_reference for other sizes")
    if _native_ok(q, k, v):
        fix = lambda t: t if t.stride(-1) == 1 else t.contiguous()  # noqa: E731
        return _FlashAttnBHSD.apply(fix(q), fix(k), fix(v), bool(causal_mask), scale)
    return attention_reference(q, k, v, causal_mask, scale)


class _FusedRopeAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv2d, cos, sin, S, B, nh, D, pre_rotated):
        qkv = qkv2d.view(S, B, 3, nh, D)
        if not pre_rotated:
            rope_inplace_native(qkv, cos, sin, S, B, nh, D, parts=2, token_stride=3 * nh * D, backward=False)
        out = torch.empty((S, B, nh, D), dtype=qkv2d.dtype, device=qkv2d.device)
        scale = 1.0 / math.sqrt(D)
        lse = flash_fwd_native(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], out, True, scale)
        ctx.save_for_backward(qkv2d, out, lse, cos, sin)
        ctx.dims = (S, B, nh, D, scale)
        return out.view(S * B, nh * D)

    @staticmethod
    def backward(ctx, dout2d):
        qkv2d, out, lse, cos, sin = ctx.saved_tensors
        S, B, nh, D, scale = ctx.dims
        qkv = qkv2d.view(S, B, 3, nh, D)
        dout = dout2d.contiguous().view(S, B, nh, D)
        dqkv = torch.empty_like(qkv)
        # the inverse rotation of dq / dk happens in the backward kernels' epilogues
        flash_bwd_native(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], out, dout, lse,
                         dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2], True, scale, rope=(cos, sin))
        return dqkv.view(S * B, 3 * nh * D), None, None, None, None, None, None, None


def fused_rope_attention(qkv2d: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, S: int, B: int, nh: int,
                         D: int, pre_rotated: bool = False) -> torch.Tensor:
    """RoPE on q,k + causal attention from the packed ``[S*B, 3*nh*D]`` projection output.

    ``cos``/``sin`` are fp32 ``[>=S, D/2]`` tables. On CUDA bf16 the input buffer is
    rotated in place (it is an intermediate owned by the caller's projection), unless
    ``pre_rotated`` says the producing GEMM already rotated q and k in its epilogue; either
    way the returned gradient is w.r.t. the un-rotated projection output.
    """
    if qkv2d.is_cuda and qkv2d.dtype == torch.bfloat16 and D in (64, 128):
        return _FusedRopeAttention.apply(qkv2d.contiguous(), cos, sin, S, B, nh, D, pre_rotated)
    assert not pre_rotated, "pre_rotated inputs exist only on the native path"
    qkv = qkv2d.view(S, B, 3, nh, D)
    q, k, v = qkv.unbind(2)
    q = rope_reference(q, cos[:S], sin[:S])
    k = rope_reference(k, cos[:S], sin[:S])
    o = attention_reference(q.permute(1, 2, 0, 3), k.permute(1, 2, 0, 3), v.permute(1, 2, 0, 3), True)
    return o.permute(2, 0, 1, 3).reshape(S * B, nh * D)
