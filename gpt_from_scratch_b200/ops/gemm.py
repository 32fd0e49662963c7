"""bf16 GEMMs of a linear layer (forward, dgrad, wgrad) on the tcgen05 kernel.

On CUDA bf16 tensors the three products run on ``gfs_gemm_bf16`` (csrc/gemm.cu);
on any other device/dtype they are plain ``torch.matmul`` calls so the same model
code runs in fp32 on CPU.

Counterpart in the reference: ``F.linear`` and its autograd in
core/tensor_parallel/layers.py:47,82.
"""
from __future__ import annotations

import torch

from . import _lib

import os

_WS_BYTES = 96 << 20
# CTA-pair kernel (csrc/gemm2.cu): used when the problem has at least this many 256 x 256 tiles
_PAIR_MIN_TILES = int(os.environ.get("GFS_GEMM_PAIR_MIN_TILES", "60"))
_PAIR_ENABLED = os.environ.get("GFS_GEMM_PAIR", "1") != "0"
_workspaces: dict[int, torch.Tensor] = {}


def _workspace(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _workspaces.get(idx)
    if ws is None:
        ws = torch.empty(_WS_BYTES // 4, dtype=torch.float32, device=device)
        _workspaces[idx] = ws
    return ws


def use_native(*tensors: torch.Tensor) -> bool:
    return all(t.is_cuda and t.dtype == torch.bfloat16 for t in tensors)


def _rowmajor_2d(t: torch.Tensor) -> torch.Tensor:
    """Return a 2-D tensor whose last dim is contiguous and whose pitch/base fit TMA."""
    assert t.dim() == 2
    if t.stride(1) != 1 or t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
        t = t.contiguous()
    return t


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, *, a_mn_major: bool = False, b_mn_major: bool = False,
              out: torch.Tensor | None = None, addend: torch.Tensor | None = None,
              force_split: int = 0, rope: tuple | None = None, pair: bool | None = None) -> torch.Tensor:
    """``out[M,N] = op(a) @ op(b) (+ addend)`` with fp32 accumulation.

    ``a`` is ``[M,K]`` (K-major) or ``[K,M]`` (``a_mn_major``); ``b`` is ``[N,K]``
    (K-major) or ``[K,N]`` (``b_mn_major``). ``addend`` may alias ``out``.
    ``rope = (cos, sin, rope_cols, head_dim, batch)`` rotates the first ``rope_cols`` output
    columns in the epilogue (fp32 tables ``[positions, head_dim/2]``; row ``r`` is position
    ``r // batch``).
    """
    a = _rowmajor_2d(a)
    b = _rowmajor_2d(b)
    if a_mn_major:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn_major:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, (a.shape, b.shape, a_mn_major, b_mn_major)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    assert out.shape == (M, N) and out.stride(1) == 1
    if pair is None:
        pair = (_PAIR_ENABLED and force_split == 0 and K >= 256 and
                ((M + 255) // 256) * ((N + 255) // 256) >= _PAIR_MIN_TILES)
    if pair:
        if rope is not None:
            cos, sin, rope_cols, head_dim, batch = rope
            rargs = (cos.data_ptr(), sin.data_ptr(), rope_cols, head_dim, batch)
        else:
            rargs = (0, 0, 0, 0, 1)
        rc = _lib.lib().gfs_gemm2_bf16(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), _lib.ptr(addend), M, N, K, a.stride(0), b.stride(0),
            out.stride(0), addend.stride(0) if addend is not None else 0,
            1 if a_mn_major else 0, 1 if b_mn_major else 0, *rargs, _lib.stream_ptr())
        _lib.check(rc, "gfs_gemm2_bf16")
        return out
    ws = _workspace(a.device)
    if rope is None:
        rc = _lib.lib().gfs_gemm_bf16(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), _lib.ptr(addend),
            M, N, K, a.stride(0), b.stride(0), out.stride(0),
            addend.stride(0) if addend is not None else 0,
            1 if a_mn_major else 0, 1 if b_mn_major else 0, 1 if addend is not None else 0,
            ws.data_ptr(), ws.numel() * 4, force_split, _lib.stream_ptr())
    else:
        cos, sin, rope_cols, head_dim, batch = rope
        assert cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
        assert cos.shape[1] == head_dim // 2 and cos.shape[0] * batch >= M
        rc = _lib.lib().gfs_gemm_bf16_rope(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), _lib.ptr(addend),
            M, N, K, a.stride(0), b.stride(0), out.stride(0),
            addend.stride(0) if addend is not None else 0,
            1 if a_mn_major else 0, 1 if b_mn_major else 0, 1 if addend is not None else 0,
            ws.data_ptr(), ws.numel() * 4, force_split, cos.data_ptr(), sin.data_ptr(), rope_cols, head_dim, batch,
            _lib.stream_ptr())
    _lib.check(rc, "gfs_gemm_bf16")
    return out


def linear_fwd(x2d: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None = None,
               out: torch.Tensor | None = None, rope: tuple | None = None) -> torch.Tensor:
    """``x2d[M,K] @ w[N,K]^T (+ residual[M,N])``; ``rope`` only on the native path."""
    if use_native(x2d, w):
        return gemm_bf16(x2d, w, out=out, addend=residual, rope=rope)
    assert rope is None, "the rotary epilogue exists only in the native GEMM"
    y = x2d @ w.t()
    if residual is not None:
        y = y + residual
    if out is not None:
        out.copy_(y)
        return out
    return y


def linear_dgrad(dy2d: torch.Tensor, w: torch.Tensor, addend: torch.Tensor | None = None,
                 out: torch.Tensor | None = None) -> torch.Tensor:
    """``dy2d[M,N] @ w[N,K] (+ addend[M,K])``."""
    if use_native(dy2d, w):
        return gemm_bf16(dy2d, w, b_mn_major=True, out=out, addend=addend)
    dx = dy2d @ w
    if addend is not None:
        dx = dx + addend
    if out is not None:
        out.copy_(dx)
        return out
    return dx


def linear_wgrad(dy2d: torch.Tensor, x2d: torch.Tensor, out: torch.Tensor | None = None,
                 accumulate: bool = False) -> torch.Tensor:
    """``dy2d[M,N]^T @ x2d[M,K]`` -> ``[N,K]``; written or accumulated into ``out``."""
    if use_native(dy2d, x2d) and (out is None or use_native(out)):
        return gemm_bf16(dy2d, x2d, a_mn_major=True, b_mn_major=True, out=out,
                         addend=out if (accumulate and out is not None) else None)
    dw = dy2d.t() @ x2d
    if out is not None:
        if accumulate:
            out.add_(dw)
        else:
            out.copy_(dw)
        return out
    return dw
