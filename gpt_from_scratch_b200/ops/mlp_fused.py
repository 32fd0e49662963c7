"""SwiGLU MLP with the activation folded into the GEMM epilogues (csrc/gemm.cu, swi_mode).

Forward: the gate|up projection GEMM pairs every 128 gate columns with the matching up
columns in one tile and writes ``act = silu(gate) * up`` next to the projection, so the
separate activation kernel and its re-read of the ``[tokens, 2I]`` buffer disappear.
Backward: the down projection's dgrad GEMM never materialises ``d_act``: its epilogue
reads gate/up and writes ``d_gate | d_up`` directly.

Reference counterpart: core/mlp.py:22-33 (two linears, chunk, silu, mul as separate
kernels plus their autograd mirrors).
"""
from __future__ import annotations

import torch

from . import _lib
from . import gemm as gemm_ops


def _pair_eligible(M: int, I: int, cols_per_tile: int) -> bool:
    """Enough 256-row tiles for the CTA-pair kernel (``cols_per_tile``: columns of I covered by
    one tile, 128 forward / 256 backward)."""
    tiles = ((M + 255) // 256) * ((I + cols_per_tile - 1) // cols_per_tile)
    return gemm_ops._PAIR_ENABLED and tiles >= gemm_ops._PAIR_MIN_TILES


def _swiglu_entry(M: int, I: int, cols_per_tile: int):
    if _pair_eligible(M, I, cols_per_tile):
        return _lib.lib().gfs_gemm2_bf16_swiglu
    return _lib.lib().gfs_gemm_bf16_swiglu


def swiglu_gemm_fwd(x2d: torch.Tensor, w_gu: torch.Tensor):
    """Returns ``(gu [M, 2I], act [M, I])``."""
    M, K = x2d.shape
    I = w_gu.shape[0] // 2
    gu = torch.empty((M, 2 * I), dtype=torch.bfloat16, device=x2d.device)
    act = torch.empty((M, I), dtype=torch.bfloat16, device=x2d.device)
    fn = _swiglu_entry(M, I, 128)
    rc = fn(1, x2d.data_ptr(), w_gu.data_ptr(), gu.data_ptr(), act.data_ptr(), M, I, K,
            x2d.stride(0), w_gu.stride(0), gu.stride(0), act.stride(0), _lib.stream_ptr())
    _lib.check(rc, "gfs_gemm_bf16_swiglu(fwd)")
    return gu, act


def swiglu_gemm_bwd(dy2d: torch.Tensor, w_down: torch.Tensor, gu: torch.Tensor) -> torch.Tensor:
    """``d_gu [M, 2I]`` from ``dy [M, H]``, ``w_down [H, I]`` and the saved projection ``gu``."""
    M, H = dy2d.shape
    I = w_down.shape[1]
    dgu = torch.empty_like(gu)
    fn = _swiglu_entry(M, I, 256)
    rc = fn(2, dy2d.data_ptr(), w_down.data_ptr(), dgu.data_ptr(), gu.data_ptr(), M, I,
            H, dy2d.stride(0), w_down.stride(0), dgu.stride(0), gu.stride(0), _lib.stream_ptr())
    _lib.check(rc, "gfs_gemm_bf16_swiglu(bwd)")
    return dgu


class _FusedMLP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_gu, w_down, residual, sink_gu, sink_down):
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        with _lib.nvtx("fused:gemm_swiglu_fwd"):
            gu, act = swiglu_gemm_fwd(x2, w_gu)
        res2 = residual.reshape(-1, w_down.shape[0]) if residual is not None else None
        out = gemm_ops.linear_fwd(act, w_down, res2)
        ctx.save_for_backward(x2, gu, act, w_gu, w_down)
        ctx.sinks = (sink_gu, sink_down)
        ctx.has_res = residual is not None
        ctx.in_shape = x.shape
        return out.view(*x.shape[:-1], w_down.shape[0])

    @staticmethod
    def backward(ctx, dout):
        x2, gu, act, w_gu, w_down = ctx.saved_tensors
        sink_gu, sink_down = ctx.sinks
        d2 = dout.reshape(-1, w_down.shape[0])
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        if x2.shape[-1] >= MIN_HIDDEN_FOR_BWD_FUSION or _pair_eligible(d2.shape[0], gu.shape[1] // 2, 256):
            with _lib.nvtx("fused:gemm_swiglu_bwd"):
                dgu = swiglu_gemm_bwd(d2, w_down, gu)
        else:
            # short contraction: the plain dgrad GEMM + the SwiGLU backward kernel are faster
            dact = gemm_ops.linear_dgrad(d2, w_down)
            dgu = torch.empty_like(gu)
            rc = _lib.lib().gfs_swiglu_bwd(dact.data_ptr(), gu.data_ptr(), dgu.data_ptr(), gu.shape[0],
                                           gu.shape[1] // 2, _lib.stream_ptr())
            _lib.check(rc, "gfs_swiglu_bwd")
        dw_down = dw_gu = None
        if sink_down is not None:
            gemm_ops.linear_wgrad_to_sink(d2, act, sink_down)
        else:
            dw_down = gemm_ops.linear_wgrad(d2, act)
        dx = gemm_ops.linear_dgrad(dgu, w_gu).view(ctx.in_shape)
        if sink_gu is not None:
            gemm_ops.linear_wgrad_to_sink(dgu, x2, sink_gu)
        else:
            dw_gu = gemm_ops.linear_wgrad(dgu, x2)
        return dx, dw_gu, dw_down, (dout if ctx.has_res else None), None, None


# The forward fusion pays at every size (hidden 768, 16384 rows: 132 us on CTA pairs vs 106 + 50 us
# unfused). In the backward the epilogue has to fetch gate/up and do twice the math: on CTA pairs
# (8 epilogue warps) it still wins (126 us vs 61 + 80 us); on the single-CTA kernel with a short
# contraction (K = hidden) it does not (155 us), so there it is only used from this hidden size up.
MIN_HIDDEN_FOR_BWD_FUSION = 2048


def fused_mlp_supported(x: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor) -> bool:
    return (x.is_cuda and x.dtype == w_gu.dtype == w_down.dtype == torch.bfloat16 and
            x.shape[-1] % 8 == 0 and (w_gu.shape[0] // 2) % 8 == 0 and w_down.shape[0] % 8 == 0)
