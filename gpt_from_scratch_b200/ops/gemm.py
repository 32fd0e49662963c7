"""bf16 GEMMs of a linear layer (forward, dgrad, wgrad) on the tcgen05 kernel.

On CUDA bf16 tensors the three products run on ``gfs_gemm_bf16`` (csrc/gemm.cu);
on any other device/dtype they are plain ``torch.matmul`` calls so the same model
code runs in fp32 on CPU.

Counterpart in the reference: ``F.linear`` and its autograd in
core/tensor_parallel/layers.py:47,82.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib

_WS_BYTES = 96 << 20
# CTA-pair kernel (csrc/gemm2.cu): used when the problem has at least this many 256 x 256 tiles
_PAIR_MIN_TILES = int(os.environ.get("GFS_GEMM_PAIR_MIN_TILES", "60"))
_PAIR_ENABLED = os.environ.get("GFS_GEMM_PAIR", "1") != "0"
_workspaces: dict[int, torch.Tensor] = {}


class pair_min_tiles:
    """``with pair_min_tiles(n):`` every kernel-selection rule inside the block uses ``n`` as the
    number of 256 x 256 tiles from which a problem goes to the CTA-pair kernel (``1``: always when
    eligible; a huge value: never). For tests and microbenchmarks that want a particular kernel on
    a small problem; all ranks of a group must use the same value. ``None`` changes nothing."""

    def __init__(self, n: int | None):
        self.n = n

    def __enter__(self):
        global _PAIR_MIN_TILES
        self.saved = _PAIR_MIN_TILES
        if self.n is not None:
            _PAIR_MIN_TILES = int(self.n)
        return self

    def __exit__(self, *exc):
        global _PAIR_MIN_TILES
        _PAIR_MIN_TILES = self.saved
        return False


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


def linear_fwd_ce(x2d: torch.Tensor, w: torch.Tensor):
    """LM head: ``(x2d @ w^T, partials)`` where ``partials`` (fp32 ``[parts, M, 2]``) holds the
    online-softmax statistics of every 128-column slice of each row of the bf16 logits, produced by
    the GEMM epilogue; ``None`` when the problem does not run on the CTA-pair kernel."""
    M, K = x2d.shape
    N = w.shape[0]
    if (_CE_EPILOGUE and use_native(x2d, w) and _PAIR_ENABLED and K >= 256 and N % 8 == 0 and
            ((M + 255) // 256) * ((N + 255) // 256) >= _PAIR_MIN_TILES):
        a, b = _rowmajor_2d(x2d), _rowmajor_2d(w)
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
        parts = _lib.lib().gfs_gemm2_ce_parts(N)
        partials = torch.empty((parts, M, 2), dtype=torch.float32, device=a.device)
        rc = _lib.lib().gfs_gemm2_bf16_ce(a.data_ptr(), b.data_ptr(), out.data_ptr(), partials.data_ptr(), M, N, K,
                                          a.stride(0), b.stride(0), out.stride(0), _lib.stream_ptr())
        if rc != -20:
            _lib.check(rc, "gfs_gemm2_bf16_ce")
            return out, partials
    return linear_fwd(x2d, w), None


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


class _WgradQueue:
    """Weight-gradient GEMMs waiting to be launched together.

    A layer's weight gradients are ``[out, in] = dY^T X`` with K = tokens: few output tiles,
    very deep. One at a time they occupy a fraction of the SMs (or need split-K and a
    reduction pass); several of them in ONE grouped launch (``gfs_gemm2_wgrad_grouped``) fill
    a wave of CTA pairs. A weight gradient is only needed at the optimizer step, so problems
    that write into a gradient sink are parked here (holding references to their operands)
    and launched when enough tiles have accumulated, at the end of the backward pass that
    parked them (an autograd-engine callback), or when :func:`flush_wgrad` is called.
    """

    MAX_GROUP = 4

    def __init__(self):
        self.items: list[tuple] = []
        self.tiles = 0
        self._callback_pending = False

    def _end_of_backward(self) -> None:
        self._callback_pending = False
        self.flush()

    @staticmethod
    def tiles_of(M: int, N: int) -> int:
        return ((M + 255) // 256) * ((N + 255) // 256)

    def push(self, dy2d, x2d, out, accumulate, done_cb) -> None:
        self.items.append((dy2d, x2d, out, accumulate, done_cb))
        self.tiles += self.tiles_of(dy2d.shape[1], x2d.shape[1])
        if not self._callback_pending:
            # whatever is still parked when this backward pass ends is launched then, so every
            # ``.grad`` is complete when ``backward()`` returns
            try:
                torch.autograd.Variable._execution_engine.queue_callback(self._end_of_backward)
                self._callback_pending = True
            except RuntimeError:
                pass   # not inside a backward pass: flush_wgrad() / optimizer.step() will launch it
        if len(self.items) == self.MAX_GROUP or self.tiles >= _PAIR_MIN_TILES:
            self.flush()

    def uses(self, tensor: torch.Tensor) -> bool:
        """True if a parked problem reads from ``tensor``'s memory."""
        lo = tensor.data_ptr()
        hi = lo + tensor.numel() * tensor.element_size()
        return any(lo <= it[k].data_ptr() < hi for it in self.items for k in (0, 1))

    def flush(self) -> None:
        items, self.items, self.tiles = self.items, [], 0
        if not items:
            return
        n = len(items)
        with _lib.nvtx("fused:grouped_wgrad"):
            rc = self._launch(items, n)
        _lib.check(rc, "gfs_gemm2_wgrad_grouped")
        for it in items:
            if it[4] is not None:
                it[4]()

    @staticmethod
    def _launch(items, n) -> int:
        U, I = ctypes.c_ulonglong * n, ctypes.c_int * n
        return _lib.lib().gfs_gemm2_wgrad_grouped(
            n, U(*[it[0].data_ptr() for it in items]), U(*[it[1].data_ptr() for it in items]),
            U(*[it[2].data_ptr() for it in items]), I(*[it[0].shape[1] for it in items]),
            I(*[it[1].shape[1] for it in items]), I(*[it[0].shape[0] for it in items]),
            I(*[it[0].stride(0) for it in items]), I(*[it[1].stride(0) for it in items]),
            I(*[it[2].stride(0) for it in items]), I(*[1 if it[3] else 0 for it in items]), _lib.stream_ptr())


_CE_EPILOGUE = os.environ.get("GFS_CE_EPILOGUE", "1") != "0"
_wgrad_queue = _WgradQueue()
_WGRAD_GROUPING = os.environ.get("GFS_WGRAD_GROUPING", "1") != "0"


def flush_wgrad() -> None:
    """Launch every parked weight-gradient GEMM (no-op when nothing is parked)."""
    _wgrad_queue.flush()


def flush_wgrad_if_uses(tensor: torch.Tensor) -> None:
    """Launch the parked weight-gradient GEMMs if one of them still reads ``tensor`` (call before a
    reused buffer is overwritten)."""
    if _wgrad_queue.items and _wgrad_queue.uses(tensor):
        _wgrad_queue.flush()


def linear_wgrad_to_sink(dy2d: torch.Tensor, x2d: torch.Tensor, sink) -> None:
    """Weight gradient ``dy2d^T @ x2d`` written (or accumulated) into ``sink``'s slice of the
    gradient buffer. Small problems are grouped (see :class:`_WgradQueue`); the operands must
    not be modified before :func:`flush_wgrad`."""
    out = sink.target()
    accumulate = sink.consume_accumulate()
    N_out, N_in = dy2d.shape[1], x2d.shape[1]
    if (_WGRAD_GROUPING and _PAIR_ENABLED and use_native(dy2d, x2d, out)
            and _WgradQueue.tiles_of(N_out, N_in) < _PAIR_MIN_TILES and dy2d.shape[0] >= 256
            and N_out % 8 == 0 and N_in % 8 == 0 and out.stride(1) == 1 and out.stride(0) % 8 == 0):
        _wgrad_queue.push(_rowmajor_2d(dy2d), _rowmajor_2d(x2d), out, accumulate, sink.done)
        if hasattr(sink, "parked"):
            sink.parked()
        return
    linear_wgrad(dy2d, x2d, out=out, accumulate=accumulate)
    sink.done()


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
