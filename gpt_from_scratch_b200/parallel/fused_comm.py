"""Fused compute + collective operators (``--comm-impl fused``).

Each operator here replaces "NCCL collective, then (or after) a library kernel" of the
reference with ONE of our kernels that moves the data over peer memory while it computes:

* :func:`allgather_linear`      sequence-parallel all-gather -> GEMM   (column-parallel forward,
                                row-parallel dgrad)            csrc/gemm.cu, mode 1
* :func:`linear_reduce_scatter` GEMM -> reduce-scatter (+ residual)    (row-parallel forward,
                                column-parallel dgrad)         csrc/gemm.cu, mode 2
                                (both also on CTA pairs for large problems: csrc/gemm2.cu)
* :func:`embedding_reduce_scatter` embedding lookup written straight into the owner's
                                sequence shard                 csrc/comm.cu
* :func:`ce_exchange_combine`   cross-entropy statistics exchange + combine   csrc/comm.cu
* :class:`DataParallelComm`     gradient reduce-scatter + norm, clip + AdamW + parameter
                                all-gather                     csrc/comm.cu

Reference call sites: core/tensor_parallel/mappings.py:22,35 (N1, N2),
core/tensor_parallel/layers.py:134, core/tensor_parallel/loss.py:15,45,
core/optimizer.py:81,95,101.
"""
from __future__ import annotations

import ctypes
import math
import os

import torch

from ..ops import _lib
from ..ops import gemm as gemm_ops
from ..ops.embedding import embedding_bwd_native, sort_ids_async
from ..ops.grad_sink import GradSink
from . import parallel_state as ps
from . import symm

WAIT_NS = int(float(os.environ.get("GFS_PEER_WAIT_NS", "20e9")))
MODE_AG, MODE_RS = 1, 2


def _site_flag_ptrs(grp: symm.SymmGroup, site: symm.Site):
    cache = grp.__dict__.setdefault("_site_flag_ptrs", {})
    ptrs = cache.get(site.slot0)
    if ptrs is None:
        ptrs = (ctypes.c_ulonglong * grp.world)(*[int(grp.flag_ptrs[r]) + 4 * site.slot0 for r in range(grp.world)])
        cache[site.slot0] = ptrs
    return ptrs


def _gemm_comm(mode: int, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, residual, M: int, N: int, K: int,
               b_mn_major: bool, grp: symm.SymmGroup, buf: symm.SymmBuffer, site: symm.Site, rope=None) -> None:
    if rope is not None:
        cos, sin, rope_cols, head_dim, batch = rope
        rc_args = (cos.data_ptr(), sin.data_ptr(), rope_cols, head_dim, batch)
    else:
        rc_args = (0, 0, 0, 0, 1)
    with _lib.nvtx("fused:allgather_gemm" if mode == MODE_AG else "fused:gemm_reduce_scatter"):
        _gemm_comm_launch(mode, a, b, out, residual, M, N, K, b_mn_major, grp, buf, site, rc_args)


def _gemm_comm_launch(mode, a, b, out, residual, M, N, K, b_mn_major, grp, buf, site, rc_args) -> None:
    args = (mode, a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(), out.stride(0),
            _lib.ptr(residual), residual.stride(0) if residual is not None else 0, M, N, K, 1 if b_mn_major else 0,
            grp.world, grp.rank, buf.ptrs, _site_flag_ptrs(grp, site), ctypes.byref(site.target), *rc_args, WAIT_NS,
            _lib.stream_ptr())
    # CTA-pair kernel when the problem has enough 256 x 256 tiles (every rank takes the same
    # decision: it depends on the global shape only); -20 = not eligible, nothing launched
    if gemm_ops._PAIR_ENABLED and (M // 256) * ((N + 255) // 256) >= gemm_ops._PAIR_MIN_TILES:
        rc = _lib.lib().gfs_gemm2_bf16_comm(*args)
        if rc != -20:
            _lib.check(rc, "gfs_gemm2_bf16_comm")
            return
    rc = _lib.lib().gfs_gemm_bf16_comm(*args)
    _lib.check(rc, "gfs_gemm_bf16_comm")


_next_weight_key = 0


def _weight_site_key(weight: torch.Tensor) -> int:
    """Key of the gathered-input buffer and flag slots that belong to ``weight``'s call site.

    Symmetric allocation is collective, so every rank must derive the same sequence of keys: the
    key is a counter assigned at the weight's first use (ranks run the same program, so the
    counters agree) and stored on the tensor object. ``id(weight)`` would not do: a freed
    tensor's id can be handed to a new tensor on one rank and not on another, and the ranks
    would then disagree on whether a buffer has to be created."""
    global _next_weight_key
    key = getattr(weight, "_gfs_site_key", None)
    if key is None:
        key = _next_weight_key
        _next_weight_key += 1
        weight._gfs_site_key = key
    return key


def _check_generation(buf: symm.SymmBuffer, expected: int) -> None:
    """The gathered input of a call site lives in ONE symmetric buffer per site, kept from the
    forward to the backward for the weight gradient. A second forward through the same layer before
    the first one's backward (e.g. two micro-batches forwarded, then both backwarded) overwrites it:
    raise instead of computing a wrong gradient."""
    if buf.generation != expected:
        raise RuntimeError("fused tensor-parallel layers keep one gathered input per layer: run each forward's "
                           "backward before the next forward through the same layer (or use --comm-impl nccl)")


def _as2d(t: torch.Tensor, cols: int) -> torch.Tensor:
    t2 = t.reshape(-1, cols)
    if not t2.is_contiguous() or t2.data_ptr() % 16:
        t2 = t2.contiguous()
    return t2


def supported(rows_per_rank: int, *dims: int) -> bool:
    return rows_per_rank % 128 == 0 and all(d % 8 == 0 for d in dims)


# --------------------------------------------------------------------------- column parallel
def _allgather_gemm_ce(x2, weight, out, M, N, K, grp, gathered, site):
    """LM head: all-gather GEMM on CTA pairs whose epilogue also emits the cross-entropy statistics
    of every 128-column slice (``[parts, M, 2]`` fp32). ``None`` when the problem does not qualify
    for the CTA-pair kernel (nothing launched)."""
    if not (gemm_ops._CE_EPILOGUE and gemm_ops._PAIR_ENABLED and
            (M // 256) * ((N + 255) // 256) >= gemm_ops._PAIR_MIN_TILES and weight.stride(1) == 1):
        return None
    parts = _lib.lib().gfs_gemm2_ce_parts(N)
    partials = torch.empty((parts, M, 2), dtype=torch.float32, device=x2.device)
    with _lib.nvtx("fused:allgather_gemm_ce_stats"):
        rc = _lib.lib().gfs_gemm2_bf16_allgather_ce(
            x2.data_ptr(), x2.stride(0), weight.data_ptr(), weight.stride(0), out.data_ptr(), out.stride(0),
            partials.data_ptr(), M, N, K, grp.world, grp.rank, gathered.ptrs, _site_flag_ptrs(grp, site),
            ctypes.byref(site.target), WAIT_NS, _lib.stream_ptr())
    if rc == -20:
        return None
    _lib.check(rc, "gfs_gemm2_bf16_allgather_ce")
    return partials


class _AllGatherLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, weight, sink, rope, site_key, ce_stats=False):
        grp = symm.get_group("tp")
        K = x_shard.shape[-1]
        N = weight.shape[0]
        x2 = _as2d(x_shard, K)
        Ms = x2.shape[0]
        M = Ms * grp.world
        gathered = grp.alloc(("ag", site_key), M * K, torch.bfloat16)     # lives until backward
        site = grp.site(("ag", site_key))
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x2.device)
        partials = None
        if ce_stats and rope is None:
            partials = _allgather_gemm_ce(x2, weight, out, M, N, K, grp, gathered, site)
        if partials is None:
            _gemm_comm(MODE_AG, x2, weight, out, None, M, N, K, False, grp, gathered, site, rope)
        ctx.save_for_backward(weight)
        ctx.gathered = gathered
        gathered.generation += 1
        ctx.generation = gathered.generation
        ctx.sink = sink
        ctx.dims = (M, N, K, Ms, x_shard.shape)
        y = out.view(x_shard.shape[0] * grp.world, *x_shard.shape[1:-1], N)
        if not ce_stats:
            return y
        if partials is None:
            partials = x2.new_empty(0, dtype=torch.float32)
        ctx.mark_non_differentiable(partials)
        return y, partials

    @staticmethod
    def backward(ctx, dy, _dpartials=None):
        (weight,) = ctx.saved_tensors
        grp = symm.get_group("tp")
        M, N, K, Ms, in_shape = ctx.dims
        _check_generation(ctx.gathered, ctx.generation)
        dy2 = _as2d(dy, N)
        # dX = reduce_scatter(dY @ W): GEMM with the reduce-scatter in its epilogue
        stage, site = grp.pooled("rs", M * K, torch.bfloat16)
        dx = torch.empty((Ms, K), dtype=torch.bfloat16, device=dy2.device)
        _gemm_comm(MODE_RS, dy2, weight, dx, None, M, K, N, True, grp, stage, site)
        x_full = ctx.gathered.tensor.view(M, K)
        sink = ctx.sink
        dw = None
        if sink is not None:
            gemm_ops.linear_wgrad_to_sink(dy2, x_full, sink)     # small problems join the layer's grouped launch
        else:
            dw = gemm_ops.linear_wgrad(dy2, x_full)
        return dx.view(in_shape), dw, None, None, None, None


def allgather_linear(x_shard: torch.Tensor, weight: torch.Tensor, rope=None, ce_stats: bool = False) -> torch.Tensor:
    """``gather_S(x_shard) @ weight^T`` with the all-gather done by the GEMM kernel.

    ``ce_stats``: the output is the LM head's logits and the return value is ``(logits, partials)``;
    when the CTA-pair kernel serves the problem its epilogue also produces the per-row softmax
    statistics (the vocabulary-parallel cross entropy then makes no pass over the logits in the
    forward), otherwise ``partials`` is ``None``."""
    world = ps.get_tensor_model_parallel_world_size()
    rows = x_shard.numel() // x_shard.shape[-1]
    if not (x_shard.dtype == weight.dtype == torch.bfloat16 and supported(rows, x_shard.shape[-1], weight.shape[0])):
        from . import mappings
        from .layers import linear_with_sink
        return linear_with_sink(mappings.gather_from_sequence_parallel_region(x_shard), weight, rope=rope,
                                ce_stats=ce_stats)
    if not ce_stats:
        return _AllGatherLinear.apply(x_shard, weight, GradSink.of(weight), rope, _weight_site_key(weight), False)
    out, partials = _AllGatherLinear.apply(x_shard, weight, GradSink.of(weight), rope, _weight_site_key(weight),
                                           True)
    return out, (partials if partials.numel() else None)


# --------------------------------------------------------------------------- row parallel
class _LinearReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, residual, sink):
        grp = symm.get_group("tp")
        Kp = x.shape[-1]
        N = weight.shape[0]
        x2 = _as2d(x, Kp)
        M = x2.shape[0]
        Ms = M // grp.world
        stage, site = grp.pooled("rs", M * N, torch.bfloat16)
        out = torch.empty((Ms, N), dtype=torch.bfloat16, device=x2.device)
        res2 = _as2d(residual, N) if residual is not None else None
        _gemm_comm(MODE_RS, x2, weight, out, res2, M, N, Kp, False, grp, stage, site)
        ctx.save_for_backward(x2, weight)
        ctx.sink = sink
        ctx.has_res = residual is not None
        ctx.dims = (M, N, Kp, Ms, x.shape)
        return out.view(x.shape[0] // grp.world, *x.shape[1:-1], N)

    @staticmethod
    def backward(ctx, dout):
        x2, weight = ctx.saved_tensors
        grp = symm.get_group("tp")
        M, N, Kp, Ms, in_shape = ctx.dims
        d2 = _as2d(dout, N)
        # dX = gather_S(dOut) @ W: all-gather fused into the dgrad GEMM; the gathered dOut is
        # then reused by the wgrad GEMM (gathered once, used twice)
        gathered, site = grp.pooled("agb", M * N, torch.bfloat16)
        gemm_ops.flush_wgrad_if_uses(gathered.tensor)    # a parked weight gradient may still read this buffer
        dx = torch.empty((M, Kp), dtype=torch.bfloat16, device=d2.device)
        _gemm_comm(MODE_AG, d2, weight, dx, None, M, Kp, N, True, grp, gathered, site)
        dy_full = gathered.tensor.view(M, N)
        sink = ctx.sink
        dw = None
        if sink is not None:
            gemm_ops.linear_wgrad_to_sink(dy_full, x2, sink)
        else:
            dw = gemm_ops.linear_wgrad(dy_full, x2)
        return dx.view(in_shape), dw, (dout if ctx.has_res else None), None


def linear_reduce_scatter(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor | None = None):
    """``reduce_scatter_S(x @ weight^T) (+ residual)`` with the reduction done by the GEMM kernel."""
    world = ps.get_tensor_model_parallel_world_size()
    rows = x.numel() // x.shape[-1]
    if not (x.dtype == weight.dtype == torch.bfloat16 and rows % world == 0 and
            supported(rows // world, x.shape[-1], weight.shape[0])):
        from . import mappings
        from .layers import linear_with_sink
        out = mappings.reduce_scatter_to_sequence_parallel_region(linear_with_sink(x, weight))
        return out + residual if residual is not None else out
    return _LinearReduceScatter.apply(x, weight, residual, GradSink.of(weight))


# --------------------------------------------------------------------------- SwiGLU MLP
def _swiglu_comm(swi_mode, a, b, out, extra, M, I, K, grp, buf, site) -> None:
    with _lib.nvtx("fused:allgather_gemm_swiglu_fwd" if swi_mode == 1 else "fused:allgather_gemm_swiglu_bwd"):
        rc = _lib.lib().gfs_gemm2_bf16_comm_swiglu(
            swi_mode, a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(), out.stride(0),
            extra.data_ptr(), extra.stride(0), M, I, K, grp.world, grp.rank, buf.ptrs, _site_flag_ptrs(grp, site),
            ctypes.byref(site.target), WAIT_NS, _lib.stream_ptr())
    _lib.check(rc, "gfs_gemm2_bf16_comm_swiglu")


class _FusedCommMLP(torch.autograd.Function):
    """Tensor-parallel SwiGLU MLP on the sequence shard: all-gather -> gate|up GEMM with
    ``silu(gate) * up`` in its epilogue -> down GEMM -> reduce-scatter (+ residual). Backward:
    all-gather of dOut -> dgrad of the down projection whose epilogue applies the SwiGLU backward
    (writes d_gate | d_up), then the gate|up dgrad with its reduce-scatter; the two gathered
    buffers feed the weight gradients. No standalone activation kernel in either direction."""

    @staticmethod
    def forward(ctx, x_shard, w_gu, w_down, residual, sink_gu, sink_down, site_key):
        grp = symm.get_group("tp")
        H = x_shard.shape[-1]
        I = w_gu.shape[0] // 2
        x2 = _as2d(x_shard, H)
        Ms = x2.shape[0]
        M = Ms * grp.world
        gathered = grp.alloc(("ag", site_key), M * H, torch.bfloat16)     # lives until backward
        site = grp.site(("ag", site_key))
        gu = torch.empty((M, 2 * I), dtype=torch.bfloat16, device=x2.device)
        act = torch.empty((M, I), dtype=torch.bfloat16, device=x2.device)
        _swiglu_comm(1, x2, w_gu, gu, act, M, I, H, grp, gathered, site)
        stage, site_rs = grp.pooled("rs", M * H, torch.bfloat16)
        out = torch.empty((Ms, H), dtype=torch.bfloat16, device=x2.device)
        res2 = _as2d(residual, H) if residual is not None else None
        _gemm_comm(MODE_RS, act, w_down, out, res2, M, H, I, False, grp, stage, site_rs)
        ctx.save_for_backward(gu, act, w_gu, w_down)
        ctx.gathered = gathered
        gathered.generation += 1
        ctx.generation = gathered.generation
        ctx.sinks = (sink_gu, sink_down)
        ctx.has_res = residual is not None
        ctx.dims = (M, Ms, H, I, x_shard.shape)
        return out.view(x_shard.shape)

    @staticmethod
    def backward(ctx, dout):
        gu, act, w_gu, w_down = ctx.saved_tensors
        sink_gu, sink_down = ctx.sinks
        grp = symm.get_group("tp")
        M, Ms, H, I, in_shape = ctx.dims
        _check_generation(ctx.gathered, ctx.generation)
        d2 = _as2d(dout, H)
        # d_gu = swiglu'(gather_S(dOut) @ W_down, gu): all-gather fused into the dgrad GEMM, SwiGLU
        # backward in its epilogue; the gathered dOut then feeds the down projection's wgrad
        gathered_d, site_d = grp.pooled("agb", M * H, torch.bfloat16)
        gemm_ops.flush_wgrad_if_uses(gathered_d.tensor)
        dgu = torch.empty_like(gu)
        _swiglu_comm(2, d2, w_down, dgu, gu, M, I, H, grp, gathered_d, site_d)
        dy_full = gathered_d.tensor.view(M, H)
        dw_down = dw_gu = None
        if sink_down is not None:
            gemm_ops.linear_wgrad_to_sink(dy_full, act, sink_down)
        else:
            dw_down = gemm_ops.linear_wgrad(dy_full, act)
        # dX = reduce_scatter(d_gu @ W_gu)
        stage, site_rs = grp.pooled("rs", M * H, torch.bfloat16)
        dx = torch.empty((Ms, H), dtype=torch.bfloat16, device=d2.device)
        _gemm_comm(MODE_RS, dgu, w_gu, dx, None, M, H, 2 * I, True, grp, stage, site_rs)
        x_full = ctx.gathered.tensor.view(M, H)
        if sink_gu is not None:
            gemm_ops.linear_wgrad_to_sink(dgu, x_full, sink_gu)
        else:
            dw_gu = gemm_ops.linear_wgrad(dgu, x_full)
        return dx.view(in_shape), dw_gu, dw_down, (dout if ctx.has_res else None), None, None, None


def fused_mlp_eligible(x_shard: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor) -> bool:
    """The SwiGLU epilogues exist on the CTA-pair kernel only: rows per rank a multiple of 256 and
    enough tiles for it in both directions."""
    if not (x_shard.is_cuda and x_shard.dtype == w_gu.dtype == w_down.dtype == torch.bfloat16 and
            gemm_ops._PAIR_ENABLED):
        return False
    world = ps.get_tensor_model_parallel_world_size()
    H = x_shard.shape[-1]
    I = w_gu.shape[0] // 2
    Ms = x_shard.numel() // H
    M = Ms * world
    if Ms % 256 or H % 8 or I % 8 or H < 256 or I < 256 or w_gu.stride(1) != 1 or w_down.stride(1) != 1:
        return False
    tiles_fwd = (M // 256) * ((I + 127) // 128)
    tiles_bwd = (M // 256) * ((I + 255) // 256)
    return min(tiles_fwd, tiles_bwd) >= gemm_ops._PAIR_MIN_TILES


def swiglu_mlp(x_shard: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor, residual=None) -> torch.Tensor:
    """``reduce_scatter_S(swiglu(gather_S(x) @ w_gu^T) @ w_down^T) (+ residual)`` in two fused kernels."""
    return _FusedCommMLP.apply(x_shard, w_gu, w_down, residual, GradSink.of(w_gu), GradSink.of(w_down),
                               _weight_site_key(w_gu))


# --------------------------------------------------------------------------- generic all-gather
def allgather_rows(x2d: torch.Tensor, kind: str, group: str = "tp") -> torch.Tensor:
    """Push-style all-gather of a ``[rows, cols]`` block over a group ("tp", "dp", "world") ->
    ``[world*rows, cols]`` (a view of a pooled symmetric buffer, valid until two later calls of the
    same kind and size). The kernel moves 16-byte vectors: any dtype works as long as a row is a
    multiple of 16 bytes and starts on a 16-byte boundary."""
    grp = symm.get_group(group)
    if x2d.dtype != torch.bfloat16:
        x2d = x2d.view(torch.bfloat16)
    rows, cols = x2d.shape
    buf, site = grp.pooled(kind, grp.world * rows * cols, x2d.dtype)
    rc = _lib.lib().gfs_allgather(x2d.data_ptr(), rows, cols, x2d.stride(0), buf.ptrs, grp.flag_ptrs, grp.world,
                                  grp.rank, site.slot0, ctypes.byref(site.target), WAIT_NS, _lib.stream_ptr())
    _lib.check(rc, "gfs_allgather")
    return buf.tensor.view(grp.world * rows, cols)


def allreduce_sum_small(x: torch.Tensor, group: str) -> torch.Tensor:
    """Sum of a small fp32 vector (numel a multiple of 4) over a group, by a push all-gather and a
    sum in rank order: identical bits on every rank, no NCCL call, capturable in a CUDA graph.
    Replaces the scalar all-reduces of the reference's clipping (core/optimizer.py:101)."""
    assert x.dtype == torch.float32 and x.numel() % 4 == 0 and x.is_contiguous()
    world = symm.get_group(group).world
    every = allgather_rows(x.view(1, -1), "ar32", group=group)           # [world, 2*numel] as bf16 words
    return every.view(torch.float32).view(world, x.numel()).sum(0)


def sum_over_tp_inplace(buffer: torch.Tensor, index: torch.Tensor) -> None:
    """``buffer[index] = sum over the TP group of buffer[index]`` (gradients of parameters that are
    replicated across tensor-parallel ranks), summed in rank order on every rank."""
    vals = buffer.index_select(0, index)
    world = symm.get_group("tp").world
    every = allgather_rows(vals.view(1, -1), "repg").view(world, -1)
    buffer.index_copy_(0, index, every.float().sum(0).to(buffer.dtype))


# --------------------------------------------------------------------------- embedding
class _EmbeddingReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, v0, v1, sink):
        grp = symm.get_group("tp")
        B, S = ids.shape
        H = weight.shape[1]
        Ss = S // grp.world
        out, site = grp.pooled("emb", Ss * B * H, torch.bfloat16)
        rc = _lib.lib().gfs_embedding_scatter(ids.data_ptr(), weight.data_ptr(), B, S, H, v0, v1, out.ptrs,
                                              grp.flag_ptrs, grp.world, grp.rank, site.slot0,
                                              ctypes.byref(site.target), WAIT_NS, _lib.stream_ptr())
        _lib.check(rc, "gfs_embedding_scatter")
        ctx.save_for_backward(ids)
        ctx.meta = (v0, v1, sink, weight.shape, S, B, H)
        ctx.sorted_ids = sort_ids_async(ids, v0, v1) if weight.requires_grad else None   # for the backward
        # the result is layer 0's input and is saved for its backward, while the pooled symmetric
        # buffer is written again by the next forward: hand out a private copy (a few MB per step)
        return out.tensor.view(Ss, B, H).clone()

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        v0, v1, sink, wshape, S, B, H = ctx.meta
        full = allgather_rows(_as2d(dout, B * H), "embb").view(S, B, H)
        if sink is not None:
            embedding_bwd_native(ids, full, sink.target(), v0, v1, accumulate=sink.consume_accumulate(),
                                 sorted_ids=ctx.sorted_ids)
            sink.done()
            return None, None, None, None, None
        dw = torch.zeros(wshape, dtype=dout.dtype, device=dout.device)
        embedding_bwd_native(ids, full, dw, v0, v1, accumulate=True, sorted_ids=ctx.sorted_ids)
        return None, dw, None, None, None


def embedding_reduce_scatter(input_ids: torch.Tensor, module) -> torch.Tensor:
    """Vocab-parallel lookup + reduce-scatter along the sequence as one kernel: every rank writes
    the rows it owns directly into the output shard of the rank that owns the position."""
    ids = input_ids.contiguous()
    if ids.dtype != torch.int64:
        ids = ids.long()
    w = module.weight
    with _lib.nvtx("fused:embedding_reduce_scatter"):
        return _EmbeddingReduceScatter.apply(ids, w, module.vocab_start_index, module.vocab_end_index,
                                             GradSink.of(w))


# --------------------------------------------------------------------------- cross entropy
def ce_exchange_combine(stats: torch.Tensor):
    """stats ``[M, 3]`` (local max, sum-exp, target logit) -> global ``(lse, loss)``, each ``[M]``."""
    grp = symm.get_group("tp")
    M = stats.shape[0]
    buf = grp.alloc(("ce", M), grp.world * M * 3, torch.float32)
    site = grp.site(("ce", M))
    lse = torch.empty(M, dtype=torch.float32, device=stats.device)
    loss = torch.empty(M, dtype=torch.float32, device=stats.device)
    with _lib.nvtx("fused:ce_exchange_combine"):
        rc = _lib.lib().gfs_ce_exchange(stats.data_ptr(), lse.data_ptr(), loss.data_ptr(), M, buf.ptrs,
                                        grp.flag_ptrs, grp.world, grp.rank, site.slot0, ctypes.byref(site.target),
                                        WAIT_NS, _lib.stream_ptr())
    _lib.check(rc, "gfs_ce_exchange")
    return lse, loss


def barrier(kind: str = "tp") -> None:
    grp = symm.get_group(kind)
    site = grp.site("barrier")
    rc = _lib.lib().gfs_symm_barrier(grp.flag_ptrs, grp.world, grp.rank, site.slot0, ctypes.byref(site.target),
                                     WAIT_NS, _lib.stream_ptr())
    _lib.check(rc, "gfs_symm_barrier")


# --------------------------------------------------------------------------- data-parallel optimizer
class DataParallelComm:
    """Buffers and kernels of the distributed optimizer's collectives (csrc/comm.cu), no NCCL call
    and no host sync:

    * ``push_bucket(b)``: as soon as the backward pass has finished bucket ``b`` of the flat
      gradient buffer, every rank copies each peer's slice of it into that peer's staging buffer
      over NVLink with the copy engines (the reduce-scatter's data movement, overlapped with the
      rest of backward without taking SMs from it; nothing in it waits, so it cannot stall anything
      it shares the GPU with), then signals the owners;
    * ``sum_and_norm()``: the owner sums the staged contributions in rank order + squared norm;
    * ``adam_and_gather()``: global-norm clip + AdamW on the fp32 shard + bf16 parameters stored
      into every rank's parameter buffer.

    ``buckets``: list of ``(start, end)`` ranges of the flat buffer, each a multiple of
    ``8 * world`` long; rank ``r`` owns ``[start + r*len/world, start + (r+1)*len/world)`` of each
    and its optimizer shard is the concatenation of those slices."""

    def __init__(self, padded_numel: int, shard_size: int, device: torch.device, buckets=None):
        self.grp = symm.get_group("dp")
        g = self.grp
        buckets = buckets or [(0, padded_numel)]
        assert buckets[0][0] == 0 and buckets[-1][1] == padded_numel
        nb = len(buckets)
        self.buckets = buckets
        flat0, slices, offs = [], [], [0]
        for (a, b) in buckets:
            assert (b - a) % (8 * g.world) == 0 and b > a
            flat0.append(a)
            slices.append((b - a) // g.world)
            offs.append(offs[-1] + slices[-1])
        assert offs[-1] == shard_size
        self.nb, self.flat0, self.slices, self.offs = nb, flat0, slices, offs
        L = ctypes.c_longlong
        self._c_flat0, self._c_slice, self._c_off = (L * nb)(*flat0), (L * nb)(*slices), (L * (nb + 1))(*offs)
        self._param = g.alloc("dp:params", padded_numel, torch.bfloat16, zero=True)
        self._stage = g.alloc("dp:stage", g.world * shard_size, torch.bfloat16, zero=True)
        self._norm = g.alloc("dp:norm", 16, torch.float32, zero=True)
        self.param_buffer = self._param.tensor
        self.grad_buffer = torch.zeros(padded_numel, dtype=torch.bfloat16, device=device)   # read locally only
        self.shard_size = shard_size
        self.reduced = torch.zeros(shard_size, dtype=torch.bfloat16, device=device)
        self.norm_out = torch.zeros(1, dtype=torch.float32, device=device)
        self.scratch = torch.zeros(_lib.lib().gfs_dp_reduce_norm_scratch_floats(), dtype=torch.float32,
                                   device=device)
        self.site_push = g.site("dp:push")
        self.site_norm = g.site("dp:norm")
        self.site_param = g.site("dp:param")

    # ---- layout helpers ----
    def shard_slices(self, rank: int | None = None):
        """``(flat_start, flat_end, shard_start)`` of every slice owned by ``rank`` (default: this rank)."""
        r = self.grp.rank if rank is None else rank
        return [(f + r * s, f + (r + 1) * s, o) for f, s, o in zip(self.flat0, self.slices, self.offs)]

    def gather_shard(self, flat: torch.Tensor, rank: int | None = None) -> torch.Tensor:
        """This rank's shard of a flat-buffer-shaped tensor (copy, in shard order)."""
        return torch.cat([flat[a:b] for a, b, _ in self.shard_slices(rank)])

    def push_bucket(self, b: int) -> None:
        g = self.grp
        rc = _lib.lib().gfs_dp_push_grads(
            self.grad_buffer.data_ptr(), self._stage.ptrs, g.flag_ptrs, self.nb, self._c_flat0, self._c_slice,
            self._c_off, b, g.world, g.rank, self.site_push.slot0, ctypes.byref(self.site_push.target),
            _lib.stream_ptr())
        _lib.check(rc, "gfs_dp_push_grads")

    def sum_and_norm(self) -> None:
        g = self.grp
        rc = _lib.lib().gfs_dp_sum_norm(
            self.grad_buffer.data_ptr(), self._stage.ptrs, g.flag_ptrs, self._norm.ptrs, self.reduced.data_ptr(),
            self.nb, self._c_flat0, self._c_slice, self._c_off, g.world, g.rank, self.site_push.slot0, self.site_push.target.value, self.site_norm.slot0,
            ctypes.byref(self.site_norm.target), self.scratch.data_ptr(), WAIT_NS, _lib.stream_ptr())
        _lib.check(rc, "gfs_dp_sum_norm")

    def adam_and_gather(self, master, exp_avg, exp_avg_sq, *, step, lr, beta1, beta2, eps, weight_decay, clip,
                        grad_scale, extern_sumsq=None, step_dev=None) -> None:
        g = self.grp
        bc1 = 1.0 - beta1 ** step
        bc2_sqrt = math.sqrt(1.0 - beta2 ** step)
        rc = _lib.lib().gfs_dp_adam_gather(
            self._param.ptrs, g.flag_ptrs, self._norm.ptrs, self.reduced.data_ptr(), master.data_ptr(),
            exp_avg.data_ptr(), exp_avg_sq.data_ptr(), self.nb, self._c_flat0, self._c_slice, self._c_off, g.world,
            g.rank, self.site_norm.slot0, self.site_norm.target.value, self.site_param.slot0,
            ctypes.byref(self.site_param.target), _lib.ptr(extern_sumsq), self.norm_out.data_ptr(),
            lr, beta1, beta2, eps, weight_decay, bc1, bc2_sqrt, clip, grad_scale, _lib.ptr(step_dev), WAIT_NS,
            _lib.stream_ptr())
        _lib.check(rc, "gfs_dp_adam_gather")

    def step(self, opt, state, *, step, lr, beta1, beta2, eps, weight_decay, clip, grad_scale) -> None:
        """Everything after the pushes (the caller has pushed every bucket, on this stream or on a
        stream this one has waited for)."""
        with _lib.nvtx("fused:dp_reduce_scatter_norm"):
            self.sum_and_norm()
        if opt._rep_index_shard is not None and not opt.reference_quirks and opt._rep_index_shard.numel():
            # gradients of parameters replicated over TP (norm weights, row-parallel biases): sum this
            # shard's share of them over the TP group (commutes with the DP sum done above)
            if opt._rep_index_shard.numel() % 8 == 0:
                sum_over_tp_inplace(self.reduced, opt._rep_index_shard)
            else:
                import torch.distributed as dist
                vals = self.reduced.index_select(0, opt._rep_index_shard)
                dist.all_reduce(vals, group=ps.get_tensor_model_parallel_group())
                self.reduced.index_copy_(0, opt._rep_index_shard, vals)
        extern = None
        if opt.tp_world_size > 1 and not opt.reference_quirks and clip > 0:
            # global norm over TP x DP with replicated parameters counted once
            local = opt._sumsq
            from ..ops import adam as adam_ops
            adam_ops.sumsq_bf16(self.reduced, local[0:1])
            if opt._rep_index_shard is not None:
                local[1] = self.reduced.index_select(0, opt._rep_index_shard).float().pow(2).sum()
            else:
                local[1:2].zero_()
            extern = opt._global_sumsq(local)
        with _lib.nvtx("fused:dp_clip_adam_allgather"):
            self.adam_and_gather(opt.fp32_master_shard.data, state["exp_avg"], state["exp_avg_sq"], step=step, lr=lr,
                                 beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay, clip=clip,
                                 grad_scale=grad_scale, extern_sumsq=extern, step_dev=opt.step_dev())
