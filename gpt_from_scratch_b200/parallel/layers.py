"""Tensor-parallel building blocks: ColumnParallelLinear, RowParallelLinear,
VocabParallelEmbedding.

Constructor signatures, attribute names, weight shapes and the sequence-parallel data flow
follow the reference (core/tensor_parallel/layers.py:15-136): column-parallel layers gather
their ``[S/P, B, H]`` input along the sequence before the GEMM, row-parallel layers
reduce-scatter their output back to the sequence shard and add the bias afterwards, the
embedding looks up its vocabulary slice and reduce-scatters.

What is different is underneath: on CUDA/bf16 the GEMMs are the tcgen05 kernel, weight
gradients are written straight into the flat gradient buffer (no autograd accumulation
pass), the residual add is folded into the row-parallel GEMM epilogue, and with
``--comm-impl fused`` the gather/reduce-scatter are done by the GEMM kernels themselves
over peer memory (``fused_comm``).
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.init as init

from ..ops import gemm as gemm_ops
from ..ops.embedding import embedding_bwd_native, embedding_fwd_native, sort_ids_async
from ..ops.grad_sink import GradSink
from . import mappings
from . import parallel_state as ps


def _init_sharded(weight: torch.Tensor, init_method, salt: int) -> None:
    """Initialise a TP-sharded weight with a generator that is equal across DP replicas and
    different across TP ranks (the reference seeds nothing, so its replicas start different)."""
    gen = ps.sharded_param_generator(weight.device, salt)
    if init_method is init.xavier_uniform_:
        fan_out, fan_in = weight.shape
        bound = (6.0 / (fan_in + fan_out)) ** 0.5
        with torch.no_grad():
            weight.uniform_(-bound, bound, generator=gen)
    elif callable(init_method) and getattr(init_method, "_takes_generator", False):
        init_method(weight, gen)
    else:
        init_method(weight)


def reset_init_salts() -> None:
    """Restart the per-layer salt sequence of the weight initialisers, so that two models built
    in the same process with the same seed get identical weights."""
    ColumnParallelLinear._salt = 0
    RowParallelLinear._salt = 1000


def normal_init(std: float = 0.02):
    """``normal(0, std)`` initialiser usable as ``init_method`` (deterministic per TP rank)."""
    def fn(weight, gen):
        with torch.no_grad():
            weight.normal_(0.0, std, generator=gen)
    fn._takes_generator = True
    return fn


class _LinearFn(torch.autograd.Function):
    """``y = x @ W^T (+ residual)`` with explicit dgrad/wgrad so the weight gradient can go
    to a :class:`GradSink`."""

    @staticmethod
    def forward(ctx, x, weight, residual, sink, rope=None, ce_stats=False):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        res2 = residual.reshape(-1, weight.shape[0]) if residual is not None else None
        partials = None
        if ce_stats and residual is None and rope is None:
            y2, partials = gemm_ops.linear_fwd_ce(x2, weight)
        else:
            y2 = gemm_ops.linear_fwd(x2, weight, res2, rope=rope)
        ctx.save_for_backward(x2, weight)
        ctx.sink = sink
        ctx.has_res = residual is not None
        ctx.in_shape = x.shape
        y = y2.view(*x.shape[:-1], weight.shape[0])
        if not ce_stats:
            return y
        # second output: the softmax statistics of the logits (an empty tensor when the GEMM that
        # served the problem has no statistics epilogue); not differentiable
        if partials is None:
            partials = x2.new_empty(0, dtype=torch.float32)
        ctx.mark_non_differentiable(partials)
        return y, partials

    @staticmethod
    def backward(ctx, dy, _dpartials=None):
        x2, weight = ctx.saved_tensors
        N = weight.shape[0]
        dy2 = dy.reshape(-1, N)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm_ops.linear_dgrad(dy2, weight).view(ctx.in_shape)
        dw = None
        sink = ctx.sink
        if sink is not None:
            gemm_ops.linear_wgrad_to_sink(dy2, x2, sink)
        elif ctx.needs_input_grad[1]:
            dw = gemm_ops.linear_wgrad(dy2, x2)
        dres = dy if ctx.has_res else None
        return dx, dw, dres, None, None, None


def linear_with_sink(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor | None = None,
                     rope: tuple | None = None, ce_stats: bool = False) -> torch.Tensor:
    """``rope``: rotary epilogue of the native GEMM. Its inverse is NOT applied by this
    function's backward: the caller's next operator must return gradients w.r.t. the
    un-rotated output (the fused attention backward does).

    ``ce_stats``: the output is the LM head's logits and the return value is ``(logits, partials)``;
    when the CTA-pair GEMM serves the problem ``partials`` holds the per-row softmax statistics its
    epilogue produced (pass them to :func:`vocab_parallel_cross_entropy`, which then skips its pass
    over the logits), otherwise it is ``None``."""
    if not ce_stats:
        return _LinearFn.apply(x, weight, residual, GradSink.of(weight), rope, False)
    out, partials = _LinearFn.apply(x, weight, residual, GradSink.of(weight), rope, True)
    return out, (partials if partials.numel() else None)


class ColumnParallelLinear(nn.Module):
    """``Y = gather_S(X) W_r^T (+ b_r)``, output sharded on the feature dim."""
    _salt = 0

    def __init__(self, input_size, output_size, bias=True, init_method=init.xavier_uniform_):
        super().__init__()
        self.input_size = input_size
        self.output_size = output_size
        world = ps.get_tensor_model_parallel_world_size()
        if output_size % world != 0:
            raise ValueError(f"output_size {output_size} is not divisible by the TP size {world}")
        self.output_size_per_partition = output_size // world
        dev = ps.get_device()
        self.weight = nn.Parameter(torch.empty(self.output_size_per_partition, input_size, device=dev,
                                               dtype=torch.float32))
        if bias:
            self.bias = nn.Parameter(torch.zeros(self.output_size_per_partition, device=dev, dtype=torch.float32))
        else:
            self.register_parameter("bias", None)
        ColumnParallelLinear._salt += 1
        _init_sharded(self.weight, init_method, ColumnParallelLinear._salt)

    def forward(self, input_, rope=None, ce_stats=False):
        """``ce_stats=True`` (LM head): returns ``(logits, partials)`` where ``partials`` are the
        softmax statistics produced by the GEMM epilogue, or ``None`` when there are none."""
        world = ps.get_tensor_model_parallel_world_size()
        want = ce_stats and self.bias is None
        if world > 1 and ps.get_comm_impl() == "fused" and input_.is_cuda:
            from . import fused_comm
            out = fused_comm.allgather_linear(input_, self.weight, rope=rope, ce_stats=want)
        else:
            full = mappings.gather_from_sequence_parallel_region(input_)
            out = linear_with_sink(full, self.weight, rope=rope, ce_stats=want)
        partials = None
        if want:
            out, partials = out
        if self.bias is not None:
            out = out + self.bias
        return (out, partials) if ce_stats else out


class RowParallelLinear(nn.Module):
    """``Y = reduce_scatter_S(X_r W_r^T) (+ b)``; the bias is added after the reduction.

    ``forward(x, residual=None)``: an optional ``[S/P, B, out]`` tensor is added to the
    result (folded into the GEMM epilogue when no reduction is needed).
    """
    _salt = 1000

    def __init__(self, input_size, output_size, bias=True, init_method=init.xavier_uniform_):
        super().__init__()
        self.input_size = input_size
        self.output_size = output_size
        world = ps.get_tensor_model_parallel_world_size()
        if input_size % world != 0:
            raise ValueError(f"input_size {input_size} is not divisible by the TP size {world}")
        self.input_size_per_partition = input_size // world
        dev = ps.get_device()
        self.weight = nn.Parameter(torch.empty(output_size, self.input_size_per_partition, device=dev,
                                               dtype=torch.float32))
        if bias:
            self.bias = nn.Parameter(torch.zeros(output_size, device=dev, dtype=torch.float32))
            # added after the reduce-scatter, so every TP rank holds a copy that only sees its
            # sequence shard's gradient: the optimizer sums those over the TP group
            self.bias.tp_replicated = True
        else:
            self.register_parameter("bias", None)
        RowParallelLinear._salt += 1
        _init_sharded(self.weight, init_method, RowParallelLinear._salt)

    def forward(self, input_, residual=None):
        world = ps.get_tensor_model_parallel_world_size()
        if world == 1:
            out = linear_with_sink(input_, self.weight, residual)
        elif ps.get_comm_impl() == "fused" and input_.is_cuda:
            from . import fused_comm
            out = fused_comm.linear_reduce_scatter(input_, self.weight, residual)
        else:
            partial = linear_with_sink(input_, self.weight)
            out = mappings.reduce_scatter_to_sequence_parallel_region(partial)
            if residual is not None:
                out = out + residual
        if self.bias is not None:
            out = out + self.bias
        return out


class _EmbeddingFn(torch.autograd.Function):
    """Local vocabulary-slice lookup producing ``[S, B, H]`` (zeros for foreign ids)."""

    @staticmethod
    def forward(ctx, ids, weight, v0, v1, sink):
        ctx.save_for_backward(ids)
        ctx.meta = (v0, v1, sink, weight.shape)
        out = embedding_fwd_native(ids, weight, v0, v1)
        # the backward needs the ids sorted: start that now, on a side stream
        ctx.sorted_ids = sort_ids_async(ids, v0, v1) if weight.requires_grad else None
        return out

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        v0, v1, sink, wshape = ctx.meta
        dout = dout.contiguous()
        if sink is not None:
            embedding_bwd_native(ids, dout, sink.target(), v0, v1, accumulate=sink.consume_accumulate(),
                                 sorted_ids=ctx.sorted_ids)
            sink.done()
            return None, None, None, None, None
        dw = torch.zeros(wshape, dtype=dout.dtype, device=dout.device)
        embedding_bwd_native(ids, dout, dw, v0, v1, accumulate=True, sorted_ids=ctx.sorted_ids)
        return None, dw, None, None, None


class VocabParallelEmbedding(nn.Module):
    """Embedding table split along the vocabulary; ``forward(ids[B, S]) -> [S/P, B, H]``."""

    def __init__(self, num_embeddings, embedding_dim, init_method=init.xavier_uniform_):
        super().__init__()
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        world = ps.get_tensor_model_parallel_world_size()
        rank = ps.get_tensor_model_parallel_group_rank()
        assert num_embeddings % world == 0, "Vocab size must be divisible by tensor model parallel size"
        per = num_embeddings // world
        self.vocab_start_index = per * rank
        self.vocab_end_index = per * (rank + 1)
        self.num_embeddings_per_partition = per
        self.weight = nn.Parameter(torch.zeros(per, embedding_dim, device=ps.get_device(), dtype=torch.float32))
        _init_sharded(self.weight, init_method, 5000)

    def forward(self, input_ids):
        w = self.weight
        v0, v1 = self.vocab_start_index, self.vocab_end_index
        world = ps.get_tensor_model_parallel_world_size()
        native = w.is_cuda and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0
        if native and world > 1 and ps.get_comm_impl() == "fused":
            from . import fused_comm
            return fused_comm.embedding_reduce_scatter(input_ids, self)
        if native:
            ids = input_ids.contiguous()
            if ids.dtype != torch.int64:
                ids = ids.long()
            out = _EmbeddingFn.apply(ids, w, v0, v1, GradSink.of(w))
        else:
            mask = (input_ids >= v0) & (input_ids < v1)
            local = (input_ids - v0).masked_fill(~mask, 0)
            out = torch.nn.functional.embedding(local, w)
            out = out.masked_fill(~mask.unsqueeze(-1), 0.0)
            out = out.transpose(0, 1).contiguous()
        return mappings.reduce_scatter_to_sequence_parallel_region(out)
