"""Vocab-parallel cross entropy: ``_VocabParallelCrossEntropy.apply(logits[S,B,V/P],
target[S,B]) -> loss[S,B]``.

Math as in the reference (core/tensor_parallel/loss.py:9-72): global max, sum of
exponentials and the target logit are combined across the TP group; the backward is
``(softmax - onehot) * grad``. On CUDA/bf16 the local statistics come from one pass over
the logits (fp32 accumulation), the three per-token scalars of every rank are exchanged
once, and the backward rewrites the logits buffer in place. The loss is returned in fp32.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import cross_entropy as ce_ops
from . import parallel_state as ps


class _VocabParallelCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, vocab_parallel_logits, target, partials=None):
        world = ps.get_tensor_model_parallel_world_size()
        rank = ps.get_tensor_model_parallel_group_rank()
        group = ps.get_tensor_model_parallel_group()
        Vp = vocab_parallel_logits.shape[-1]
        v0 = rank * Vp
        lg = vocab_parallel_logits
        native = lg.is_cuda and lg.dtype == torch.bfloat16 and Vp % 8 == 0
        if native:
            lg2 = lg.reshape(-1, Vp)
            if lg2.stride(1) != 1 or lg2.stride(0) % 8 != 0:
                lg2 = lg2.contiguous()
            tgt = target.reshape(-1).contiguous()
            if tgt.dtype != torch.int64:
                tgt = tgt.long()
            if (partials is not None and lg2.data_ptr() == lg.data_ptr() and partials.shape[1] == lg2.shape[0]
                    and partials.device == lg2.device):
                # statistics already produced by the LM-head GEMM epilogue: no pass over the logits
                stats, lse, loss = ce_ops.ce_stats_from_partials(partials, lg2, tgt, v0, single_rank=(world == 1))
            else:
                stats, lse, loss = ce_ops.ce_local_stats(lg2, tgt, v0, single_rank=(world == 1))
            if world > 1:
                if ps.get_comm_impl() == "fused":
                    from . import fused_comm
                    lse, loss = fused_comm.ce_exchange_combine(stats)
                else:
                    stats_all = torch.empty((world, *stats.shape), dtype=stats.dtype, device=stats.device)
                    dist.all_gather_into_tensor(stats_all, stats, group=group)
                    lse, loss = ce_ops.ce_combine(stats_all)
            ctx.save_for_backward(lg2, lse, tgt)
            ctx.native = True
            ctx.v0 = v0
            ctx.shape = lg.shape
            return loss.view(target.shape)
        # ---- composition path (CPU / fp32) ----
        logits = lg.float()
        lmax = logits.max(dim=-1)[0]
        if world > 1:
            dist.all_reduce(lmax, op=dist.ReduceOp.MAX, group=group)
        logits = logits - lmax.unsqueeze(-1)
        exp_logits = logits.exp()
        sum_exp = exp_logits.sum(dim=-1)
        mask = (target >= v0) & (target < v0 + Vp)
        local_t = (target - v0).masked_fill(~mask, 0)
        tlogit = logits.gather(-1, local_t.unsqueeze(-1)).squeeze(-1).masked_fill(~mask, 0.0)
        if world > 1:
            packed = torch.stack((sum_exp, tlogit), dim=-1)
            dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
            sum_exp, tlogit = packed.unbind(-1)
        loss = sum_exp.log() - tlogit
        softmax = exp_logits / sum_exp.unsqueeze(-1)
        ctx.save_for_backward(softmax, mask, local_t)
        ctx.native = False
        ctx.out_dtype = lg.dtype
        return loss

    @staticmethod
    def backward(ctx, grad_output):
        if ctx.native:
            lg2, lse, tgt = ctx.saved_tensors
            g = grad_output.reshape(-1).float().contiguous()
            dlogits = ce_ops.ce_backward_inplace(lg2, lse, tgt, g, ctx.v0)
            return dlogits.view(ctx.shape), None, None
        softmax, mask, local_t = ctx.saved_tensors
        grad = softmax.clone()
        grad.scatter_add_(-1, local_t.unsqueeze(-1), -mask.unsqueeze(-1).to(grad.dtype))
        grad = grad * grad_output.unsqueeze(-1)
        return grad.to(ctx.out_dtype), None, None


def vocab_parallel_cross_entropy(vocab_parallel_logits: torch.Tensor, target: torch.Tensor,
                                 partials: torch.Tensor | None = None) -> torch.Tensor:
    """Public wrapper (the reference exposes only the private Function, train.py:12,180).

    ``partials``: softmax statistics of these logits produced by the LM-head GEMM epilogue
    (``GPTModel.forward(..., return_ce_stats=True)``); with them the forward makes no pass over the
    logits."""
    return _VocabParallelCrossEntropy.apply(vocab_parallel_logits, target, partials)
