"""Vocab-sharded embedding lookup kernels (csrc/elementwise.cu).

Forward writes ``out[s, b, :] = W[id - v0]`` (zero when the id belongs to another rank)
directly in sequence-first layout, replacing the reference's mask / clamp / F.embedding /
masked_fill / transpose-copy chain (core/tensor_parallel/layers.py:120-133). Backward is a
deterministic segmented sum over token ids sorted on the device (by a single-CTA bitonic sort of
this library for up to 32768 tokens per micro-batch).
"""
from __future__ import annotations

import torch

from . import _lib


def embedding_fwd_native(ids_bs: torch.Tensor, weight: torch.Tensor, v0: int, v1: int, s0: int = 0,
                         s_count: int | None = None) -> torch.Tensor:
    B, S = ids_bs.shape
    H = weight.shape[1]
    s_count = S if s_count is None else s_count
    out = torch.empty((s_count, B, H), dtype=weight.dtype, device=weight.device)
    rc = _lib.lib().gfs_embedding_fwd(ids_bs.data_ptr(), weight.data_ptr(), out.data_ptr(), B, S, H, v0, v1, s0,
                                      s_count, _lib.stream_ptr())
    _lib.check(rc, "gfs_embedding_fwd")
    return out


def embedding_bwd_native(ids_bs: torch.Tensor, dout_sbh: torch.Tensor, dweight: torch.Tensor, v0: int, v1: int,
                         accumulate: bool) -> None:
    """``dweight[id - v0] (+)= sum over tokens with that id of dout[s, b]``; dout covers the full sequence."""
    B, S = ids_bs.shape
    H = dweight.shape[1]
    if not accumulate:
        dweight.zero_()
    # up to 32768 tokens: sorted by one CTA of the library (no library sort, nothing allocated but a
    # key buffer); larger batches fall back to torch.sort
    keys = torch.empty(S * B, dtype=torch.int32, device=dweight.device)
    rc = _lib.lib().gfs_embedding_bwd_sorted(ids_bs.data_ptr(), dout_sbh.data_ptr(), dweight.data_ptr(),
                                             keys.data_ptr(), B, S, H, v0, v1, _lib.stream_ptr())
    if rc != -20:
        _lib.check(rc, "gfs_embedding_bwd_sorted")
        _lib.add_launches(1)
        return
    flat = ids_bs.t().reshape(-1)  # [S*B] in dout row order
    sorted_ids, perm = torch.sort(flat, stable=True)
    rc = _lib.lib().gfs_embedding_bwd(sorted_ids.data_ptr(), perm.data_ptr(), dout_sbh.data_ptr(),
                                      dweight.data_ptr(), S * B, H, v0, v1, _lib.stream_ptr())
    _lib.check(rc, "gfs_embedding_bwd")
