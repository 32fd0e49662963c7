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


_sort_streams: dict[int, torch.cuda.Stream] = {}


class SortedIds:
    """Token ids of one micro-batch sorted for the embedding backward (keys, shift) plus the event
    that marks the end of the sort, which runs on a side stream."""
    __slots__ = ("keys", "shift", "event")

    def __init__(self, keys, shift, event):
        self.keys, self.shift, self.event = keys, shift, event


def sort_ids_async(ids_bs: torch.Tensor, v0: int, v1: int) -> SortedIds | None:
    """Start sorting ``ids_bs`` (``[B, S]`` int64 on the GPU) for :func:`embedding_bwd_native` on a
    side stream: the sort needs only the ids, so launched from the forward pass it is finished long
    before the backward pass wants it (one CTA of this library, no library sort). ``None`` when the
    batch is too large for it (the backward then sorts with ``torch.sort``)."""
    B, S = ids_bs.shape
    dev = ids_bs.device
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    side = _sort_streams.get(idx)
    if side is None:
        side = _sort_streams[idx] = torch.cuda.Stream(dev)
    keys = torch.empty(S * B, dtype=torch.int32, device=dev)
    main = torch.cuda.current_stream(dev)
    side.wait_stream(main)                       # the ids (and the key buffer) are ready on the main stream
    with torch.cuda.stream(side):
        rc = _lib.lib().gfs_embedding_sort_keys(ids_bs.data_ptr(), keys.data_ptr(), B, S, v0, v1, _lib.stream_ptr())
        if rc == -20:
            return None
        if rc <= 0:
            _lib.check(rc if rc < 0 else -1, "gfs_embedding_sort_keys")
        _lib.add_launches(1)
        ev = torch.cuda.Event()
        ev.record(side)
    keys.record_stream(side)
    return SortedIds(keys, rc, ev)


def embedding_bwd_native(ids_bs: torch.Tensor, dout_sbh: torch.Tensor, dweight: torch.Tensor, v0: int, v1: int,
                         accumulate: bool, sorted_ids: SortedIds | None = None) -> None:
    """``dweight[id - v0] (+)= sum over tokens with that id of dout[s, b]``; dout covers the full sequence.
    ``sorted_ids``: result of :func:`sort_ids_async` for the same ids and vocabulary range."""
    B, S = ids_bs.shape
    H = dweight.shape[1]
    if not accumulate:
        dweight.zero_()
    if sorted_ids is None:
        sorted_ids = sort_ids_async(ids_bs, v0, v1)
    if sorted_ids is not None:
        torch.cuda.current_stream(dweight.device).wait_event(sorted_ids.event)
        rc = _lib.lib().gfs_embedding_bwd_keys(sorted_ids.keys.data_ptr(), dout_sbh.data_ptr(), dweight.data_ptr(),
                                               S * B, H, sorted_ids.shift, _lib.stream_ptr())
        _lib.check(rc, "gfs_embedding_bwd_keys")
        return
    flat = ids_bs.t().reshape(-1)  # [S*B] in dout row order
    sorted_ids, perm = torch.sort(flat, stable=True)
    rc = _lib.lib().gfs_embedding_bwd(sorted_ids.data_ptr(), perm.data_ptr(), dout_sbh.data_ptr(),
                                      dweight.data_ptr(), S * B, H, v0, v1, _lib.stream_ptr())
    _lib.check(rc, "gfs_embedding_bwd")
