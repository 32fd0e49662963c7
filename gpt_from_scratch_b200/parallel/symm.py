"""Symmetric-memory workspaces for the fused communication kernels.

A :class:`SymmGroup` wraps one process group (TP or DP). It hands out symmetric buffers
(``torch.distributed._symmetric_memory``: the same-size allocation on every rank, mapped
into every peer's address space, so a kernel can load/store a peer's copy directly over
NVLink) together with the table of all ranks' device pointers, and manages the signalling
counters: one symmetric ``uint32`` array per group out of which every call site reserves
``world`` consecutive slots, plus a host-side cumulative target per site. Counters are
never reset; a waiter compares against the target, so no reset races exist.

CUDA graphs: a captured step replays with frozen kernel arguments, so the targets cannot stay
host-side cumulative counts. Every counter therefore has a local "base" word behind the
counters (``csrc/common.cuh``); a kernel waits for ``base + target``. :func:`begin_graph_capture`
moves the counts reached so far into the base words and restarts the host counts at zero,
:func:`graph_epilogue` (called inside the capture, last) adds the step's per-site totals to the
base words, and :func:`end_graph_capture` records those totals and restarts the host counts
again. Launches made outside the graph afterwards count on the host again while the flags advance
on the device; :func:`fold_pending`, called before every replay, moves such counts into the base
words so that the captured waits keep starting from the flags' actual values.

Allocation is collective: all ranks of the group must create the same buffers in the same
order, which holds because they run the same program.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

NUM_FLAG_SLOTS = 8192      # must equal gfs_flag_slots() of the native library (checked at first use)
# Debug aid (GFS_SYMM_CANARIES=1): every symmetric buffer gets a 256-byte guard region on both
# sides, filled with a pattern; check_canaries() verifies them (the multi-GPU tests do so after
# exercising every fused kernel). Stands in for a memory checker on peer stores.
CANARIES = os.environ.get("GFS_SYMM_CANARIES", "0") == "1"
# GFS_MULTIMEM=0: never hand kernels a multicast address (they then use per-peer stores)
MULTIMEM = os.environ.get("GFS_MULTIMEM", "1") != "0"
GUARD_BYTES = 256
CANARY_BYTE = 0xA5
_groups: dict = {}


class SymmBuffer:
    __slots__ = ("tensor", "ptrs", "handle", "generation")

    def __init__(self, tensor, ptrs, handle):
        self.tensor = tensor
        self.ptrs = ptrs          # ctypes array: `world` device pointers (this rank included) + multicast address
        self.handle = handle
        self.generation = 0       # bumped by every operator that overwrites the buffer (reuse check)


class Site:
    """Flag slots + cumulative target of one call site. ``target`` is a ``c_uint`` that lives inside
    the group's target array when one is given (so "has any site counted since the last fold" is one
    vector test)."""
    __slots__ = ("slot0", "target")

    def __init__(self, slot0: int, store=None):
        self.slot0 = slot0
        self.target = ctypes.c_uint(0) if store is None else ctypes.c_uint.from_buffer(store, 4 * slot0)


class SymmGroup:
    def __init__(self, group, world: int, rank: int, device: torch.device):
        self.group = group if group is not None else dist.group.WORLD
        self.world = world
        self.rank = rank
        self.device = device
        self._buffers: dict = {}
        self._raw: dict = {}
        self._sites: dict = {}
        self._pools: dict = {}
        self._next_slot = 0
        self.has_multicast = False
        import numpy as np
        self._target_store = (ctypes.c_uint * NUM_FLAG_SLOTS)()        # Site.target objects point into it
        self._target_view = np.frombuffer(self._target_store, dtype=np.uint32)
        # counters [0, NUM_FLAG_SLOTS) + their base words [NUM_FLAG_SLOTS, 2*NUM_FLAG_SLOTS)
        flags = self.alloc("__flags__", 2 * NUM_FLAG_SLOTS, torch.int32, zero=True)
        self.flags = flags
        self.flag_ptrs = flags.ptrs
        self.base = flags.tensor[NUM_FLAG_SLOTS:]
        self.per_step = torch.zeros(NUM_FLAG_SLOTS, dtype=torch.int32, device=device)
        # make sure every rank has zeroed its flags before anyone signals
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)

    def alloc(self, name: str, numel: int, dtype: torch.dtype, zero: bool = False) -> SymmBuffer:
        import torch.distributed._symmetric_memory as symm_mem
        key = (name, numel, dtype)
        buf = self._buffers.get(key)
        if buf is not None:
            return buf
        guard = (GUARD_BYTES // dtype.itemsize) if CANARIES else 0
        raw = symm_mem.empty(numel + 2 * guard, dtype=dtype, device=self.device)
        t = raw[guard:guard + numel] if guard else raw
        if guard:
            # guard regions in front of and behind the usable range, checked by check_canaries()
            raw.view(torch.uint8)[:GUARD_BYTES].fill_(CANARY_BYTE)
            raw.view(torch.uint8)[-GUARD_BYTES:].fill_(CANARY_BYTE)
        if zero:
            t.zero_()
        handle = symm_mem.rendezvous(raw, self.group)
        off = guard * dtype.itemsize
        # entries [0, world): every rank's copy; entry [world]: the NVSwitch multicast address of the
        # same allocation (a store to it lands in every copy), 0 when the fabric offers none
        mc = int(getattr(handle, "multicast_ptr", 0) or 0) if MULTIMEM else 0
        ptrs = (ctypes.c_ulonglong * (self.world + 1))(*[int(p) + off for p in handle.buffer_ptrs],
                                                       (mc + off) if mc else 0)
        assert int(ptrs[self.rank]) == t.data_ptr()
        self.has_multicast = bool(mc)
        buf = SymmBuffer(t, ptrs, handle)
        self._buffers[key] = buf
        if guard:
            self._raw[key] = raw
        return buf

    def check_canaries(self) -> None:
        """Raise if any kernel (of any rank) wrote outside the usable range of one of this rank's
        symmetric buffers. Only meaningful with GFS_SYMM_CANARIES=1; synchronises the device."""
        torch.cuda.synchronize(self.device)
        for key, raw in self._raw.items():
            b = raw.view(torch.uint8)
            ok = bool((b[:GUARD_BYTES] == CANARY_BYTE).all()) and bool((b[-GUARD_BYTES:] == CANARY_BYTE).all())
            if not ok:
                raise RuntimeError(f"symmetric buffer {key[0]!r}: guard region overwritten on rank {self.rank}")

    def site(self, name) -> Site:
        s = self._sites.get(name)
        if s is None:
            if self._next_slot + self.world > NUM_FLAG_SLOTS:
                raise RuntimeError("out of flag slots")
            s = Site(self._next_slot, self._target_store)
            self._next_slot += self.world
            self._sites[name] = s
        return s

    def pooled(self, kind: str, numel: int, dtype: torch.dtype):
        """One of two alternating buffers shared by all call sites of this kind and size.
        Two are enough: a rank can only be one collective ahead of its slowest peer, because
        finishing a fused collective needs data that every peer produces inside the same call."""
        key = (kind, numel, dtype)
        st = self._pools.get(key)
        if st is None:
            st = {"count": 0,
                  "bufs": [self.alloc(f"pool:{kind}:{i}", numel, dtype) for i in range(2)],
                  "sites": [self.site(("pool", kind, numel, dtype, i)) for i in range(2)]}
            self._pools[key] = st
        i = st["count"] & 1
        st["count"] += 1
        return st["bufs"][i], st["sites"][i]


    # ---------------------------------------------------------------- CUDA-graph support
    def _host_counts(self) -> torch.Tensor:
        import numpy as np
        counts = np.zeros(NUM_FLAG_SLOTS, dtype=np.uint32)
        for s in self._sites.values():
            counts[s.slot0:s.slot0 + self.world] = s.target.value
        return torch.from_numpy(counts.view(np.int32)).to(self.device)

    def fold_targets_into_base(self) -> None:
        """base += host counts; host counts restart at zero (launches keep waiting for the same
        absolute values)."""
        self.base.add_(self._host_counts())
        for s in self._sites.values():
            s.target.value = 0

    def record_per_step(self) -> None:
        """After a capture: the host counts are the step's per-site totals. Store them where the
        graph's epilogue reads them and restart the host counts."""
        self.per_step.copy_(self._host_counts())
        for s in self._sites.values():
            s.target.value = 0


def begin_graph_capture() -> None:
    """Call on every rank right before a step is captured (outside the capture)."""
    for g in _groups.values():
        g.fold_targets_into_base()


def fold_pending() -> None:
    """Call before replaying a captured step: launches made outside the graph since the capture (an
    evaluation pass, :meth:`DistributedOptimizer.sync_params`) advanced the flags and the host
    counts but not the base words the captured waits start from; fold them in. Local, cheap when
    nothing is pending (one vector test per group)."""
    for g in _groups.values():
        if g._target_view.any():
            g.fold_targets_into_base()


def graph_epilogue() -> None:
    """Call inside the capture after the step's last kernel: one small launch per group that
    advances the base words by the step's totals (filled in by :func:`end_graph_capture`)."""
    for g in _groups.values():
        g.base.add_(g.per_step)


def end_graph_capture() -> None:
    """Call right after the capture, before the first replay."""
    for g in _groups.values():
        g.record_per_step()


def abort_graph_capture() -> None:
    """A capture failed after :func:`begin_graph_capture`: the launches it recorded never ran, so
    the counts they added on the host are dropped (the base words already hold everything that
    did run)."""
    for g in _groups.values():
        for s in g._sites.values():
            s.target.value = 0


def get_group(kind: str) -> SymmGroup:
    """``kind``: "tp", "dp" or "world" (all ranks of the job)."""
    from . import parallel_state as ps
    g = _groups.get(kind)
    if g is None:
        from ..ops import _lib
        assert _lib.lib().gfs_flag_slots() == NUM_FLAG_SLOTS
        dev = ps.get_device()
        if kind == "tp":
            g = SymmGroup(ps.get_tensor_model_parallel_group(), ps.get_tensor_model_parallel_world_size(),
                          ps.get_tensor_model_parallel_group_rank(), dev)
        elif kind == "dp":
            g = SymmGroup(ps.get_data_parallel_group(), ps.get_data_parallel_world_size(),
                          ps.get_data_parallel_group_rank(), dev)
        elif kind == "world":
            g = SymmGroup(None, dist.get_world_size(), dist.get_rank(), dev)
        else:
            raise ValueError(kind)
        _groups[kind] = g
    return g


def check_all_canaries() -> None:
    for g in _groups.values():
        g.check_canaries()


def reset() -> None:
    _groups.clear()
