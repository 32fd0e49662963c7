"""Single-GPU stand-in for a group of ranks ("fake peers").

The fused collectives address their peers only through tables of device pointers (buffers and
flag arrays). :class:`FakePeerGroup` builds those tables out of ordinary allocations on ONE
GPU: this process plays rank ``rank`` of a group of ``world``; the other ranks are plain
buffers that nothing executes for. What the absent ranks would have contributed is either

* pre-set (``peers_ready=True``): the flag words that the absent ranks would have advanced
  start at a value every wait accepts, and the test writes the data they would have pushed
  into this rank's buffers beforehand. Every fused kernel then runs to completion exactly as
  it does as one rank of a real group - same code path, same signalling, same waits - so its
  numerics can be checked against PyTorch and it can be profiled on a single GPU;
* or left missing (``peers_ready=False``): the flags never move, so a kernel's bounded wait
  runs out and reports ``STATUS_TIMEOUT_PEER_FLAG``. This exercises the time-out path of the
  signal protocol without a second process and without hanging anything (used with a
  millisecond limit, comm kernels only).

Installed with ``with fake_peers(world, rank): ...`` it takes the place of the tensor- and
data-parallel :class:`~.symm.SymmGroup` objects, so the operators of ``fused_comm`` run
unmodified. The reference has no counterpart (it has no tests of its collectives at all).
"""
from __future__ import annotations

import contextlib
import ctypes

import torch

from . import symm

# a counter value that satisfies every wait of a test (targets stay far below it) and is still
# "reached" under the kernels' wrap-safe signed comparison
READY = 0x20000000


class FakePeerGroup(symm.SymmGroup):
    def __init__(self, world: int, rank: int, device: torch.device, peers_ready: bool = True):
        self.group = None
        self.world = world
        self.rank = rank
        self.device = device
        self.peers_ready = peers_ready
        self._buffers = {}
        self._raw = {}
        self._sites = {}
        self._pools = {}
        self._next_slot = 0
        self.has_multicast = False
        import numpy as np
        self._target_store = (ctypes.c_uint * symm.NUM_FLAG_SLOTS)()
        self._target_view = np.frombuffer(self._target_store, dtype=np.uint32)
        flags = self.alloc("__flags__", 2 * symm.NUM_FLAG_SLOTS, torch.int32, zero=True)
        self.flags = flags
        self.flag_ptrs = flags.ptrs
        self.base = flags.tensor[symm.NUM_FLAG_SLOTS:]
        self.per_step = torch.zeros(symm.NUM_FLAG_SLOTS, dtype=torch.int32, device=device)

    def alloc(self, name, numel, dtype, zero=False):
        key = (name, numel, dtype)
        buf = self._buffers.get(key)
        if buf is not None:
            return buf
        # one allocation per (fake) rank; all zero-filled so that what an absent rank "sent" is
        # well defined until a test writes something else
        per_rank = [torch.zeros(numel, dtype=dtype, device=self.device) for _ in range(self.world)]
        ptrs = (ctypes.c_ulonglong * (self.world + 1))(*[t.data_ptr() for t in per_rank], 0)   # no multicast
        buf = symm.SymmBuffer(per_rank[self.rank], ptrs, per_rank)     # handle = every rank's tensor
        self._buffers[key] = buf
        return buf

    def site(self, name):
        s = self._sites.get(name)
        new = s is None
        s = super().site(name)
        if new and self.peers_ready:
            # flags[this rank][slot0 + src] for every absent source
            mine = self.flags.tensor
            for src in range(self.world):
                if src != self.rank:
                    mine[s.slot0 + src] = READY
        return s

    def pooled(self, kind, numel, dtype):
        """No alternation: there is no second rank that could still be reading the buffer."""
        key = (kind, numel, dtype)
        st = self._pools.get(key)
        if st is None:
            st = (self.alloc(f"pool:{kind}", numel, dtype), self.site(("pool", kind, numel, dtype)))
            self._pools[key] = st
        return st

    def rank_tensors(self, buf: symm.SymmBuffer) -> list[torch.Tensor]:
        """The tensors standing for every rank's copy of a symmetric buffer."""
        return buf.handle

    def check_canaries(self) -> None:
        return None


@contextlib.contextmanager
def fake_peers(world: int, rank: int = 0, kinds=("tp", "dp", "world"), peers_ready: bool = True,
               device: torch.device | None = None):
    """Install fake-peer groups for the given kinds; restores the previous groups on exit."""
    from . import parallel_state as ps
    device = device or ps.get_device()
    saved = dict(symm._groups)
    try:
        for k in kinds:
            symm._groups[k] = FakePeerGroup(world, rank, device, peers_ready)
        yield {k: symm._groups[k] for k in kinds}
    finally:
        torch.cuda.synchronize(device)
        symm._groups.clear()
        symm._groups.update(saved)
