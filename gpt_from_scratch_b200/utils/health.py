"""Host-side failure detection. The reference has none: a dead rank hangs NCCL until the
watchdog fires. Here every rank publishes a heartbeat (its step counter and a wall-clock
stamp) in the job's key-value store after every step; at every log interval the training
loop waits (bounded) until all peers have reported that step before it launches the next one,
so a rank that died or stalled between steps is reported as a Python exception on the
survivors instead of a hang inside the next collective (``train.py --heartbeat-timeout``). Recovery is a restart from the last
checkpoint (``torchrun --max-restarts``); no in-job elasticity is claimed.

Device-side waits are bounded separately (see ``csrc/common.cuh``): they end with a status
word, which :func:`check_device_status` turns into an exception.
"""
from __future__ import annotations

import time

import torch.distributed as dist


class PeerFailure(RuntimeError):
    def __init__(self, rank: int, age: float, last_step: int):
        super().__init__(f"rank {rank} has not reported for {age:.1f}s (last step {last_step})")
        self.rank, self.age, self.last_step = rank, age, last_step


class Heartbeat:
    def __init__(self, store, rank: int, world: int, stale_after: float = 60.0, prefix: str = "gfs_hb"):
        self.store, self.rank, self.world = store, rank, world
        self.stale_after = stale_after
        self.prefix = prefix

    def beat(self, step: int) -> None:
        self.store.set(f"{self.prefix}/{self.rank}", f"{step}:{time.time():.3f}")

    def peers(self) -> dict[int, tuple[int, float]]:
        out = {}
        for r in range(self.world):
            try:
                if hasattr(self.store, "check") and not self.store.check([f"{self.prefix}/{r}"]):
                    continue
                raw = self.store.get(f"{self.prefix}/{r}").decode()
            except Exception:
                continue
            step, stamp = raw.split(":")
            out[r] = (int(step), float(stamp))
        return out

    def check(self, now: float | None = None) -> None:
        """Raise :class:`PeerFailure` if any peer that has reported before is stale."""
        now = time.time() if now is None else now
        for r, (step, stamp) in self.peers().items():
            if r != self.rank and now - stamp > self.stale_after:
                raise PeerFailure(r, now - stamp, step)


    def wait_for_peers(self, step: int, timeout: float | None = None, poll: float = 0.02) -> None:
        """Block until every peer has reported ``step`` (or a later one); raise
        :class:`PeerFailure` for the first peer that has not done so within ``timeout`` seconds
        (default: ``stale_after``). Call it between steps, before the next collective is
        launched."""
        timeout = self.stale_after if timeout is None else timeout
        start = time.time()
        while True:
            seen = self.peers()
            behind = [r for r in range(self.world) if r != self.rank and seen.get(r, (-1, 0.0))[0] < step]
            if not behind:
                return
            now = time.time()
            if now - start > timeout:
                r = behind[0]
                last_step, stamp = seen.get(r, (-1, start))
                raise PeerFailure(r, now - stamp, last_step)
            time.sleep(poll)


def default_heartbeat(stale_after: float = 60.0) -> Heartbeat | None:
    if not (dist.is_available() and dist.is_initialized()):
        return None
    store = dist.distributed_c10d._get_default_store()
    return Heartbeat(store, dist.get_rank(), dist.get_world_size(), stale_after)


def check_device_status() -> None:
    """Raise if a kernel of this process recorded a timed-out wait or a bad argument."""
    from ..ops import _lib
    _lib.raise_on_status()
