"""Failure detection exercised on the host only (CPU/gloo ranks; no GPU is faulted): a rank
that stops reporting, a rank that never joins a collective, a wrong world size."""
import datetime
import time

import pytest
import torch
import torch.distributed as dist

from dist_utils import run_ranks


def _hb_worker(rank, world):
    from gpt_from_scratch_b200.utils.health import Heartbeat, PeerFailure
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, stale_after=0.5)
    hb.beat(0)
    dist.barrier()
    hb.check()                       # everybody is fresh
    if rank == 1:
        return "stopped"             # rank 1 "dies" between steps: it never beats again
    deadline = time.time() + 10
    while time.time() < deadline:
        hb.beat(1)
        try:
            hb.check()
        except PeerFailure as e:
            return ("detected", e.rank, e.last_step)
        time.sleep(0.1)
    return "missed"


def test_stalled_rank_is_reported(tmp_path):
    res = run_ranks(_hb_worker, 2, tmp_path=tmp_path)
    assert res[0] == ("detected", 1, 0)
    assert res[1] == "stopped"


def _timeout_worker(rank, world):
    # a second, short-timeout group: rank 1 never joins the collective
    g = dist.new_group(ranks=list(range(world)), timeout=datetime.timedelta(seconds=2), backend="gloo")
    if rank == 1:
        time.sleep(4)
        return "absent"
    t = torch.ones(4)
    try:
        dist.all_reduce(t, group=g)
    except Exception as e:  # noqa: BLE001
        return ("error", type(e).__name__)
    return "no error"


def test_collective_with_absent_rank_times_out(tmp_path):
    res = run_ranks(_timeout_worker, 2, tmp_path=tmp_path)
    assert res[0][0] == "error", res


def _bad_world_worker(rank, world):
    from gpt_from_scratch_b200.parallel import parallel_state as ps
    ps.set_device("cpu")
    try:
        ps.initialize_parallel_state(3)    # 2 ranks cannot host TP=3
    except ValueError as e:
        return str(e)
    return "accepted"


def test_wrong_tensor_parallel_size_is_rejected(tmp_path):
    res = run_ranks(_bad_world_worker, 2, tmp_path=tmp_path)
    assert all("not divisible" in r for r in res)
