"""Helpers to run a function as N gloo ranks on CPU (spawned processes, 127.0.0.1 rendezvous)."""
import os
import socket
import sys
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, result_dir, init):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.set_num_threads(1)
    try:
        if init:
            dist.init_process_group("gloo", rank=rank, world_size=world)
        out = fn(rank, world, *args)
        torch.save(out, os.path.join(result_dir, f"rank{rank}.pt"))
    except Exception:
        traceback.print_exc()
        sys.exit(1)
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_ranks(fn, world: int, args=(), tmp_path=None, init: bool = True):
    """Run ``fn(rank, world, *args)`` on ``world`` CPU ranks; returns the list of results.
    ``init=False`` leaves the process group to ``fn`` (the rendezvous variables are set)."""
    result_dir = str(tmp_path)
    mp.spawn(_entry, args=(world, free_port(), fn, args, result_dir, init), nprocs=world, join=True)
    return [torch.load(os.path.join(result_dir, f"rank{r}.pt"), weights_only=False) for r in range(world)]
