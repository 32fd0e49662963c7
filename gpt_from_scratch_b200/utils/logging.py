"""Rank-0 logging. The console line has the reference's format (train.py:201-204) so logs
diff cleanly; ``JsonlLogger`` adds machine-readable records (loss, grad norm, device step
time, tokens/s, MFU, peak memory)."""
from __future__ import annotations

import json
import time

import torch
import torch.distributed as dist


def is_rank0() -> bool:
    return not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0


def print_rank0(*args, **kwargs) -> None:
    if is_rank0():
        print(*args, **kwargs, flush=True)


def format_step_line(step: int, max_steps: int, avg_loss: float, tokens_per_sec: float, elapsed: float) -> str:
    return (f"Step {step:>6d}/{max_steps} | Loss: {avg_loss:.4f} | "
            f"Tokens/s: {tokens_per_sec:.0f} | Time: {elapsed:.1f}s")


class JsonlLogger:
    def __init__(self, path: str | None):
        self.f = open(path, "a") if (path and is_rank0()) else None

    def log(self, **record) -> None:
        if self.f is None:
            return
        record.setdefault("time", time.time())
        for k, v in list(record.items()):
            if torch.is_tensor(v):
                record[k] = float(v)
        self.f.write(json.dumps(record) + "\n")
        self.f.flush()

    def close(self) -> None:
        if self.f is not None:
            self.f.close()
            self.f = None
