"""Checkpoint save / resume. The reference never saves anything (its optimizer
``state_dict`` even omits the fp32 master weights); this module stores, per
(tp_rank, dp_rank): the model ``state_dict`` in the reference's key layout, the optimizer
shard (fp32 master, moments, step), and the loop state (step, epoch, batches consumed in that
epoch, RNG)."""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .parallel import parallel_state as ps


def _rank_file(directory: str, step: int) -> str:
    tp, dp = ps.get_tensor_model_parallel_group_rank(), ps.get_data_parallel_group_rank()
    return os.path.join(directory, f"step_{step:08d}", f"tp{tp:02d}_dp{dp:02d}.pt")


def save_checkpoint(directory: str, step: int, model, optimizer, extra: dict | None = None) -> str:
    path = _rank_file(directory, step)
    os.makedirs(os.path.dirname(path), exist_ok=True)
    payload = {
        "step": step,
        "tp_size": ps.get_tensor_model_parallel_world_size(),
        "dp_size": ps.get_data_parallel_world_size(),
        "model": {k: v.detach().cpu() for k, v in model.state_dict().items()},
        "optimizer": _to_cpu(optimizer.full_state_dict()),
        "torch_rng": torch.get_rng_state(),
        "cuda_rng": torch.cuda.get_rng_state() if torch.cuda.is_available() else None,
        "extra": extra or {},
    }
    tmp = path + ".tmp"
    torch.save(payload, tmp)
    os.replace(tmp, path)
    # `latest` may only name a step whose files are all in place: every rank's rename has to be
    # done before the pointer moves (a crash in between leaves the previous checkpoint current)
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
    if ps.get_tensor_model_parallel_group_rank() == 0 and ps.get_data_parallel_group_rank() == 0:
        latest = os.path.join(directory, "latest")
        with open(latest + ".tmp", "w") as f:
            f.write(str(step))
        os.replace(latest + ".tmp", latest)
    return path


def _to_cpu(obj):
    if torch.is_tensor(obj):
        return obj.detach().cpu()
    if isinstance(obj, dict):
        return {k: _to_cpu(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_cpu(v) for v in obj)
    return obj


def latest_step(directory: str) -> int | None:
    p = os.path.join(directory, "latest")
    if not os.path.exists(p):
        return None
    return int(open(p).read().strip())


def load_checkpoint(directory: str, model, optimizer, step: int | None = None) -> dict:
    step = latest_step(directory) if step is None else step
    if step is None:
        raise FileNotFoundError(f"no checkpoint in {directory}")
    path = _rank_file(directory, step)
    payload = torch.load(path, map_location="cpu", weights_only=False)
    if payload["tp_size"] != ps.get_tensor_model_parallel_world_size() or \
            payload["dp_size"] != ps.get_data_parallel_world_size():
        raise ValueError("checkpoint was written with a different TP/DP layout")
    # parameters are views into the optimizer's flat buffer: copy in place
    own = model.state_dict()
    with torch.no_grad():
        for k, v in payload["model"].items():
            own[k].copy_(v.to(own[k].device, dtype=own[k].dtype))
    dev = optimizer.fp32_master_shard.device
    osd = payload["optimizer"]
    osd["fp32_master_shard"] = osd["fp32_master_shard"].to(dev)
    optimizer.load_full_state_dict(osd)
    torch.set_rng_state(payload["torch_rng"])
    if payload.get("cuda_rng") is not None and torch.cuda.is_available():
        torch.cuda.set_rng_state(payload["cuda_rng"])
    return payload
