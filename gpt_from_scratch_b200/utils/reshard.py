"""Convert between an unsharded (TP=1) ``state_dict`` and per-TP-rank shards.

Because the packed projections are stored as ``[q|k|v] x local heads x D`` and
``[gate_local | up_local]`` (the reference's layouts, core/transformer_layer.py:42-44 and
core/mlp.py:25), a TP shard is not a contiguous slice of the TP=1 tensor: the q, k, v (and
gate, up) blocks have to be sliced separately.
"""
from __future__ import annotations

import re

import torch


def _kind(key: str) -> str:
    if key.endswith("qkv_proj.weight") or key.endswith("qkv_proj.bias"):
        return "col3"
    if key.endswith("gate_up_proj.weight") or key.endswith("gate_up_proj.bias"):
        return "col2"
    if key in ("embedding.weight", "output.weight", "output.bias"):
        return "col1"
    if key.endswith("out_proj.weight") or key.endswith("down_proj.weight"):
        return "row"
    return "replicated"


def shard_state_dict(full: dict, tp_rank: int, tp_size: int) -> dict:
    out = {}
    for k, v in full.items():
        kind = _kind(k)
        if kind.startswith("col"):
            blocks = int(kind[3])
            parts = v.chunk(blocks, dim=0)
            out[k] = torch.cat([p.chunk(tp_size, dim=0)[tp_rank] for p in parts], dim=0).clone()
        elif kind == "row":
            out[k] = v.chunk(tp_size, dim=1)[tp_rank].clone()
        else:
            out[k] = v.clone()
    return out


def merge_state_dicts(shards: list[dict]) -> dict:
    tp_size = len(shards)
    out = {}
    for k in shards[0]:
        kind = _kind(k)
        vs = [s[k] for s in shards]
        if kind.startswith("col"):
            blocks = int(kind[3])
            per_rank = [v.chunk(blocks, dim=0) for v in vs]
            out[k] = torch.cat([torch.cat([per_rank[r][b] for r in range(tp_size)], dim=0) for b in range(blocks)],
                               dim=0)
        elif kind == "row":
            out[k] = torch.cat(vs, dim=1)
        else:
            out[k] = vs[0].clone()
    return out


def layer_index(key: str) -> int | None:
    m = re.match(r"layers\.(\d+)\.", key)
    return int(m.group(1)) if m else None
