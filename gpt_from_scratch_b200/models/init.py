"""Weight initialiser selection (``xavier_uniform`` on the shard, as the reference does, or
``normal(0, std)``)."""
from __future__ import annotations

import torch.nn.init as init

from ..parallel.layers import normal_init


def get_init_method(config):
    name = getattr(config, "init_method", "xavier_uniform")
    if name == "xavier_uniform":
        return init.xavier_uniform_
    if name == "normal":
        return normal_init(getattr(config, "init_std", 0.02))
    raise ValueError(f"unknown init method {name!r}")
