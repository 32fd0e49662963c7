"""Training engine: the public entry point that builds the model + distributed optimizer
and runs one optimisation step. ``train.py`` and ``bench.py`` both drive this class.

The step is the reference's loop body (train.py:172-187): ``zero_grad -> forward ->
vocab-parallel cross entropy -> mean -> backward -> optimizer.step``; the loss stays on the
device (the reference calls ``.item()`` every step, train.py:190)."""
from __future__ import annotations

import torch

from .config import GPTConfig
from .models.gpt import GPTModel
from .optimizer import DistributedOptimizer
from .parallel import parallel_state as ps
from .parallel.loss import vocab_parallel_cross_entropy


class LossHandle:
    """The loss of one step on its way to the host: an asynchronous device-to-host copy into
    pinned memory plus the event that marks its completion. ``value()`` blocks only until that
    copy is done, so a loop that reads step i's loss while step i+1 is already queued never
    drains the GPU (the reference's per-step ``.item()`` does, train.py:190)."""
    __slots__ = ("_buf", "_event")

    def __init__(self, buf: torch.Tensor, event):
        self._buf, self._event = buf, event

    def ready(self) -> bool:
        return self._event is None or self._event.query()

    def value(self) -> float:
        if self._event is not None:
            self._event.synchronize()
        return float(self._buf[0])


class TrainEngine:
    def __init__(self, config: GPTConfig, *, lr: float = 3e-4, weight_decay: float = 0.1,
                 betas: tuple[float, float] = (0.9, 0.95), clip_grad: float = 1.0,
                 dtype: torch.dtype = torch.bfloat16, grad_reduce: str = "sum", seed: int | None = None):
        if not ps.model_parallel_is_initialized():
            ps.initialize_parallel_state(1)
        if seed is not None:
            ps.set_seed(seed)
        self.config = config
        self.device = ps.get_device()
        self.model = GPTModel(config)
        self.optimizer = DistributedOptimizer(
            self.model, torch.optim.AdamW,
            {"lr": lr, "weight_decay": weight_decay, "betas": betas},
            clip_grad=clip_grad, dtype=dtype, grad_reduce=grad_reduce,
            reference_quirks=getattr(config, "reference_quirks", False))
        self.model.train()
        self.steps_done = 0
        self._loss_ring: list[torch.Tensor] = []

    @property
    def params_per_tp_rank(self) -> int:
        return sum(p.numel() for p in self.model.parameters())

    def forward_loss(self, inputs: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        """inputs, labels: ``[B, S]`` token ids on the engine's device -> mean loss (scalar)."""
        logits, ce_partials = self.model(inputs, return_ce_stats=True)        # [S, B, V/P]
        labels_t = labels.transpose(0, 1).contiguous()                        # [S, B]
        loss = vocab_parallel_cross_entropy(logits, labels_t, ce_partials)    # [S, B]
        return loss.mean()

    def train_step(self, inputs: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        self.optimizer.zero_grad()
        loss = self.forward_loss(inputs, labels)
        loss.backward()
        self.optimizer.step()
        self.steps_done += 1
        return loss.detach()

    def train_step_async(self, inputs: torch.Tensor, labels: torch.Tensor) -> LossHandle:
        """One step whose loss is copied to pinned host memory asynchronously; read it with
        ``LossHandle.value()`` (typically one step later, for logging)."""
        loss = self.train_step(inputs, labels)
        if not loss.is_cuda:
            return LossHandle(loss.float().reshape(1), None)
        if not self._loss_ring:
            self._loss_ring = [torch.empty(1, dtype=torch.float32).pin_memory() for _ in range(4)]
        buf = self._loss_ring[self.steps_done % len(self._loss_ring)]
        buf.copy_(loss.float().reshape(1), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        return LossHandle(buf, ev)
