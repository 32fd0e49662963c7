"""Training engine: the public entry point that builds the model + distributed optimizer
and runs one optimisation step. ``train.py`` and ``bench.py`` both drive this class.

The step is the reference's loop body (train.py:172-187): ``zero_grad -> forward ->
vocab-parallel cross entropy -> mean -> backward -> optimizer.step``; the loss stays on the
device (the reference calls ``.item()`` every step, train.py:190).

``cuda_graph=True``: after a few eager steps the whole step (about 230 kernel launches at
TP=1, 280 at TP=2 for the 12-layer model) is captured once into a CUDA graph and replayed, so
the host issues one launch per step instead of hundreds; the tensor-parallel configurations,
whose kernels are short, are otherwise bound by Python launch overhead. What makes the step
replayable: the batch is copied into fixed input buffers, the optimizer's step count lives on
the device, and the cross-GPU flag targets of the fused collectives are relative to per-counter
base words that the graph's last node advances (``parallel/symm.py``)."""
from __future__ import annotations

import os

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
                 dtype: torch.dtype = torch.bfloat16, grad_reduce: str = "sum", seed: int | None = None,
                 cuda_graph: bool | None = None, graph_warmup: int = 3):
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
        # one backward pass per step, every parameter used once: gradient buckets may leave for their
        # owners while backward still runs
        self.optimizer.overlap_grad_reduce = True
        self.model.train()
        self.steps_done = 0
        self._loss_ring: list[torch.Tensor] = []
        if cuda_graph is None:
            cuda_graph = os.environ.get("GFS_CUDA_GRAPH", "0") == "1"
        # a captured step replays the same dropout masks, so dropout keeps the eager loop
        self.cuda_graph = bool(cuda_graph and self.device.type == "cuda" and dtype == torch.bfloat16 and
                               getattr(config, "dropout_prob", 0.0) == 0.0)
        self.graph_warmup = max(2, graph_warmup)     # the first steps create buffers and call sites
        self._graph = None
        self._graph_shape = None
        self._graph_launches = 0
        self._host_counted = False

    @property
    def params_per_tp_rank(self) -> int:
        return sum(p.numel() for p in self.model.parameters())

    def forward_loss(self, inputs: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        """inputs, labels: ``[B, S]`` token ids on the engine's device -> mean loss (scalar)."""
        logits, ce_partials = self.model(inputs, return_ce_stats=True)        # [S, B, V/P]
        labels_t = labels.transpose(0, 1).contiguous()                        # [S, B]
        loss = vocab_parallel_cross_entropy(logits, labels_t, ce_partials)    # [S, B]
        return loss.mean()

    def _eager_step(self, inputs: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        self.optimizer.zero_grad()
        loss = self.forward_loss(inputs, labels)
        loss.backward()
        self.optimizer.step()
        return loss.detach()

    def train_step(self, inputs: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        if self.cuda_graph and self.steps_done >= self.graph_warmup:
            if self._graph is None:
                self._try_capture(inputs, labels)
            if self._graph is not None and tuple(inputs.shape) == self._graph_shape:
                return self._replay(inputs, labels)
        loss = self._eager_step(inputs, labels)
        self.steps_done += 1
        return loss

    # ------------------------------------------------------------------ CUDA graph
    def _try_capture(self, inputs: torch.Tensor, labels: torch.Tensor) -> None:
        """Capture the step; if the capture fails (an operator that cannot be captured on this
        system), undo its host-side effects, say so once and keep the eager loop."""
        import sys
        from .ops import gemm as gemm_ops
        from .ops import rmsnorm as rmsnorm_ops
        steps_before = self.optimizer._step_count
        try:
            self._capture(inputs, labels)
        except Exception as e:  # noqa: BLE001 - any capture failure means "run eagerly"
            from .parallel import symm
            self.cuda_graph = False
            self._graph = None
            symm.abort_graph_capture()
            gemm_ops._wgrad_queue.items.clear()          # parked work refers to tensors of the failed capture
            gemm_ops._wgrad_queue.tiles = 0
            rmsnorm_ops._dw_queue.items.clear()
            if self.optimizer._step_count != steps_before:   # the captured step never ran on the GPU
                self.optimizer._step_count = steps_before
                st = self.optimizer._adam_state()
                st["step"].fill_(float(steps_before))
            torch.cuda.synchronize(self.device)
            print(f"[gpt_from_scratch_b200] CUDA-graph capture of the training step failed "
                  f"({type(e).__name__}: {str(e)[:200]}); continuing with eager launches", file=sys.stderr)

    def _capture(self, inputs: torch.Tensor, labels: torch.Tensor) -> None:
        """Capture one whole step (all ranks do so at the same step). Nothing runs on the GPU here;
        the first replay executes the captured step."""
        from .ops import _lib
        from .parallel import symm
        self._static_inputs = inputs.clone()
        self._static_labels = labels.clone()
        self._graph_shape = tuple(inputs.shape)
        torch.cuda.synchronize(self.device)
        self.optimizer.enter_graph_mode()
        symm.begin_graph_capture()
        launches0 = _lib.launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            loss = self._eager_step(self._static_inputs, self._static_labels)
            symm.graph_epilogue()
            self._static_loss = loss
        symm.end_graph_capture()
        self._graph_launches = _lib.launch_count() - launches0
        self._graph = graph
        self._host_counted = True      # the capture already advanced the host-side step counters once

    def _replay(self, inputs: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        from .ops import _lib
        self._static_inputs.copy_(inputs, non_blocking=True)
        self._static_labels.copy_(labels, non_blocking=True)
        from .parallel import symm
        symm.fold_pending()          # launches made outside the graph since the last replay
        self._graph.replay()
        if self._host_counted:
            self._host_counted = False
        else:
            self.optimizer.note_replayed_step()
            _lib.add_launches(self._graph_launches)
        self.steps_done += 1
        return self._static_loss.clone()

    @property
    def launches_per_graph_step(self) -> int:
        """Kernels of the native library inside one captured step (0 before the capture)."""
        return self._graph_launches

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
