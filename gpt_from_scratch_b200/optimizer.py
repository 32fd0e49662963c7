"""DistributedOptimizer: bf16 compute with fp32 master weights, optimizer state sharded
over the data-parallel group (ZeRO-1 style).

Semantics follow the reference (core/optimizer.py:18-112):

* every trainable parameter, in module registration order, becomes a view into one flat
  ``param_buffer``; every ``.grad`` a view into one flat ``grad_buffer`` (same dtype);
* the flat length is padded so the DP size divides it; DP rank ``r`` owns the contiguous
  slice ``[r*shard_size, (r+1)*shard_size)`` and keeps an fp32 master copy plus the AdamW
  moments for that slice only;
* ``step()`` = reduce-scatter(SUM) of the gradients over DP -> clip by the global norm ->
  AdamW on the fp32 shard -> all-gather of the bf16-rounded parameters;
* ``state_dict()`` / ``load_state_dict()`` pass through to the inner ``torch.optim.AdamW``
  (which here also carries the state used by the fused kernels).

Differences that are deliberate:

* On CUDA/bf16 the clip + AdamW + cast is one kernel and the clip decision stays on the
  device (the reference synchronises the host on ``if norm > clip``, core/optimizer.py:103).
* ``zero_grad()`` does not memset: backward kernels overwrite each gradient slice on first
  use in a step (see ``ops/grad_sink.py``); a parameter whose gradient arrives through plain
  autograd instead (a bias, a fallback path) has its slice cleared by a tensor hook right
  before autograd accumulates into it.
* The gradient norm is global over TP x DP with replicated parameters counted once, and
  the gradients of TP-replicated parameters (the RMSNorm weights, which only see their
  sequence shard) are summed over the TP group before the step. ``reference_quirks=True``
  restores the reference's per-TP-rank norm and missing TP reduction.
* ``grad_reduce="mean"`` divides the DP-summed gradient by the DP size (the reference sums).
* With ``comm_impl == "fused"`` and DP > 1 the reduce-scatter, norm partial, AdamW and
  parameter all-gather run as peer-memory kernels (``parallel/fused_comm.py``), and the
  reduce-scatter's data movement overlaps the backward pass: the flat buffer is cut into a few
  buckets of whole parameters, every rank owns one slice of EVERY bucket (its optimizer shard is
  the concatenation of those slices instead of one contiguous range), and as soon as backward
  has written a bucket its slices are pushed to their owners on a side stream.
  ``state_dict()`` / ``load_state_dict()`` still speak the reference's layout (the contiguous
  range ``[r*shard_size, (r+1)*shard_size)``): they convert with a collective over the DP group.
"""
from __future__ import annotations

import math
import os

import torch
import torch.distributed as dist

from .ops import adam as adam_ops
from .ops import gemm as gemm_ops
from .ops.rmsnorm import flush_dw_reductions
from .parallel import mappings
from .parallel import parallel_state as ps


class DistributedOptimizer:
    def __init__(self, model: torch.nn.Module, optimizer_cls=torch.optim.AdamW, optimizer_kwargs: dict | None = None,
                 clip_grad: float = 1.0, dtype: torch.dtype = torch.bfloat16, grad_reduce: str = "sum",
                 reference_quirks: bool = False, fused: bool | None = None):
        self.model = model
        self.optimizer_kwargs = dict(optimizer_kwargs or {})
        self.dp_group = ps.get_data_parallel_group()
        self.dp_rank = ps.get_data_parallel_group_rank()
        self.dp_world_size = ps.get_data_parallel_world_size()
        self.tp_world_size = ps.get_tensor_model_parallel_world_size()
        self.clip_grad = clip_grad
        self.dtype = dtype
        self.grad_reduce = grad_reduce
        self.reference_quirks = reference_quirks
        assert grad_reduce in ("sum", "mean")

        self.params = [p for p in model.parameters() if p.requires_grad]
        if not self.params:
            raise ValueError("model has no trainable parameters")
        device = self.params[0].device
        self.device = device
        total_numel = sum(p.numel() for p in self.params)
        # pad so every DP shard is a whole number of 16-byte vectors (the reference pads to a
        # multiple of the DP size; the extra zeros are inert)
        align = self.dp_world_size * 8
        self.padding_size = (align - total_numel % align) % align
        self.padded_numel = total_numel + self.padding_size
        self.shard_size = self.padded_numel // self.dp_world_size
        self.total_numel = total_numel

        self.use_fused_kernels = (device.type == "cuda" and dtype == torch.bfloat16) if fused is None else fused
        self.use_fused_comm = (self.use_fused_kernels and self.dp_world_size > 1 and ps.get_comm_impl() == "fused")

        if self.use_fused_comm:
            from .parallel import fused_comm
            self._dp_comm = fused_comm.DataParallelComm(self.padded_numel, self.shard_size, device,
                                                        self._make_buckets())
            self.param_buffer = self._dp_comm.param_buffer
            self.grad_buffer = self._dp_comm.grad_buffer
        else:
            self._dp_comm = None
            self.param_buffer = torch.zeros(self.padded_numel, dtype=dtype, device=device)
            self.grad_buffer = torch.zeros(self.padded_numel, dtype=dtype, device=device)

        # re-point parameters and gradients into the flat buffers
        self.param_offsets: list[int] = []
        offset = 0
        replicated_ranges = []
        for p in self.params:
            n = p.numel()
            self.param_buffer[offset:offset + n].copy_(p.data.reshape(-1))
            p.data = self.param_buffer[offset:offset + n].view(p.shape)
            p.grad = self.grad_buffer[offset:offset + n].view(p.shape)
            p._grad_sink_ok = bool(self.use_fused_kernels)
            p._grad_fresh = False
            if self.use_fused_kernels:
                # a gradient that reaches this parameter through plain autograd (a bias, a
                # fallback path) is ADDED onto the slice: clear last step's values first
                p.register_hook(self._clear_stale_slice_hook(p))
            if getattr(p, "tp_replicated", False):
                replicated_ranges.append((offset, offset + n))
            self.param_offsets.append(offset)
            offset += n

        s0 = self.shard_size * self.dp_rank
        s1 = s0 + self.shard_size
        self.shard_start, self.shard_end = s0, s1
        self.interleaved = self._dp_comm is not None and self._dp_comm.nb > 1
        if self.interleaved:
            own = self._dp_comm.gather_shard(self.param_buffer)
        else:
            own = self.param_buffer[s0:s1]
        self.fp32_master_shard = own.to(torch.float32).clone().detach().requires_grad_(True)
        self.optimizer = optimizer_cls([self.fp32_master_shard], **self.optimizer_kwargs)
        if self.use_fused_comm:
            self.reduced_grad_shard = self._dp_comm.reduced
        elif self.dp_world_size > 1:
            self.reduced_grad_shard = torch.zeros(self.shard_size, dtype=dtype, device=device)
        else:
            self.reduced_grad_shard = self.grad_buffer[s0:s1]

        # indices of TP-replicated elements: whole buffer (for the TP gradient sum) and
        # inside this rank's shard (for counting them once in the global norm)
        self._rep_index_full = None
        self._rep_index_shard = None
        if self.tp_world_size > 1 and replicated_ranges:
            full = torch.cat([torch.arange(a, b, device=device) for a, b in replicated_ranges])
            self._rep_index_full = full
            if self.use_fused_comm:
                # position inside this rank's shard of every replicated element it owns
                pos = []
                for a, b, o in self._dp_comm.shard_slices():
                    sel = full[(full >= a) & (full < b)]
                    pos.append(sel - a + o)
                in_shard = torch.cat(pos)
            else:
                in_shard = full[(full >= s0) & (full < s1)] - s0
            self._rep_index_shard = in_shard
        self._sumsq = torch.zeros(4, dtype=torch.float32, device=device)   # [sumsq, replicated sumsq, 0, 0]
        # CUDA-graph mode: the step count lives on the device (a captured launch has frozen arguments)
        self.graph_mode = False
        self._step_dev = torch.zeros(1, dtype=torch.float32, device=device) if device.type == "cuda" else None
        self._norm_out = torch.zeros(1, dtype=torch.float32, device=device)
        self._step_count = 0
        self.last_grad_norm: torch.Tensor | None = None
        self._init_overlap()

    # ------------------------------------------------------------------ buckets / overlap
    NUM_BUCKETS = 6

    def _make_buckets(self) -> list[tuple[int, int]]:
        """Cut the flat buffer into at most NUM_BUCKETS ranges of roughly equal size at parameter
        boundaries (rounded down to a multiple of 8 x DP size, so a boundary may fall a few
        elements inside a parameter, which then belongs to both buckets). The walk goes from the
        END of the buffer, the order in which the backward pass produces the gradients, so the
        first bucket to leave is the LM head alone and later buckets fill up in production order."""
        align = 8 * self.dp_world_size
        target = max(align, self.padded_numel // self.NUM_BUCKETS)
        cuts, last = [self.padded_numel], self.padded_numel
        offset = sum(p.numel() for p in self.params)
        for p in reversed(self.params):
            offset -= p.numel()
            c = offset // align * align
            if last - c >= target and c >= target // 2:
                cuts.append(c)
                last = c
        # the first parameter (the embedding table: its gradient is the LAST one the backward pass
        # produces) gets a bucket of its own when it is large, so what precedes it can leave earlier
        first_end = self.params[0].numel() // align * align
        if first_end >= target // 2 and first_end < last:
            cuts.append(first_end)
        cuts.append(0)
        cuts = sorted(set(cuts))
        return [(a, b) for a, b in zip(cuts[:-1], cuts[1:]) if b > a]

    def _init_overlap(self) -> None:
        """Per-bucket bookkeeping for pushing a bucket's gradients while backward still runs.
        Armed per step by ``zero_grad()`` when ``overlap_grad_reduce`` is set (the training engine
        sets it: it guarantees exactly one backward pass between ``zero_grad()`` and ``step()``,
        with every parameter used once). A bucket is pushed early only when every parameter in it
        has reported its gradient final through its gradient sink; a parameter whose gradient
        arrives through plain autograd (a bias) never reports, so its bucket waits for ``step()``."""
        self.overlap_grad_reduce = False
        self._overlap_allowed = os.environ.get("GFS_DP_OVERLAP", "1") != "0"   # A/B switch
        self._overlap_armed = False
        self._push_stream = None
        if not self.use_fused_comm:
            return
        buckets = self._dp_comm.buckets
        self._param_buckets: dict[int, list[int]] = {}
        self._bucket_size = [0] * len(buckets)
        for p, off in zip(self.params, self.param_offsets):
            mine = [b for b, (a, e) in enumerate(buckets) if off < e and off + p.numel() > a]
            self._param_buckets[id(p)] = mine
            for b in mine:
                self._bucket_size[b] += 1
            p._grad_ready_cb = self._on_grad_ready
            p._grad_parked_cb = self._on_grad_parked
        self._pending = list(self._bucket_size)
        self._parked = [0] * len(buckets)
        self._pushed = [False] * len(buckets)
        self._push_stream = torch.cuda.Stream(self.device, priority=-1)

    def _reset_overlap(self) -> None:
        if not self.use_fused_comm:
            return
        self._pending = list(self._bucket_size)
        self._parked = [0] * len(self._bucket_size)
        self._pushed = [False] * len(self._bucket_size)
        self._overlap_armed = bool(self.overlap_grad_reduce and self._overlap_allowed)
        for p in self.params:
            p._gfs_parked = False
            p._gfs_ready = False

    def _on_grad_parked(self, p) -> None:
        """A kernel that will write ``p``'s gradient has been queued for a batched launch. If a
        bucket now waits for parked work only, launch that work."""
        if not self._overlap_armed or p._gfs_parked or p._gfs_ready:
            return
        p._gfs_parked = True
        flush = False
        for b in self._param_buckets[id(p)]:
            self._parked[b] += 1
            flush = flush or self._parked[b] == self._pending[b]
        if flush:
            gemm_ops.flush_wgrad()
            flush_dw_reductions()

    def _on_grad_ready(self, p) -> None:
        if not self._overlap_armed:
            return
        if p._gfs_ready:
            if any(self._pushed[b] for b in self._param_buckets[id(p)]):
                raise RuntimeError("a gradient was written after its bucket had been pushed to the other ranks "
                                   "(parameter used twice in one backward pass, or two backward passes in one "
                                   "step): set optimizer.overlap_grad_reduce = False for such models")
            return
        p._gfs_ready = True
        for b in self._param_buckets[id(p)]:
            if p._gfs_parked:
                self._parked[b] -= 1
            self._pending[b] -= 1
            if self._pending[b] == 0:
                self._push_bucket_async(b)

    def _push_bucket_async(self, b: int) -> None:
        """Bucket ``b`` is final on the current stream: push it on the side stream from here."""
        if self._pushed[b]:
            return
        self._pushed[b] = True
        ev = torch.cuda.Event()
        ev.record()
        self._push_stream.wait_event(ev)
        with torch.cuda.stream(self._push_stream):
            self._dp_comm.push_bucket(b)         # copy-engine transfers + a one-warp signal kernel

    def _finish_pushes(self) -> None:
        """Push whatever the backward pass did not (everything when overlap is off) and make the
        current stream wait for the side stream."""
        forked = any(self._pushed)
        for b in range(len(self._pushed)):
            if not self._pushed[b]:
                self._pushed[b] = True
                self._dp_comm.push_bucket(b)
        if forked:
            torch.cuda.current_stream().wait_stream(self._push_stream)
        self._overlap_armed = False
        self._pushed = [False] * len(self._pushed)

    # ------------------------------------------------------------------ gradients
    def zero_grad(self, set_to_zero: bool = False):
        """Prepare the gradient buffer for a new step. Never sets ``.grad`` to None (the
        views into the flat buffer must survive)."""
        gemm_ops.flush_wgrad()   # nothing parked may land in the buffer after this point
        flush_dw_reductions()
        self._reset_overlap()
        if self.use_fused_kernels and not set_to_zero:
            for p in self.params:
                p._grad_fresh = True
        else:
            self.grad_buffer.zero_()
            for p in self.params:
                p._grad_fresh = False

    @staticmethod
    def _clear_stale_slice_hook(p):
        def hook(grad):
            if getattr(p, "_grad_fresh", False):
                p.grad.zero_()
                p._grad_fresh = False
            return None
        return hook

    def _materialise_unwritten(self) -> None:
        for p in self.params:
            if getattr(p, "_grad_fresh", False):
                p.grad.zero_()
                p._grad_fresh = False

    def _sum_replicated_grads_over_tp(self) -> None:
        if self._rep_index_full is None or self.reference_quirks:
            return
        if self._fused_small_collectives() and self._rep_index_full.numel() % 8 == 0:
            from .parallel import fused_comm
            fused_comm.sum_over_tp_inplace(self.grad_buffer, self._rep_index_full)
            return
        vals = self.grad_buffer.index_select(0, self._rep_index_full)
        dist.all_reduce(vals, group=ps.get_tensor_model_parallel_group())
        self.grad_buffer.index_copy_(0, self._rep_index_full, vals)

    def _fused_small_collectives(self) -> bool:
        return self.use_fused_kernels and ps.get_comm_impl() == "fused"

    def step_dev(self):
        """Device step counter for kernels launched inside a captured step (``None`` otherwise)."""
        return self._step_dev if self.graph_mode else None

    # ------------------------------------------------------------------ step
    def step(self):
        gemm_ops.flush_wgrad()   # weight-gradient GEMMs parked for a grouped launch
        flush_dw_reductions()
        if self.graph_mode:
            self._step_dev.add_(1.0)
        self._materialise_unwritten()
        if not self.use_fused_comm:
            # (the fused DP path sums the replicated gradients over TP after its reduce-scatter, on
            # the reduced shard: the two sums commute, and buckets can leave before step())
            self._sum_replicated_grads_over_tp()
        if self.use_fused_comm:
            self._step_fused_comm()
        elif self.use_fused_kernels:
            self._step_fused_kernels()
        else:
            self._step_composition()
        self._step_count += 1

    def _hyper(self):
        g = self.optimizer.param_groups[0]
        beta1, beta2 = g.get("betas", (0.9, 0.999))
        return g["lr"], beta1, beta2, g.get("eps", 1e-8), g.get("weight_decay", 0.0)

    def _adam_state(self):
        st = self.optimizer.state[self.fp32_master_shard]
        if "exp_avg" not in st:
            st["step"] = torch.tensor(0.0, dtype=torch.float32)
            st["exp_avg"] = torch.zeros_like(self.fp32_master_shard, memory_format=torch.preserve_format)
            st["exp_avg_sq"] = torch.zeros_like(self.fp32_master_shard, memory_format=torch.preserve_format)
        return st

    def _global_sumsq(self, local: torch.Tensor) -> torch.Tensor:
        """local: fp32 [4] = {sum of squares of this shard, same over TP-replicated elements, 0, 0}."""
        world_tp = self.tp_world_size
        if self.reference_quirks or world_tp == 1:
            if self.dp_world_size > 1:
                dist.all_reduce(local[0:1], group=self.dp_group)
            return local[0:1]
        if self._fused_small_collectives():
            from .parallel import fused_comm
            local = fused_comm.allreduce_sum_small(local, "world")   # over TP x DP, no NCCL call
        else:
            dist.all_reduce(local)  # over TP x DP
        total = local[0:1] - local[1:2] * ((world_tp - 1) / world_tp)
        return total

    def _step_fused_kernels(self):
        if self.dp_world_size > 1:
            rs = mappings.reduce_scatter_dim0(self.grad_buffer, self.dp_group, self.dp_world_size, self.dp_rank)
            self.reduced_grad_shard.copy_(rs) if rs.data_ptr() != self.reduced_grad_shard.data_ptr() else None
        shard = self.reduced_grad_shard
        sumsq = None
        if self.clip_grad is not None and self.clip_grad > 0.0:
            adam_ops.sumsq_bf16(shard, self._sumsq[0:1])
            if self._rep_index_shard is not None and not self.reference_quirks:
                self._sumsq[1] = shard.index_select(0, self._rep_index_shard).float().pow(2).sum()
            else:
                self._sumsq[1:2].zero_()     # (a scalar assignment would be a host-to-device copy)
            sumsq = self._global_sumsq(self._sumsq)
        lr, beta1, beta2, eps, wd = self._hyper()
        st = self._adam_state()
        st["step"] += 1
        scale = 1.0 / self.dp_world_size if self.grad_reduce == "mean" else 1.0
        out = self.param_buffer[self.shard_start:self.shard_end]
        adam_ops.adamw_step(shard, self.fp32_master_shard.data, st["exp_avg"], st["exp_avg_sq"], out,
                            step=self._step_count + 1, lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=wd,
                            sumsq=sumsq, clip=float(self.clip_grad or 0.0), grad_scale=scale,
                            norm_out=self._norm_out, step_dev=self.step_dev())
        self.last_grad_norm = self._norm_out
        if self.dp_world_size > 1:
            dist.all_gather_into_tensor(self.param_buffer, out.clone(), group=self.dp_group)

    def _step_fused_comm(self):
        self._finish_pushes()
        lr, beta1, beta2, eps, wd = self._hyper()
        st = self._adam_state()
        st["step"] += 1
        scale = 1.0 / self.dp_world_size if self.grad_reduce == "mean" else 1.0
        self._dp_comm.step(self, st, step=self._step_count + 1, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
                           weight_decay=wd, clip=float(self.clip_grad or 0.0), grad_scale=scale)
        self.last_grad_norm = self._dp_comm.norm_out

    def _step_composition(self):
        """torch.distributed + torch.optim path (CPU/gloo, fp32, or fused=False): the reference's sequence."""
        if self.dp_world_size > 1:
            rs = mappings.reduce_scatter_dim0(self.grad_buffer, self.dp_group, self.dp_world_size, self.dp_rank)
            self.reduced_grad_shard.copy_(rs)
        shard = self.reduced_grad_shard
        if self.grad_reduce == "mean" and self.dp_world_size > 1:
            shard.div_(self.dp_world_size)
        if self.clip_grad is not None and self.clip_grad > 0.0:
            local = torch.zeros(2, dtype=torch.float32, device=shard.device)
            local[0] = shard.float().pow(2).sum()
            if self._rep_index_shard is not None and not self.reference_quirks:
                local[1] = shard.index_select(0, self._rep_index_shard).float().pow(2).sum()
            norm = torch.sqrt(self._global_sumsq(local))[0]
            self.last_grad_norm = norm
            if norm > self.clip_grad:
                shard.mul_(self.clip_grad / (norm + 1e-6))
        self.fp32_master_shard.grad = shard.to(torch.float32)
        self.optimizer.step()
        self.optimizer.zero_grad()
        new_shard = self._to_reference_layout(self.fp32_master_shard.detach()).to(self.dtype)
        if self.dp_world_size > 1:
            dist.all_gather_into_tensor(self.param_buffer, new_shard.contiguous(), group=self.dp_group)
        else:
            self.param_buffer.copy_(new_shard)

    # ------------------------------------------------------------------ state
    # -- the reference's shard is the contiguous range [r*shard, (r+1)*shard) of the flat buffer; with
    #    the bucket-interleaved layout the same elements are spread over the DP ranks
    def _to_reference_layout(self, t: torch.Tensor) -> torch.Tensor:
        if not self.interleaved or t.numel() != self.shard_size:
            return t
        world = self.dp_world_size
        every = torch.empty(world * self.shard_size, dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(every, t.detach().contiguous(), group=self.dp_group)
        every = every.view(world, self.shard_size)
        full = torch.empty(self.padded_numel, dtype=t.dtype, device=t.device)
        for r in range(world):
            for a, b, o in self._dp_comm.shard_slices(r):
                full[a:b] = every[r, o:o + (b - a)]
        return full[self.shard_start:self.shard_end].clone()

    def _from_reference_layout(self, t: torch.Tensor) -> torch.Tensor:
        if not self.interleaved or t.numel() != self.shard_size:
            return t
        t = t.to(self.device)
        full = torch.empty(self.padded_numel, dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(full, t.detach().contiguous(), group=self.dp_group)
        return self._dp_comm.gather_shard(full)

    def _convert_state(self, sd: dict, fn) -> dict:
        out = {"state": {}, "param_groups": sd["param_groups"]}
        for k, st in sd["state"].items():
            out["state"][k] = {n: (fn(v) if torch.is_tensor(v) and v.dim() == 1 else v) for n, v in st.items()}
        return out

    def state_dict(self):
        """The inner AdamW state (step, exp_avg, exp_avg_sq of the flat shard + param groups),
        as the reference returns (core/optimizer.py:106-108), in the reference's shard layout
        (a collective over the DP group when the bucket-interleaved layout is active)."""
        return self._convert_state(self.optimizer.state_dict(), self._to_reference_layout)

    def load_state_dict(self, state_dict):
        self.optimizer.load_state_dict(self._convert_state(state_dict, self._from_reference_layout))
        st = self.optimizer.state.get(self.fp32_master_shard, {})
        if "step" in st:
            self._step_count = int(float(st["step"]))
        self._sync_step_dev()

    def _sync_step_dev(self) -> None:
        if self._step_dev is not None:
            self._step_dev.fill_(float(self._step_count))

    def enter_graph_mode(self) -> None:
        """From now on ``step()`` takes the step count from device memory (incremented by the step
        itself), so a captured step stays correct when replayed."""
        self._sync_step_dev()
        self.graph_mode = True

    def note_replayed_step(self) -> None:
        """Host bookkeeping for one replay of a captured step (the device did the work)."""
        self._step_count += 1
        st = self._adam_state()
        st["step"] += 1

    def full_state_dict(self):
        """Everything needed to resume exactly: inner state + the fp32 master shard (which the
        reference's ``state_dict`` omits)."""
        return {"optimizer": self.state_dict(),
                "fp32_master_shard": self._to_reference_layout(self.fp32_master_shard.detach()).clone(),
                "step_count": self._step_count,
                "shard": (self.shard_start, self.shard_end, self.padded_numel)}

    def load_full_state_dict(self, sd):
        assert tuple(sd["shard"]) == (self.shard_start, self.shard_end, self.padded_numel), "sharding mismatch"
        self.load_state_dict(sd["optimizer"])
        with torch.no_grad():
            self.fp32_master_shard.copy_(self._from_reference_layout(sd["fp32_master_shard"]))
        self._step_count = int(sd["step_count"])
        self._sync_step_dev()
        # rebuild the low-precision parameters from the master weights
        new_shard = self._to_reference_layout(self.fp32_master_shard.detach()).to(self.dtype)
        if self.dp_world_size > 1:
            dist.all_gather_into_tensor(self.param_buffer, new_shard.contiguous(), group=self.dp_group)
        else:
            self.param_buffer.copy_(new_shard)
