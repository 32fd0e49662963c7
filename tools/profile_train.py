"""Device-timed profile of the training step: per-phase times (max over ranks), per-module
forward times, collectives by group, memory accounting, throughput and MFU, optional
chrome trace.

    python tools/profile_train.py --steps 5 --warmup 3 [--tensor-model-parallel-size P] \
        [--peak-tflops 1635] [--enable-trace --trace-path trace.json] [model flags as train.py]
    torchrun --nproc-per-node N tools/profile_train.py ...

Every duration is measured with CUDA events on the launching stream and reduced with
MAX over ranks; nothing here is taken from the host clock. The report sections mirror the
profiler the reference's author kept out of the repository (phase / forward /
communication / memory / throughput).
"""
from __future__ import annotations

import argparse
import collections
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gpt_from_scratch_b200.config import GPTConfig  # noqa: E402
from gpt_from_scratch_b200.engine import TrainEngine  # noqa: E402
from gpt_from_scratch_b200.parallel import parallel_state as ps  # noqa: E402
from gpt_from_scratch_b200.parallel.loss import vocab_parallel_cross_entropy  # noqa: E402
from gpt_from_scratch_b200.utils.timing import max_over_ranks  # noqa: E402


class TimerGroup:
    """Named CUDA-event timers; ``summary()`` returns mean milliseconds, max over ranks."""

    def __init__(self, device):
        self.device = device
        self.pending = collections.defaultdict(list)

    class _Span:
        def __init__(self, group, name):
            self.group, self.name = group, name

        def __enter__(self):
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e1 = torch.cuda.Event(enable_timing=True)
            self.e0.record()
            return self

        def __exit__(self, *exc):
            self.e1.record()
            self.group.pending[self.name].append((self.e0, self.e1))
            return False

    def span(self, name):
        return TimerGroup._Span(self, name)

    def summary(self):
        torch.cuda.synchronize()
        out = {}
        # local means first: the reduction below is itself a (possibly wrapped and timed) collective
        local = [(name, sum(a.elapsed_time(b) for a, b in evs) / max(1, len(evs)), len(evs))
                 for name, evs in sorted(self.pending.items())]
        for name, ms, n in local:
            out[name] = (max_over_ranks(ms, self.device), n)
        return out


class CommProfiler:
    """Wraps the torch.distributed collectives used by the composition path and times them
    per group (TP / DP / world). The fused kernels do their communication inside compute
    kernels, so with ``--comm-impl fused`` this section only shows what is left on NCCL."""

    OPS = ("all_gather_into_tensor", "reduce_scatter_tensor", "all_reduce")

    def __init__(self, timers: TimerGroup):
        self.timers = timers
        self.saved = {}

    def _kind(self, group):
        if group is None:
            return "world"
        if group is ps.get_tensor_model_parallel_group():
            return "tp"
        if group is ps.get_data_parallel_group():
            return "dp"
        return "other"

    def install(self):
        for op in self.OPS:
            orig = getattr(dist, op)
            self.saved[op] = orig

            def wrapped(*a, __orig=orig, __op=op, **kw):
                with self.timers.span(f"comm/{self._kind(kw.get('group'))}/{__op}"):
                    return __orig(*a, **kw)
            setattr(dist, op, wrapped)

    def remove(self):
        for op, orig in self.saved.items():
            setattr(dist, op, orig)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--vocab-size", type=int, default=50304)
    ap.add_argument("--hidden-size", type=int, default=768)
    ap.add_argument("--num-layers", type=int, default=12)
    ap.add_argument("--num-attention-heads", type=int, default=12)
    ap.add_argument("--intermediate-size", type=int, default=3072)
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--batch-size", type=int, default=16)
    ap.add_argument("--tensor-model-parallel-size", type=int, default=1)
    ap.add_argument("--comm-impl", choices=["fused", "nccl"], default="nccl")
    ap.add_argument("--steps", "--profile-steps", dest="steps", type=int, default=5)
    ap.add_argument("--warmup", "--warmup-steps", dest="warmup", type=int, default=3)
    ap.add_argument("--peak-tflops", type=float, default=None)
    ap.add_argument("--enable-trace", action="store_true")
    ap.add_argument("--trace-path", type=str, default="trace.json")
    ap.add_argument("--with-stack", action="store_true")
    args = ap.parse_args()

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if "RANK" in os.environ:
        dist.init_process_group("nccl", device_id=dev)
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    ps.set_device(dev)
    ps.initialize_parallel_state(args.tensor_model_parallel_size)
    ps.set_comm_impl(args.comm_impl)
    tp = args.tensor_model_parallel_size
    dp = world // tp
    cfg = GPTConfig(vocab_size=args.vocab_size, hidden_size=args.hidden_size, num_layers=args.num_layers,
                    num_attention_heads=args.num_attention_heads, max_position_embeddings=args.seq_len,
                    intermediate_size=args.intermediate_size)
    eng = TrainEngine(cfg, seed=1)
    timers = TimerGroup(dev)
    comm = CommProfiler(timers)
    comm.install()

    # forward hooks on the direct children of each block + top-level modules
    handles = []

    def add_hooks(name, mod):
        spans = []

        def pre(_m, _i):
            s = timers.span(f"forward/{name}")
            s.__enter__()
            spans.append(s)

        def post(_m, _i, _o):
            spans.pop().__exit__()
        handles.append(mod.register_forward_pre_hook(pre))
        handles.append(mod.register_forward_hook(post))
    add_hooks("embedding", eng.model.embedding)
    add_hooks("final_norm", eng.model.final_norm)
    add_hooks("output(lm head)", eng.model.output)
    for layer in eng.model.layers:
        add_hooks("layer.input_norm", layer.input_norm)
        add_hooks("layer.attention", layer.attention)
        add_hooks("layer.post_attention_norm", layer.post_attention_norm)
        add_hooks("layer.mlp", layer.mlp)

    g = torch.Generator().manual_seed(7 + rank // tp)
    B, S = args.batch_size, args.seq_len

    def batch():
        t = torch.randint(0, min(args.vocab_size, 50257), (B, S + 1), generator=g)
        return t[:, :-1].contiguous().pin_memory(), t[:, 1:].contiguous().pin_memory()

    def step(profile: bool):
        hx, hy = batch()
        sp = timers.span if profile else (lambda name: _Null())
        with sp("phase/step"):
            with sp("phase/data_h2d"):
                x, y = hx.to(dev, non_blocking=True), hy.to(dev, non_blocking=True)
            with sp("phase/zero_grad"):
                eng.optimizer.zero_grad()
            with sp("phase/forward"):
                logits = eng.model(x)
            with sp("phase/loss"):
                loss = vocab_parallel_cross_entropy(logits, y.t().contiguous()).mean()
            with sp("phase/backward"):
                loss.backward()
            with sp("phase/optimizer_step"):
                eng.optimizer.step()
        return loss

    class _Null:
        def __enter__(self):
            return self

        def __exit__(self, *exc):
            return False

    for h in handles:
        pass
    for _ in range(args.warmup):
        step(False)
    timers.pending.clear()
    torch.cuda.reset_peak_memory_stats()
    prof = None
    if args.enable_trace:
        prof = torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU,
                                                  torch.profiler.ProfilerActivity.CUDA],
                                      with_stack=args.with_stack)
        prof.__enter__()
    for _ in range(args.steps):
        step(True)
    if prof is not None:
        prof.__exit__(None, None, None)
        if rank == 0:
            prof.export_chrome_trace(args.trace_path)
    summ = timers.summary()
    comm.remove()
    for h in handles:
        h.remove()

    step_ms = summ["phase/step"][0]
    tokens = B * S * dp
    tps = tokens / (step_ms / 1e3)
    fpt = cfg.flops_per_token(S)
    peak = args.peak_tflops
    if peak is None:
        try:
            peak = json.load(open(os.path.join(os.path.dirname(__file__), "..", "MEASURED_PEAKS.json")))["bf16_tflops"]
        except Exception:
            peak = None
    # memory accounting: what the flat buffers and optimizer shards must take vs what torch reports
    opt = eng.optimizer
    theory = {"param_buffer (bf16)": opt.padded_numel * 2, "grad_buffer (bf16)": opt.padded_numel * 2,
              "fp32 master shard": opt.shard_size * 4, "adam moments (fp32 x2)": opt.shard_size * 8}
    if rank == 0:
        print(f"=== configuration: world {world} (TP {tp} x DP {dp}), comm {args.comm_impl}, B {B}, S {S}, "
              f"{sum(p.numel() for p in eng.model.parameters()) / 1e6:.1f}M params per TP rank")
        for section in ("phase", "forward", "comm"):
            rows = sorted(((k, v) for k, v in summ.items() if k.startswith(section + "/")), key=lambda kv: -kv[1][0])
            if not rows:
                continue
            print(f"--- {section} (ms per call, device time, max over ranks; calls over {args.steps} steps)")
            for k, (ms, n) in rows:
                print(f"  {k[len(section) + 1:]:32s} {ms:9.3f} ms  x{n}")
        print("--- memory")
        for k, v in theory.items():
            print(f"  {k:32s} {v / 2 ** 20:10.1f} MiB (by construction)")
        print(f"  {'torch peak allocated':32s} {torch.cuda.max_memory_allocated() / 2 ** 20:10.1f} MiB")
        print(f"  {'torch reserved':32s} {torch.cuda.memory_reserved() / 2 ** 20:10.1f} MiB")
        print("--- throughput")
        print(f"  step {step_ms:.3f} ms, {tps:,.0f} tokens/s, {fpt / 1e9:.3f} GFLOP/token", end="")
        if peak:
            print(f", MFU {tps * fpt / (world * peak * 1e12):.3f} of {peak:.0f} TFLOP/s per GPU")
        else:
            print()
        if args.enable_trace:
            print(f"chrome trace written to {args.trace_path}")
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
