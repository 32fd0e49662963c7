"""Training-throughput benchmark: whole-job tokens/s of one optimisation step
(zero_grad, forward, vocab-parallel cross entropy, backward, distributed optimizer step),
timed on the device with CUDA events, maximum over ranks.

    python bench.py                       # 1 GPU, default steps
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Default workload: GPT-124M shape (12 layers, hidden 768, 12 heads, SwiGLU 3072, vocab 50304,
sequence 1024), micro-batch 16 per GPU, TP=1 x DP=N, bf16 compute with fp32 master weights
in the sharded optimizer; weak scaling (per-GPU work fixed). Data: seeded uniform-random
token ids in [0, 50257); weights: random init.

``--impl reference`` runs the unmodified reference implementation installed under
``baseline/_ref`` (its GPTModel, DistributedOptimizer, Triton attention/RoPE, NCCL) on the
same workload with the same timing harness and prints the same JSON line.

The JSON line carries two measurements: ``value`` (inputs already resident on the device)
and ``e2e`` (every step copies its token batch from pinned host memory and reads the loss
back to the host). With N >= 2 GPUs and the default config the same processes then rebuild the
model as TP=2 (+ sequence parallel) x DP=N/2 with micro-batch 8 and report that layout's numbers
under ``"tp"`` (same fields), for either ``--impl``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist

REPO = os.path.dirname(os.path.abspath(__file__))

CONFIGS = {
    # name: (layers, hidden, heads, ffn, vocab, seq, micro_batch, tp)
    "gpt124m": dict(num_layers=12, hidden_size=768, num_attention_heads=12, intermediate_size=3072,
                    vocab_size=50304, seq_len=1024, micro_batch=16, tp=1),
    "gpt124m_tp2": dict(num_layers=12, hidden_size=768, num_attention_heads=12, intermediate_size=3072,
                        vocab_size=50304, seq_len=1024, micro_batch=8, tp=2),
    "gpt1p3b_tp8": dict(num_layers=24, hidden_size=2048, num_attention_heads=16, intermediate_size=5632,
                        vocab_size=50304, seq_len=2048, micro_batch=4, tp=8),
    "gpt7b_tp4": dict(num_layers=32, hidden_size=4096, num_attention_heads=32, intermediate_size=11008,
                      vocab_size=50304, seq_len=4096, micro_batch=1, tp=4),
    "tiny": dict(num_layers=2, hidden_size=256, num_attention_heads=4, intermediate_size=512,
                 vocab_size=1024, seq_len=256, micro_batch=2, tp=1),
}
TOKEN_ID_RANGE = 50257


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", choices=["ours", "reference"], default="ours")
    p.add_argument("--config", choices=sorted(CONFIGS), default="gpt124m")
    p.add_argument("--tp", type=int, default=None, help="override the config's tensor-parallel size")
    p.add_argument("--micro-batch", type=int, default=None)
    p.add_argument("--comm-impl", choices=["fused", "nccl"], default=None)
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-graph", action="store_true",
                   help="ours: launch every kernel from Python instead of replaying the captured step")
    p.add_argument("--no-tp", action="store_true",
                   help="skip the tensor-parallel (TP2 x DP N/2) sub-measurement that runs for N >= 2")
    return p.parse_args()


def flops_per_token(c) -> float:
    H, I, L, V, S = c["hidden_size"], c["intermediate_size"], c["num_layers"], c["vocab_size"], c["seq_len"]
    return 3.0 * (L * (2.0 * (4 * H * H + 3 * H * I) + 2.0 * S * H) + 2.0 * H * V)


def measured_peak_tflops() -> float | None:
    try:
        with open(os.path.join(REPO, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops"])
    except Exception:
        return None


def setup_dist(n_gpus: int, force_init: bool):
    """Returns (rank, world, local_rank). Initialises NCCL when launched by torchrun, or
    (force_init) as a single-rank group for code that requires a process group."""
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local_rank)
    if "RANK" in os.environ and int(os.environ.get("WORLD_SIZE", "1")) >= 1 and "MASTER_ADDR" in os.environ:
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local_rank))
    elif force_init:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        os.environ["RANK"] = "0"
        os.environ["WORLD_SIZE"] = "1"
        os.environ["LOCAL_RANK"] = "0"
        dist.init_process_group(backend="nccl", rank=0, world_size=1)
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    if world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} but the job has {world} rank(s); launch with torchrun for N > 1")
    return rank, world, local_rank


def make_batches(n: int, micro_batch: int, seq_len: int, seed: int):
    """n pinned host batches of int64 token ids: (inputs [B,S], labels [B,S])."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        t = torch.randint(0, TOKEN_ID_RANGE, (micro_batch, seq_len + 1), generator=g, dtype=torch.int64)
        out.append((t[:, :-1].contiguous().pin_memory(), t[:, 1:].contiguous().pin_memory()))
    return out


def barrier_sync():
    if dist.is_initialized():
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x: float) -> float:
    if dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return x


def timed_loop(step_fn, batches, steps, stage: str):
    """Runs `steps` steps; returns device milliseconds (CUDA events, max over ranks)."""
    dev = torch.device("cuda", torch.cuda.current_device())
    if stage == "device":
        staged = [(a.to(dev), b.to(dev)) for a, b in batches[:steps]]
    barrier_sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    last = None
    step_async = getattr(step_fn, "step_async", None)
    pending = None
    for i in range(steps):
        if stage == "device":
            x, y = staged[i]
            last = step_fn(x, y)
        else:
            hx, hy = batches[i % len(batches)]
            x = hx.to(dev, non_blocking=True)
            y = hy.to(dev, non_blocking=True)
            if step_async is not None:
                # every step copies its loss device -> pinned host memory (asynchronously); the
                # host reads the value of step i while step i+1 is already queued, the last one
                # before the closing event
                handle = step_async(x, y)
                if pending is not None:
                    last = pending.value()
                pending = handle
            else:
                last = float(step_fn(x, y))     # device -> host read of this step's loss (blocking)
    if pending is not None:
        last = pending.value()
    e1.record()
    barrier_sync()
    return max_over_ranks(e0.elapsed_time(e1)), last


def build_ours(cfgd, args, world):
    sys.path.insert(0, REPO)
    from gpt_from_scratch_b200.config import GPTConfig
    from gpt_from_scratch_b200.engine import TrainEngine
    from gpt_from_scratch_b200.ops import _lib
    from gpt_from_scratch_b200.parallel import parallel_state as ps
    ps.set_device(torch.device("cuda", torch.cuda.current_device()))
    ps.initialize_parallel_state(cfgd["tp"])
    if args.comm_impl:
        ps.set_comm_impl(args.comm_impl)
    elif world > 1:
        ps.set_comm_impl(os.environ.get("GFS_COMM_IMPL", "fused"))
    _lib.lib()
    cfg = GPTConfig(vocab_size=cfgd["vocab_size"], hidden_size=cfgd["hidden_size"], num_layers=cfgd["num_layers"],
                    num_attention_heads=cfgd["num_attention_heads"], max_position_embeddings=cfgd["seq_len"],
                    intermediate_size=cfgd["intermediate_size"])
    engine = TrainEngine(cfg, lr=3e-4, weight_decay=0.1, betas=(0.9, 0.95), clip_grad=1.0, dtype=torch.bfloat16,
                         seed=1234, cuda_graph=not args.no_graph, graph_warmup=2)

    def step_fn(x, y):
        return engine.train_step(x, y)
    step_fn.step_async = engine.train_step_async   # loss via asynchronous copy to pinned memory

    def launches():
        return _lib.launch_count()

    def check():
        _lib.raise_on_status()
    return step_fn, launches, check, ps.get_comm_impl()


def build_reference(cfgd, args):
    ref_root = os.path.join(REPO, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "core")):
        return None, "baseline/_ref is missing (reference not installed)"
    # the reference's `core` is a namespace package (no __init__.py); this repository's own
    # `core/` alias package would shadow it, so the repository root leaves the import path
    sys.path[:] = [ref_root] + [q for q in sys.path if os.path.abspath(q or ".") != REPO]
    for name in [m for m in sys.modules if m == "core" or m.startswith("core.") or m == "train"]:
        del sys.modules[name]
    try:
        import train as ref_train
        from core.models.gpt import GPTModel
        from core.optimizer import DistributedOptimizer
        from core.parallel_state import initialize_parallel_state
        from core.tensor_parallel.loss import _VocabParallelCrossEntropy
    except Exception as e:  # noqa: BLE001
        return None, f"reference import failed: {type(e).__name__}: {e}"
    initialize_parallel_state(cfgd["tp"])
    ns = argparse.Namespace(tensor_model_parallel_size=cfgd["tp"], num_attention_heads=cfgd["num_attention_heads"],
                            hidden_size=cfgd["hidden_size"], seq_len=cfgd["seq_len"])
    ref_train.warmup_triton(ns)
    config = ref_train.GPTConfig(vocab_size=cfgd["vocab_size"], hidden_size=cfgd["hidden_size"],
                                 num_layers=cfgd["num_layers"], num_attention_heads=cfgd["num_attention_heads"],
                                 max_position_embeddings=cfgd["seq_len"], intermediate_size=cfgd["intermediate_size"])
    model = GPTModel(config)
    optimizer = DistributedOptimizer(model=model, optimizer_cls=torch.optim.AdamW,
                                     optimizer_kwargs={"lr": 3e-4, "weight_decay": 0.1, "betas": (0.9, 0.95)},
                                     clip_grad=1.0)
    model.train()

    def step_fn(x, y):  # the reference's loop body, train.py:172-187
        optimizer.zero_grad()
        logits = model(x)
        labels_t = y.transpose(0, 1).contiguous()
        loss = _VocabParallelCrossEntropy.apply(logits, labels_t).mean()
        loss.backward()
        optimizer.step()
        return loss.detach()
    return step_fn, None


def release_ours():
    """Drop the engine of a finished measurement (model, optimizer, symmetric buffers, groups) so
    the next layout can be built in the same processes."""
    import gc
    from gpt_from_scratch_b200.ops import gemm as gemm_ops
    from gpt_from_scratch_b200.parallel import parallel_state as ps
    from gpt_from_scratch_b200.parallel import symm
    gemm_ops.flush_wgrad()
    torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()
    symm.reset()
    ps.destroy_model_parallel()
    gc.collect()
    torch.cuda.empty_cache()


def measure(config_name: str, cfgd: dict, args, rank: int, world: int, local_rank: int, with_e2e: bool):
    """Build the model in layout ``cfgd`` for ``args.impl`` and time it. Returns the fields of the
    JSON line that depend on the layout (``None`` plus a reason if the reference is unavailable)."""
    from gpt_from_scratch_b200.utils.timing import ClockSampler   # timing harness only (no kernels)
    tp = cfgd["tp"]
    dp = world // tp
    B, S = cfgd["micro_batch"], cfgd["seq_len"]
    launches = None
    check = None
    comm = "nccl"
    if args.impl == "ours":
        step_fn, launches, check, comm = build_ours(cfgd, args, world)
    else:
        step_fn, why = build_reference(cfgd, args)
        if step_fn is None:
            return None, why

    # TP peers read the same batch, DP replicas different ones
    dp_rank = rank // tp
    n_batches = max(args.steps, args.warmup, 4)
    batches = make_batches(n_batches, B, S, seed=4321 + dp_rank)

    timed_loop(step_fn, batches, args.warmup, "device")          # warm-up (untimed)
    if check:
        check()
    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    e2e = None
    if with_e2e:
        # the end-to-end loop is the headline and goes first; the resident-input loop after it
        # explains it (two identical loops run back to back have differed by a percent or two in
        # either direction on the same GPU, so the order is fixed rather than meaningful)
        ms_e2e, last_loss = timed_loop(step_fn, batches, args.steps, "e2e")
    l0 = launches() if launches else 0
    ms_dev, _ = timed_loop(step_fn, batches, args.steps, "device")
    n_launch = (launches() - l0) if launches else None
    clocks = sampler.stop() if sampler else None
    if check:
        check()

    tokens_per_step = B * S * dp
    value = tokens_per_step * args.steps / (ms_dev / 1e3)
    fpt = flops_per_token(cfgd)
    peak = measured_peak_tflops()
    if with_e2e:
        e2e = {"value": tokens_per_step * args.steps / (ms_e2e / 1e3), "unit": "tokens/s",
               "ms_per_step": ms_e2e / args.steps,
               "h2d_bytes_per_step": 2 * B * S * 8, "d2h_bytes_per_step": 4, "last_loss": last_loss,
               "loss_read": ("asynchronous copy to pinned memory every step, value read one step later "
                             "(TrainEngine.train_step_async)" if args.impl == "ours" else
                             "blocking read every step")}
    par = (f"tp{tp}" if tp > 1 else "") + (f"dp{dp}" if (dp > 1 or tp == 1) else "")
    out = {
        "value": value, "unit": "tokens/s", "ms_per_step": ms_dev / args.steps,
        "config": {"model": config_name, "layers": cfgd["num_layers"], "hidden": cfgd["hidden_size"],
                   "heads": cfgd["num_attention_heads"], "ffn": cfgd["intermediate_size"],
                   "vocab": cfgd["vocab_size"], "global_batch": B * dp, "micro_batch": B, "seq_len": S,
                   "parallelism": par, "optimizer": "AdamW, fp32 master weights, sharded over DP, clip 1.0",
                   "l2": "per-step working set (weights+grads+activations, >2 GB) exceeds the 126 MB L2; "
                         "no explicit flush"},
        # how the collectives and the launches are done: implementation labels, not workload
        "comm_impl": comm,
        "step_launch": ("CUDA graph replay of the whole step" if (args.impl == "ours" and not args.no_graph)
                        else "one host launch per kernel"),
        "mfu_of_measured_peak": (value * fpt / (world * peak * 1e12)) if peak else None,
        "flops_per_token": fpt,
        "clocks": clocks,
        "e2e": e2e,
        "gpu_launches": n_launch,
    }
    del step_fn
    return out, None


def main():
    args = parse_args()
    cfgd = dict(CONFIGS[args.config])
    if args.tp:
        cfgd["tp"] = args.tp
    if args.micro_batch:
        cfgd["micro_batch"] = args.micro_batch
    if not torch.cuda.is_available():
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "no CUDA device in this process"}))
            return
        raise SystemExit("bench.py needs a CUDA device")
    rank, world, local_rank = setup_dist(args.gpus, force_init=(args.impl == "reference"))
    if world % cfgd["tp"] != 0:
        raise SystemExit(f"{world} GPUs cannot host TP={cfgd['tp']}")

    head, why = measure(args.config, cfgd, args, rank, world, local_rank, with_e2e=not args.no_e2e)
    if head is None:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": why}))
        return

    # Second layout of the same model on the same GPUs: tensor parallel 2 (+ sequence parallel) x
    # data parallel N/2, micro-batch 8 per DP rank. It exercises the tensor-parallel collectives
    # (all-gather -> GEMM, GEMM -> reduce-scatter, embedding, cross entropy), which the data-parallel
    # headline layout does not touch. Reported under "tp"; the headline fields are unaffected.
    tp_block = None
    if world >= 2 and world % 2 == 0 and args.config == "gpt124m" and not args.tp and not args.no_tp:
        if args.impl == "ours":
            release_ours()
        else:
            import gc
            gc.collect()
            torch.cuda.empty_cache()
        tcfg = dict(CONFIGS["gpt124m_tp2"])
        try:
            tp_block, why = measure("gpt124m_tp2", tcfg, args, rank, world, local_rank, with_e2e=not args.no_e2e)
            if tp_block is None:
                tp_block = {"unavailable": why}
        except Exception as e:  # noqa: BLE001 - the headline number must survive a failure here
            tp_block = {"unavailable": f"{type(e).__name__}: {e}"[:300]}

    if rank == 0:
        line = {
            "metric": "train tokens/sec (whole job, device-timed, max over ranks)",
            "value": head["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform-random token ids in [0,50257), random-init weights",
            "config": head["config"],
            "impl": args.impl,
            "comm_impl": head["comm_impl"],
            "step_launch": head["step_launch"],
            "mfu_of_measured_peak": head["mfu_of_measured_peak"],
            "flops_per_token": head["flops_per_token"],
            "clocks": head["clocks"],
            "e2e": head["e2e"],
            "gpu_launches": head["gpu_launches"],
        }
        if tp_block is not None:
            line["tp"] = tp_block
        print(json.dumps(line))
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
