"""GPT pre-training entry point.

    torchrun --nproc_per_node=N train.py --data-path train.bin --tensor-model-parallel-size P ...

The flags of the reference (train.py:29-56) are kept with the same names and defaults;
everything else is additive. Without ``torchrun`` the script runs as a single process.
"""
from __future__ import annotations

import argparse
import os
import time

import torch
import torch.distributed as dist

from gpt_from_scratch_b200.checkpoint import latest_step, load_checkpoint, save_checkpoint
from gpt_from_scratch_b200.config import GPTConfig
from gpt_from_scratch_b200.data import PrefetchLoader, create_distributed_dataloader, write_synthetic_tokens
from gpt_from_scratch_b200.engine import TrainEngine
from gpt_from_scratch_b200.parallel import parallel_state as ps
from gpt_from_scratch_b200.utils.health import default_heartbeat
from gpt_from_scratch_b200.utils.logging import JsonlLogger, format_step_line, print_rank0


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="gpt_from_scratch_b200 GPT training")
    # model (reference flags)
    p.add_argument("--vocab-size", type=int, default=50304)
    p.add_argument("--hidden-size", type=int, default=768)
    p.add_argument("--num-layers", type=int, default=12)
    p.add_argument("--num-attention-heads", type=int, default=12)
    p.add_argument("--max-position-embeddings", type=int, default=1024)
    p.add_argument("--intermediate-size", type=int, default=3072)
    # training (reference flags)
    p.add_argument("--data-path", type=str, default=None, help="uint16 token file (.bin)")
    p.add_argument("--seq-len", type=int, default=1024)
    p.add_argument("--batch-size", type=int, default=8, help="micro batch per data-parallel rank")
    p.add_argument("--num-workers", type=int, default=4)
    p.add_argument("--lr", type=float, default=3e-4)
    p.add_argument("--weight-decay", type=float, default=0.1)
    p.add_argument("--max-steps", type=int, default=100000)
    p.add_argument("--clip-grad", type=float, default=1.0)
    p.add_argument("--log-interval", type=int, default=10)
    # parallelism (reference flag)
    p.add_argument("--tensor-model-parallel-size", type=int, default=1)
    # additions
    p.add_argument("--seed", type=int, default=1234)
    p.add_argument("--init-method", choices=["xavier_uniform", "normal"], default="xavier_uniform")
    p.add_argument("--init-std", type=float, default=0.02)
    p.add_argument("--dtype", choices=["bf16", "fp32"], default=None, help="default: bf16 on CUDA, fp32 on CPU")
    p.add_argument("--backend", choices=["nccl", "gloo"], default=None)
    p.add_argument("--device", choices=["cuda", "cpu"], default=None)
    p.add_argument("--attention-impl", choices=["fused", "torch"], default="fused")
    p.add_argument("--comm-impl", choices=["fused", "nccl"], default="nccl",
                   help="fused: peer-memory kernels that overlap the collective with the GEMM")
    p.add_argument("--cuda-graph", action="store_true",
                   help="capture the whole step in a CUDA graph after a few eager steps (one launch per step)")
    p.add_argument("--synthetic-data", action="store_true", help="generate a seeded random token file")
    p.add_argument("--synthetic-tokens", type=int, default=None)
    p.add_argument("--dp-grad-reduce", choices=["sum", "mean"], default="sum")
    p.add_argument("--reference-quirks", action="store_true")
    p.add_argument("--dropout-prob", type=float, default=0.0)
    p.add_argument("--rms-norm-eps", type=float, default=1e-5)
    p.add_argument("--save-dir", type=str, default=None)
    p.add_argument("--save-interval", type=int, default=0)
    p.add_argument("--load", type=str, default=None, help="checkpoint directory to resume from")
    p.add_argument("--log-jsonl", type=str, default=None)
    p.add_argument("--peak-tflops", type=float, default=None, help="per-GPU peak for the MFU column")
    p.add_argument("--heartbeat-timeout", type=float, default=300.0,
                   help="seconds a peer may lag behind at a log interval before PeerFailure is raised "
                        "(0 disables the heartbeat)")
    return p.parse_args(argv)


def build_config(args) -> GPTConfig:
    return GPTConfig(
        vocab_size=args.vocab_size, hidden_size=args.hidden_size, num_layers=args.num_layers,
        num_attention_heads=args.num_attention_heads,
        max_position_embeddings=max(args.max_position_embeddings, args.seq_len),
        intermediate_size=args.intermediate_size, rms_norm_eps=args.rms_norm_eps,
        dropout_prob=args.dropout_prob, init_method=args.init_method, init_std=args.init_std,
        attention_impl=args.attention_impl, reference_quirks=args.reference_quirks)


def init_distributed(args):
    use_cuda = (args.device or ("cuda" if torch.cuda.is_available() else "cpu")) == "cuda"
    if "RANK" in os.environ and "WORLD_SIZE" in os.environ:
        backend = args.backend or ("nccl" if use_cuda else "gloo")
        local_rank = int(os.environ.get("LOCAL_RANK", 0))
        if use_cuda:
            torch.cuda.set_device(local_rank)
        dist.init_process_group(backend=backend)
    if use_cuda:
        ps.set_device(torch.device("cuda", torch.cuda.current_device()))
    else:
        ps.set_device("cpu")
    ps.initialize_parallel_state(args.tensor_model_parallel_size)
    ps.set_seed(args.seed)
    ps.set_comm_impl(args.comm_impl)
    return use_cuda


def main(argv=None):
    args = parse_args(argv)
    use_cuda = init_distributed(args)
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    tp = args.tensor_model_parallel_size
    dp = world // tp
    print_rank0(f"World size: {world}, TP size: {tp}, DP size: {dp}")

    dtype = {"bf16": torch.bfloat16, "fp32": torch.float32, None: torch.bfloat16 if use_cuda else torch.float32}[
        args.dtype]
    config = build_config(args)
    engine = TrainEngine(config, lr=args.lr, weight_decay=args.weight_decay, betas=(0.9, 0.95),
                         clip_grad=args.clip_grad, dtype=dtype, grad_reduce=args.dp_grad_reduce, seed=args.seed,
                         cuda_graph=args.cuda_graph)
    print_rank0(f"Model params (per TP rank): {engine.params_per_tp_rank / 1e6:.1f}M")

    data_path = args.data_path
    if args.synthetic_data or data_path is None:
        data_path = data_path or os.path.join("/tmp", f"gfs_synth_{args.seed}_{args.seq_len}.bin")
        if rank == 0:
            n = args.synthetic_tokens or (args.seq_len * args.batch_size * dp * 64 + 1)
            write_synthetic_tokens(data_path, n, min(args.vocab_size, 50257), args.seed)
        if dist.is_initialized():
            dist.barrier()
    loader, sampler = create_distributed_dataloader(data_path, args.seq_len, args.batch_size, args.num_workers,
                                                    seed=args.seed)
    print_rank0(f"Dataset loaded: {len(loader.dataset)} samples, {len(loader)} batches/epoch")

    step = 0
    epoch = 0
    batches_in_epoch = 0      # batches of the current epoch already consumed (saved for resume)
    if args.load and latest_step(args.load) is not None:
        payload = load_checkpoint(args.load, engine.model, engine.optimizer)
        step = payload["step"]
        epoch = payload.get("extra", {}).get("epoch", 0)
        batches_in_epoch = payload.get("extra", {}).get("batches_in_epoch", 0)
        print_rank0(f"Resumed from {args.load} at step {step} (epoch {epoch}, batch {batches_in_epoch})")
    heartbeat = default_heartbeat(args.heartbeat_timeout) if args.heartbeat_timeout > 0 else None
    print_rank0(f"Starting training for {args.max_steps} steps...")

    jsonl = JsonlLogger(args.log_jsonl)
    device = engine.device
    batches = PrefetchLoader(loader, device) if use_cuda else loader
    log_loss = torch.zeros((), dtype=torch.float32, device=device)
    log_start = time.time()
    flops_per_token = config.flops_per_token(args.seq_len)
    while step < args.max_steps:
        sampler.set_epoch(epoch)
        if batches_in_epoch:
            if batches_in_epoch >= len(loader):     # the checkpoint was written at the epoch's last batch
                epoch, batches_in_epoch = epoch + 1, 0
                continue
            sampler.skip_samples(batches_in_epoch * args.batch_size)
        for batch in batches:
            if step >= args.max_steps:
                break
            inputs = batch["input"].to(device, non_blocking=True)
            labels = batch["label"].to(device, non_blocking=True)
            loss = engine.train_step(inputs, labels)
            step += 1
            batches_in_epoch += 1
            log_loss += loss.float()
            if heartbeat is not None:
                heartbeat.beat(step)
            if step % args.log_interval == 0:
                if heartbeat is not None:
                    # every peer must have finished this step before the next collective is
                    # launched: raises PeerFailure instead of hanging on a dead or stalled rank
                    heartbeat.wait_for_peers(step)
                avg_loss = float(log_loss) / args.log_interval     # one host sync per log interval
                elapsed = time.time() - log_start
                tps = args.log_interval * args.batch_size * args.seq_len * dp / elapsed
                print_rank0(format_step_line(step, args.max_steps, avg_loss, tps, elapsed))
                rec = {"step": step, "loss": avg_loss, "tokens_per_sec": tps, "seconds": elapsed}
                if engine.optimizer.last_grad_norm is not None:
                    rec["grad_norm"] = float(engine.optimizer.last_grad_norm)
                if args.peak_tflops:
                    rec["mfu"] = tps * flops_per_token / (world * args.peak_tflops * 1e12)
                if use_cuda:
                    rec["peak_mem_gb"] = torch.cuda.max_memory_allocated() / 2 ** 30
                    from gpt_from_scratch_b200.ops import _lib
                    code, detail = _lib.read_status(clear=False)
                    rec["device_status"] = code
                    if code != 0:
                        raise RuntimeError(f"a kernel reported status {code} ({_lib.STATUS_NAMES.get(code)})")
                jsonl.log(**rec)
                log_loss.zero_()
                log_start = time.time()
            if args.save_dir and args.save_interval and step % args.save_interval == 0:
                save_checkpoint(args.save_dir, step, engine.model, engine.optimizer,
                                {"epoch": epoch, "batches_in_epoch": batches_in_epoch})
        epoch += 1
        batches_in_epoch = 0

    print_rank0("Training finished.")
    jsonl.close()
    if dist.is_initialized():
        dist.barrier()      # rank 0 hosts the key-value store: it must not leave while peers still read it
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
