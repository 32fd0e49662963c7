"""Microbenchmark of the fused compute + collective operators against their rooflines.

    torchrun --nnodes=1 --nproc-per-node P --master-addr 127.0.0.1 -m gpt_from_scratch_b200.fused_bench \
        [--hidden 768 --ffn 3072 --vocab 50304 --tokens 8192] [--iters 20]

Every operator is run forward-only with TP = world on synthetic bf16 data, timed with CUDA
events on the launching stream after warm-up (a buffer larger than L2 is rewritten between
timed launches; a device-side delay in front of the first event lets the host enqueue the
operator ahead of time), and the MAX over ranks is reported next to the same operation built from an
NCCL collective plus the plain GEMM (``--comm-impl nccl`` path). The roofline of a fused path
is the slower of (FLOPs / measured GEMM peak) and (bytes that must cross NVLink per GPU /
measured peer-copy bandwidth, 770 GB/s per direction here); ``frac`` = roofline time
/ measured time.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .ops import gemm as gemm_ops
from .parallel import fused_comm, mappings
from .parallel import parallel_state as ps
from .parallel.layers import VocabParallelEmbedding

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LINK_BYTES_PER_S = 770e9


def gemm_peak() -> float:
    try:
        with open(os.path.join(REPO, "MEASURED_PEAKS.json")) as f:
            return json.load(f)["bf16_tflops"] * 1e12
    except Exception:
        return 1.59e15


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=768)
    ap.add_argument("--ffn", type=int, default=3072)
    ap.add_argument("--vocab", type=int, default=50304)
    ap.add_argument("--tokens", type=int, default=8192, help="global tokens S*B (rows of the gathered activations)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    ps.set_device(dev)
    ps.initialize_parallel_state(world)
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    peak = gemm_peak()

    def timed(fn) -> float:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        total = 0.0
        for _ in range(args.iters):
            flush.zero_()
            dist.barrier()          # ranks enter the operator together, as inside a training step
            # a short device-side delay in front of the timed region: the host enqueues the
            # operator while the GPU is still busy, so launch latency is not part of the number
            torch.cuda._sleep(600_000)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        t = torch.tensor([total / args.iters * 1e3], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    H, I, V, M, B = args.hidden, args.ffn, args.vocab, args.tokens, args.batch
    S = M // B
    Ms = M // world
    g = torch.Generator(device="cuda").manual_seed(1 + rank)
    rnd = lambda *s: (torch.randn(*s, device=dev, generator=g) * 0.05).bfloat16()  # noqa: E731
    rows = []

    def bench_ag(name, N, K):
        x_shard, w = rnd(Ms // B, B, K), rnd(N // world, K)
        flops = 2.0 * M * (N // world) * K
        link = (M - Ms) * K * 2          # bytes every GPU receives
        ps.set_comm_impl("fused")
        t_f = timed(lambda: fused_comm.allgather_linear(x_shard, w))
        ps.set_comm_impl("nccl")
        t_n = timed(lambda: gemm_ops.linear_fwd(mappings.gather_from_sequence_parallel_region(x_shard).view(M, K), w))
        rows.append((name, t_f, t_n, flops, link))

    def bench_rs(name, N, K):
        x, w, res = rnd(S, B, K // world), rnd(N, K // world), rnd(Ms // B, B, N)
        flops = 2.0 * M * N * (K // world)
        link = (M - Ms) * N * 2          # bf16 partial rows every GPU sends
        ps.set_comm_impl("fused")
        t_f = timed(lambda: fused_comm.linear_reduce_scatter(x, w, res))
        ps.set_comm_impl("nccl")
        t_n = timed(lambda: mappings.reduce_scatter_to_sequence_parallel_region(
            gemm_ops.linear_fwd(x.view(M, K // world), w).view(S, B, N)) + res)
        rows.append((name, t_f, t_n, flops, link))

    with torch.no_grad():
        bench_ag("all-gather -> GEMM   QKV      ", 3 * H, H)
        bench_ag("all-gather -> GEMM   gate_up  ", 2 * I, H)
        bench_ag("all-gather -> GEMM   LM head  ", V, H)
        # LM head + local cross-entropy statistics: statistics in the all-gather GEMM's epilogue vs
        # the plain fused all-gather GEMM followed by one pass over the logits ("nccl us" column)
        from .ops import cross_entropy as ce_ops
        x_lm, w_lm = rnd(Ms // B, B, H), rnd(V // world, H)
        tgt = torch.randint(0, V, (M,), device=dev, generator=torch.Generator(device="cuda").manual_seed(9))
        v0 = rank * (V // world)
        ps.set_comm_impl("fused")

        def lm_epilogue_stats():
            out, partials = fused_comm.allgather_linear(x_lm, w_lm, ce_stats=True)
            return ce_ops.ce_stats_from_partials(partials, out.view(M, -1), tgt, v0, False)

        def lm_then_pass():
            out = fused_comm.allgather_linear(x_lm, w_lm)
            return ce_ops.ce_local_stats(out.view(M, -1), tgt, v0, False)
        t_f, t_n = timed(lm_epilogue_stats), timed(lm_then_pass)
        rows.append(("AG -> GEMM LM head + CE stats (vs + pass)", t_f, t_n, 2.0 * M * (V // world) * H,
                     (M - Ms) * H * 2))
        bench_rs("GEMM -> reduce-scatter out_proj (+res)", H, H)
        bench_rs("GEMM -> reduce-scatter down     (+res)", H, I)
        # embedding lookup -> reduce-scatter
        emb = VocabParallelEmbedding(V, H)
        emb.weight.data = emb.weight.data.bfloat16()
        ids = torch.randint(0, V, (B, S), device=dev, generator=torch.Generator(device="cuda").manual_seed(7))
        link = (M - Ms) * H * 2 // world  # rows owned by other ranks' vocabulary slices, on average
        ps.set_comm_impl("fused")
        t_f = timed(lambda: emb(ids))
        ps.set_comm_impl("nccl")
        t_n = timed(lambda: emb(ids))
        rows.append(("embedding -> reduce-scatter            ", t_f, t_n, 0.0, link))
        # cross-entropy statistics exchange
        stats = torch.randn(M, 3, device=dev, generator=g)
        ps.set_comm_impl("fused")
        t_f = timed(lambda: fused_comm.ce_exchange_combine(stats))

        def nccl_ce():
            allst = torch.empty((world, M, 3), dtype=stats.dtype, device=dev)
            dist.all_gather_into_tensor(allst, stats, group=ps.get_tensor_model_parallel_group())
            from .ops import cross_entropy as ce_ops
            return ce_ops.ce_combine(allst)
        t_n = timed(nccl_ce)
        rows.append(("CE statistics exchange + combine       ", t_f, t_n, 0.0, (world - 1) * M * 12))

    if rank == 0:
        print(f"world {world}, tokens {M} (S {S} x B {B}), hidden {H}, ffn {I}, vocab {V}; "
              f"GEMM peak {peak / 1e12:.0f} TFLOP/s, link {LINK_BYTES_PER_S / 1e9:.0f} GB/s per direction")
        print(f"{'operator':42s} {'fused us':>9s} {'nccl us':>9s} {'roofline us':>11s} {'bound':>8s} {'frac':>5s}")
        for name, t_f, t_n, flops, link in rows:
            t_c, t_l = flops / peak * 1e6, link / LINK_BYTES_PER_S * 1e6
            roof = max(t_c, t_l)
            print(f"{name:42s} {t_f:9.1f} {t_n:9.1f} {roof:11.1f} {'compute' if t_c >= t_l else 'link':>8s} "
                  f"{roof / t_f:5.2f}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
