"""Run the fused compute+collective kernels on ONE GPU for profiling.

A profiler that replays kernels (Nsight Compute) cannot follow a multi-process job whose
kernels wait for each other. Here this process plays rank 0 of a group of ``--world`` ranks
whose other members are plain buffers on the same GPU with their flags pre-set
(``parallel/fake_peer.py``), so every fused kernel runs its real code path - push to the peers'
buffers, signal, wait, tensor-core tiles, reduce - to completion, alone. The peers' buffers are
local memory, so what would be NVLink traffic shows up as ordinary DRAM/L2 traffic:

    python -m gpt_from_scratch_b200.fused_profile --op ag_gemm --shape 7b --world 4 --iters 3
    ncu --set full --clock-control none -k regex:gemm2_kernel -c 2 -o prof \\
        python -m gpt_from_scratch_b200.fused_profile --op ag_gemm --shape 7b --world 4 --iters 2

Operators: ``ag_gemm`` (all-gather -> QKV GEMM), ``gemm_rs`` (out-projection GEMM ->
reduce-scatter + residual), ``mlp`` (the SwiGLU MLP: both of the above with the activation in the
epilogues, forward and backward), ``lm_head`` (all-gather -> LM-head GEMM with cross-entropy
statistics, fold, exchange), ``embedding`` (lookup -> reduce-scatter), ``dp`` (gradient push,
sum + norm, clip + AdamW + parameter all-gather). Each prints its CUDA-event time per launch
(host launch overhead included: these are eager calls).

``--trace`` (GEMM operators): instead of timing, run the operator once with the CTA-pair kernel's
phase stamps switched on (``gfs_gemm2_set_trace``) and print, per phase, the SM-clock cycles since
kernel entry over all CTAs (min / median / max) - where inside the kernel the time goes.
"""
from __future__ import annotations

import argparse

import torch

SHAPES = {
    # name: (tokens M over the whole TP group, hidden, heads, ffn, vocab)
    "124m": (8192, 768, 12, 3072, 50304),
    "1p3b": (8192, 2048, 16, 5632, 50304),
    "7b": (4096, 4096, 32, 11008, 50304),
}


def _time(fn, iters: int) -> float:
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


TRACE_SLOTS = ["global_ns", "entry", "setup_done", "first_tma", "first_mma", "epi_begin", "epi_first", "epi_last",
               "red_begin", "red_end", "push_done", "exit", "tiles"]


def trace_once(fn) -> None:
    """Run ``fn`` (one fused GEMM call) with the phase stamps on and print the per-phase table."""
    import ctypes
    from .ops import _lib
    lib = _lib.lib()
    lib.gfs_gemm2_set_trace.argtypes = [ctypes.c_void_p]
    lib.gfs_gemm2_set_trace.restype = None
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    n_cta = lib.gfs_sm_count()
    buf = torch.zeros(n_cta * 16, dtype=torch.int64, device="cuda")
    lib.gfs_gemm2_set_trace(buf.data_ptr())
    try:
        fn()
        torch.cuda.synchronize()
    finally:
        lib.gfs_gemm2_set_trace(None)
    t = buf.view(n_cta, 16).cpu()
    t = t[t[:, 1] != 0]
    print(f"CTAs {t.shape[0]}, kernel entry spread {int(t[:, 0].max() - t[:, 0].min())} ns, "
          f"tiles per CTA pair up to {int(t[:, 12].max())} (stamps of the LAST traced launch of the call)")
    print(f"{'phase':12s} {'min':>8s} {'median':>8s} {'max':>8s}   cycles since kernel entry")
    for slot in (2, 3, 4, 5, 6, 7, 10, 8, 9, 11):
        col = t[:, slot]
        ok = col != 0
        if int(ok.sum()) == 0:
            continue
        rel = (col[ok] - t[ok, 1]).float()
        print(f"{TRACE_SLOTS[slot]:12s} {int(rel.min()):8d} {int(rel.median()):8d} {int(rel.max()):8d}")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--trace", action="store_true", help="print the CTA-pair GEMM kernel's phase stamps instead")
    ap.add_argument("--op", required=True, choices=["ag_gemm", "gemm_rs", "mlp", "lm_head", "embedding", "dp"])
    ap.add_argument("--shape", choices=sorted(SHAPES), default="124m")
    ap.add_argument("--world", type=int, default=2)
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()

    from .ops import cross_entropy as ce_ops
    from .parallel import fused_comm
    from .parallel import parallel_state as ps
    from .parallel.fake_peer import fake_peers
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    ps.set_device(dev)
    ps.initialize_parallel_state(1)
    M, H, nh, I, V = SHAPES[a.shape]
    P = a.world
    Ms = M // P
    g = torch.Generator(device="cuda").manual_seed(0)
    rnd = lambda *s, scale=1.0: (torch.randn(*s, device=dev, generator=g) * scale).bfloat16()  # noqa: E731

    with fake_peers(P, 0):
        if a.op == "ag_gemm":
            x, w = rnd(Ms, H), rnd(3 * H // P, H, scale=0.05)
            if a.trace:
                return trace_once(lambda: fused_comm.allgather_linear(x, w))
            us = _time(lambda: fused_comm.allgather_linear(x, w), a.iters)
            flops = 2.0 * M * (3 * H // P) * H
        elif a.op == "gemm_rs":
            x, w, r = rnd(M, H // P), rnd(H, H // P, scale=0.05), rnd(Ms, H)
            if a.trace:
                return trace_once(lambda: fused_comm.linear_reduce_scatter(x, w, r))
            us = _time(lambda: fused_comm.linear_reduce_scatter(x, w, r), a.iters)
            flops = 2.0 * M * H * (H // P)
        elif a.op == "mlp":
            x = rnd(Ms, H).requires_grad_()
            w_gu, w_dn = rnd(2 * I // P, H, scale=0.05).requires_grad_(), rnd(H, I // P, scale=0.05).requires_grad_()
            r, dy = rnd(Ms, H), rnd(Ms, H)
            assert fused_comm.fused_mlp_eligible(x, w_gu, w_dn), "shape not served by the CTA-pair SwiGLU kernels"

            def step():
                fused_comm.swiglu_mlp(x, w_gu, w_dn, r).backward(dy)
            us = _time(step, a.iters)
            flops = 3 * 2.0 * M * (3 * I // P) * H
        elif a.op == "lm_head":
            x, w = rnd(Ms, H), rnd(V // P, H, scale=0.05)
            tgt = torch.randint(0, V, (M,), device=dev, generator=g)

            def step():
                logits, parts = fused_comm.allgather_linear(x, w, ce_stats=True)
                stats, _, _ = (ce_ops.ce_stats_from_partials(parts, logits, tgt, 0, False) if parts is not None
                               else ce_ops.ce_local_stats(logits, tgt, 0, False))
                return fused_comm.ce_exchange_combine(stats)
            us = _time(step, a.iters)
            flops = 2.0 * M * (V // P) * H
        elif a.op == "embedding":
            B = 8
            S = M // B
            ids = torch.randint(0, V, (B, S), device=dev, generator=g)

            class Emb:
                weight = rnd(V // P, H)
                vocab_start_index, vocab_end_index = 0, V // P
            us = _time(lambda: fused_comm.embedding_reduce_scatter(ids, Emb), a.iters)
            flops = 0.0
        else:  # dp
            n = (12 * (4 * H * H + 3 * H * I) // 8) // (64 * P) * (64 * P)     # an eighth of the layers' weights
            shard = n // P
            cut = n // 2 // (8 * P) * (8 * P)
            dpc = fused_comm.DataParallelComm(n, shard, dev, buckets=[(0, cut), (cut, n)])
            dpc.grad_buffer.copy_(rnd(n, scale=0.01))
            master = torch.randn(shard, device=dev, generator=g)
            m, v = torch.zeros_like(master), torch.zeros_like(master)

            def step():
                dpc.push_bucket(1)
                dpc.push_bucket(0)
                dpc.sum_and_norm()
                dpc.adam_and_gather(master, m, v, step=1, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8,
                                    weight_decay=0.1, clip=1.0, grad_scale=1.0)
            us = _time(step, a.iters)
            flops = 0.0
        torch.cuda.synchronize()
    from .ops import _lib
    code, detail = _lib.read_status()
    tf = f", {flops / us / 1e6:.0f} TFLOP/s" if flops else ""
    print(f"{a.op} shape={a.shape} world={P} (fake peers, one GPU): {us:.1f} us per call{tf}; device status {code}")


if __name__ == "__main__":
    main()
