"""Per-kernel microbenchmarks with roofline fractions.

    python -m gpt_from_scratch_b200.kernel_bench                 # all kernels, GPT-124M shapes
    python -m gpt_from_scratch_b200.kernel_bench --only gemm     # substring filter
    python -m gpt_from_scratch_b200.kernel_bench --small         # small shapes (for ncu captures)
    python -m gpt_from_scratch_b200.kernel_bench --vs-cublas     # every GEMM shape next to torch.matmul
    python -m gpt_from_scratch_b200.kernel_bench --vs-reference  # attention / RoPE next to the reference's Triton kernels

Each kernel is launched directly through the native library (no autograd), timed with CUDA
events after warm-up; between timed launches a buffer larger than the 126 MB L2 is
rewritten so every launch starts from a cold L2. Achieved bytes/s or FLOP/s are reported
as a fraction of the measured peaks in ``MEASURED_PEAKS.json`` (copy bandwidth, cuBLAS bf16
burst throughput), or of the fallback figures if that file is absent.
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch

from .ops import _lib
from .ops import adam as adam_ops
from .ops import cross_entropy as ce_ops
from .ops.attention import flash_bwd_native, flash_fwd_native
from .ops.embedding import embedding_bwd_native, embedding_fwd_native
from .ops.gemm import gemm_bf16
from .ops.mlp_fused import swiglu_gemm_bwd, swiglu_gemm_fwd
from .ops.rope import rope_inplace_native

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def peaks():
    try:
        with open(os.path.join(REPO, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    except Exception:
        return 6.65e12, 1.59e15, "fallback"


class Timer:
    def __init__(self, device):
        self.flush_buf = torch.empty(192 << 20, dtype=torch.uint8, device=device)  # > 126 MB L2

    def time_us(self, fn, iters=10, warmup=3):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(iters):
            self.flush_buf.zero_()
            # a device-side delay in front of the timed region: the host enqueues the launch while
            # the GPU is still busy, so Python launch latency is not part of a short kernel's number
            torch.cuda._sleep(600_000)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / iters * 1e3


def build_cases(dev, small: bool):
    """Returns a list of (name, fn, flops, bytes)."""
    g = torch.Generator(device="cuda").manual_seed(0)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g).bfloat16()  # noqa: E731
    if small:
        S, B, H, nh, I, V = 1024, 4, 768, 12, 3072, 8192
    else:
        S, B, H, nh, I, V = 1024, 16, 768, 12, 3072, 50304
    D = H // nh
    M = S * B
    cases = []

    def gemm_case(name, M_, N_, K_, a_mn=False, b_mn=False, add=False):
        a = rnd(K_, M_) if a_mn else rnd(M_, K_)
        b = rnd(K_, N_) if b_mn else rnd(N_, K_)
        out = torch.empty(M_, N_, device=dev, dtype=torch.bfloat16)
        fn = lambda: gemm_bf16(a, b, a_mn_major=a_mn, b_mn_major=b_mn, out=out, addend=out if add else None)  # noqa
        byt = 2 * (M_ * K_ + N_ * K_ + M_ * N_ * (2 if add else 1))
        cases.append((name, fn, 2.0 * M_ * N_ * K_, byt))

    gemm_case("gemm_fwd_qkv", M, 3 * H, H)
    gemm_case("gemm_fwd_out_residual", M, H, H, add=True)
    gemm_case("gemm_fwd_gate_up", M, 2 * I, H)
    gemm_case("gemm_fwd_down_residual", M, H, I, add=True)
    gemm_case("gemm_fwd_lm_head", M, V, H)
    from .ops.gemm import linear_fwd_ce
    xl, wl = rnd(M, H), rnd(V, H) * 0.05
    cases.append(("gemm_fwd_lm_head+ce_stats", lambda: linear_fwd_ce(xl, wl), 2.0 * M * V * H,
                  2 * (M * H + V * H + M * V)))
    gemm_case("gemm_dgrad_qkv", M, H, 3 * H, b_mn=True)
    gemm_case("gemm_dgrad_gate_up", M, H, 2 * I, b_mn=True)
    gemm_case("gemm_dgrad_down", M, I, H, b_mn=True)
    gemm_case("gemm_dgrad_lm_head", M, H, V, b_mn=True)
    gemm_case("gemm_wgrad_qkv_splitk", 3 * H, H, M, a_mn=True, b_mn=True)
    gemm_case("gemm_wgrad_gate_up", 2 * I, H, M, a_mn=True, b_mn=True)
    gemm_case("gemm_wgrad_lm_head", V, H, M, a_mn=True, b_mn=True)

    # fused MLP GEMMs
    x, wgu, wdn, dy = rnd(M, H), rnd(2 * I, H) * 0.05, rnd(H, I) * 0.05, rnd(M, H)
    gu, _ = swiglu_gemm_fwd(x, wgu)
    cases.append(("gemm_swiglu_fwd", lambda: swiglu_gemm_fwd(x, wgu), 2.0 * M * 2 * I * H,
                  2 * (M * H + 2 * I * H + 3 * M * I)))
    cases.append(("gemm_swiglu_bwd", lambda: swiglu_gemm_bwd(dy, wdn, gu), 2.0 * M * I * H,
                  2 * (M * H + I * H + 4 * M * I)))

    # attention
    qkv = rnd(S, B, 3, nh, D)
    out = torch.empty(S, B, nh, D, device=dev, dtype=torch.bfloat16)
    dout = rnd(S, B, nh, D)
    dqkv = torch.empty_like(qkv)
    scale = 1.0 / math.sqrt(D)
    lse = flash_fwd_native(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], out, True, scale)
    att_flops = 4.0 * S * S * D * B * nh / 2
    cases.append(("flash_fwd", lambda: flash_fwd_native(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], out, True, scale),
                  att_flops, 2 * 4 * S * B * nh * D))
    cases.append(("flash_bwd(dvec+dkdv+dq)",
                  lambda: flash_bwd_native(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], out, dout, lse, dqkv[:, :, 0],
                                           dqkv[:, :, 1], dqkv[:, :, 2], True, scale),
                  2.5 * att_flops, 2 * 8 * S * B * nh * D))

    # memory-bound kernels
    lib = _lib.lib()
    sp = _lib.stream_ptr
    xn, wn = rnd(M, H), torch.ones(H, device=dev, dtype=torch.bfloat16)
    yn = torch.empty_like(xn)
    rstd = torch.empty(M, device=dev)
    cases.append(("rmsnorm_fwd", lambda: lib.gfs_rmsnorm_fwd(xn.data_ptr(), wn.data_ptr(), yn.data_ptr(),
                                                             rstd.data_ptr(), M, H, 1e-5, sp()), 0, 4 * M * H))
    lib.gfs_rmsnorm_fwd(xn.data_ptr(), wn.data_ptr(), yn.data_ptr(), rstd.data_ptr(), M, H, 1e-5, sp())
    parts = lib.gfs_rmsnorm_bwd_parts(M)
    partial = torch.empty(parts * H, device=dev)
    dxn, dwn, dres = torch.empty_like(xn), torch.empty_like(wn), rnd(M, H)
    cases.append(("rmsnorm_bwd(+dres, +dw reduce)",
                  lambda: lib.gfs_rmsnorm_bwd(yn.data_ptr(), xn.data_ptr(), wn.data_ptr(), rstd.data_ptr(),
                                              dres.data_ptr(), dxn.data_ptr(), dwn.data_ptr(), partial.data_ptr(), M,
                                              H, 0, sp()), 0, 8 * M * H))
    gu2 = rnd(M, 2 * I)
    act2 = torch.empty(M, I, device=dev, dtype=torch.bfloat16)
    dgu2 = torch.empty_like(gu2)
    cases.append(("swiglu_fwd", lambda: lib.gfs_swiglu_fwd(gu2.data_ptr(), act2.data_ptr(), M, I, sp()), 0,
                  2 * 3 * M * I))
    cases.append(("swiglu_bwd", lambda: lib.gfs_swiglu_bwd(act2.data_ptr(), gu2.data_ptr(), dgu2.data_ptr(), M, I,
                                                           sp()), 0, 2 * 5 * M * I))
    ang = torch.rand(S, D // 2, device=dev)
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    cases.append(("rope_qk_inplace", lambda: rope_inplace_native(qkv, cos, sin, S, B, nh, D, 2, 3 * nh * D, False), 0,
                  2 * 2 * 2 * S * B * nh * D))
    logits = rnd(M, V)
    tgt = torch.randint(0, V, (M,), device=dev)
    stats, lse_ce, _ = ce_ops.ce_local_stats(logits, tgt, 0, True)
    grows = torch.full((M,), 1.0 / M, device=dev)
    cases.append(("ce_fwd", lambda: ce_ops.ce_local_stats(logits, tgt, 0, True), 0, 2 * M * V))
    n_parts = 2 * ((V + 255) // 256)
    ce_parts = torch.randn(n_parts, M, 2, device=dev).abs_()
    cases.append(("ce_from_gemm_partials", lambda: ce_ops.ce_stats_from_partials(ce_parts, logits, tgt, 0, True), 0,
                  8 * n_parts * M))
    cases.append(("ce_bwd_inplace", lambda: ce_ops.ce_backward_inplace(logits, lse_ce, tgt, grows, 0), 0, 4 * M * V))
    # parameter count of the benchmark model: 12 layers x (QKV + out + gate_up + down) + untied
    # embedding and LM head at vocab 50304 + norms
    # head_dim 128 at the two larger model shapes (per tensor-parallel rank): GPT-1.3B TP8
    # (B 4, 2 heads, S 2048) and GPT-7B TP4 (B 1, 8 heads, S 4096)
    for tag, (S2, B2, nh2) in (("1p3b_tp8", (2048, 4, 2)), ("7b_tp4", (4096, 1, 8))):
        if small:
            break
        cases.extend(attention_cases(dev, rnd, S2, B2, nh2, 128, f"_d128_{tag}"))

    n = 190_532_352 if not small else 8 * 1024 * 1024
    grad = rnd(n)
    master = torch.randn(n, device=dev)
    m1, m2 = torch.zeros_like(master), torch.zeros_like(master)
    pout = torch.empty(n, device=dev, dtype=torch.bfloat16)
    ss = torch.zeros(1, device=dev)
    cases.append(("sumsq_bf16", lambda: adam_ops.sumsq_bf16(grad, ss), 0, 2 * n))
    cases.append(("adamw_fused", lambda: adam_ops.adamw_step(grad, master, m1, m2, pout, step=3, lr=1e-4, beta1=0.9,
                                                             beta2=0.95, eps=1e-8, weight_decay=0.1, sumsq=ss,
                                                             clip=1.0), 0, 28 * n))
    ids = torch.randint(0, V, (B, S), device=dev)
    W = rnd(V, H)
    dW = torch.zeros_like(W)
    dsbh = rnd(S, B, H)
    cases.append(("embedding_fwd", lambda: embedding_fwd_native(ids, W, 0, V), 0, 4 * M * H))
    cases.append(("embedding_bwd(sort+segsum)", lambda: embedding_bwd_native(ids, dsbh, dW, 0, V, True), 0,
                  6 * M * H))
    return cases


def attention_cases(dev, rnd, S, B, nh, D, suffix):
    qkv = rnd(S, B, 3, nh, D)
    out = torch.empty(S, B, nh, D, device=dev, dtype=torch.bfloat16)
    dout = rnd(S, B, nh, D)
    dqkv = torch.empty_like(qkv)
    scale = 1.0 / math.sqrt(D)
    lse = flash_fwd_native(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], out, True, scale)
    att_flops = 4.0 * S * S * D * B * nh / 2
    return [("flash_fwd" + suffix,
             lambda: flash_fwd_native(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], out, True, scale),
             att_flops, 2 * 4 * S * B * nh * D),
            ("flash_bwd" + suffix,
             lambda: flash_bwd_native(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], out, dout, lse, dqkv[:, :, 0],
                                      dqkv[:, :, 1], dqkv[:, :, 2], True, scale),
             2.5 * att_flops, 2 * 8 * S * B * nh * D)]


def vs_reference(dev, timer, iters):
    """Head to head with the reference's own Triton kernels (its ``apply_flash_attn`` forward +
    backward and ``apply_rope_qk``, imported unmodified from ``baseline/_ref``) at the same shapes
    and with the same timing method. The reference's kernels autotune on first use: the warm-up
    launches absorb that. Its attention takes ``[B, nh, S, D]`` tensors and makes them contiguous
    (core/myFlashAttn.py:206-208); contiguous inputs are passed so no copy is timed."""
    import sys
    ref_root = os.path.join(REPO, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "core")):
        print("reference not installed under baseline/_ref: nothing to compare against")
        return
    sys.path[:] = [ref_root] + [q for q in sys.path if os.path.abspath(q or ".") != REPO]
    for name in [m for m in sys.modules if m == "core" or m.startswith("core.")]:
        del sys.modules[name]
    from core.myFlashAttn import apply_flash_attn as ref_attn
    from core.rope_triton import apply_rope_qk as ref_rope
    from .ops.attention import apply_flash_attn as our_attn
    g = torch.Generator(device="cuda").manual_seed(1)
    print(f"{'operator':40s} {'reference us':>13s} {'ours us':>9s} {'ratio':>6s}")
    for tag, (B, nh, S, D) in (("gpt124m  B16 nh12 S1024 D64", (16, 12, 1024, 64)),
                                ("gpt1.3b/TP8 B4 nh2 S2048 D128", (4, 2, 2048, 128)),
                                ("gpt7b/TP4 B1 nh8 S4096 D128", (1, 8, 4096, 128))):
        q, k, v = (torch.randn(B, nh, S, D, device=dev, generator=g).bfloat16().requires_grad_() for _ in range(3))
        do = torch.randn(B, nh, S, D, device=dev, generator=g).bfloat16()
        res = {}
        for who, fn in (("ref", ref_attn), ("ours", our_attn)):
            def fwd():
                return fn(q, k, v, True)

            def fwd_bwd():
                fn(q, k, v, True).backward(do)
            try:
                t_f = timer.time_us(fwd, iters=iters, warmup=4)
                t_fb = timer.time_us(fwd_bwd, iters=iters, warmup=4)
                res[who] = (t_f, t_fb - t_f)
            except Exception as e:  # noqa: BLE001 - a reference failure is a result to report
                res[who] = f"{type(e).__name__}: {str(e)[:120]}"
        for idx, what in ((0, "flash attention fwd"), (1, "flash attention bwd (fwd+bwd minus fwd)")):
            r, o = res["ref"], res["ours"]
            if isinstance(r, str) or isinstance(o, str):
                print(f"{what + ' ' + tag:40s} reference: {r if isinstance(r, str) else r[idx]}  ours: "
                      f"{o if isinstance(o, str) else o[idx]}")
            else:
                print(f"{(what + ' ' + tag)[:60]:60s} {r[idx]:9.1f} {o[idx]:9.1f} {r[idx] / o[idx]:6.2f}x")
    # RoPE on q and k of the GPT-124M shape: the reference rotates [S, B, nh, D] views with two launches
    from .ops.rope import rope_inplace_native
    S, B, nh, D = 1024, 16, 12, 64
    qkv = torch.randn(S, B, 3, nh, D, device=dev, generator=g).bfloat16()
    pos = torch.arange(S, device=dev, dtype=torch.float32)
    ang = pos[:, None] * (10000.0 ** (-torch.arange(0, D, 2, device=dev, dtype=torch.float32) / D))[None, :]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    qv, kv = qkv[:, :, 0], qkv[:, :, 1]
    cos_b, sin_b = cos.bfloat16(), sin.bfloat16()      # the reference rounds its tables to the activation dtype
    t_ref = timer.time_us(lambda: ref_rope(qv, kv, cos_b, sin_b), iters=iters, warmup=4)
    t_our = timer.time_us(lambda: rope_inplace_native(qkv, cos, sin, S, B, nh, D, parts=2, token_stride=3 * nh * D,
                                                      backward=False), iters=iters, warmup=4)
    print(f"{'rope q,k fwd gpt124m (ours: in place; in training folded into the QKV GEMM)':60s} "
          f"{t_ref:9.1f} {t_our:9.1f} {t_ref / t_our:6.2f}x")


def vs_cublas(dev, timer, iters: int, small: bool) -> None:
    """Every GEMM shape of the training step next to cuBLAS (``torch.matmul`` / ``torch.addmm`` on
    the same operands and layouts; the residual GEMMs are compared against matmul + add, which is
    what a framework without the epilogue launches)."""
    g = torch.Generator(device="cuda").manual_seed(0)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g).bfloat16()  # noqa: E731
    if small:
        S, B, H, I, V = 1024, 4, 768, 3072, 8192
    else:
        S, B, H, I, V = 1024, 16, 768, 3072, 50304
    M = S * B
    shapes = [("fwd qkv", M, 3 * H, H, False, False, False), ("fwd out + residual", M, H, H, False, False, True),
              ("fwd gate_up", M, 2 * I, H, False, False, False), ("fwd down + residual", M, H, I, False, False, True),
              ("fwd lm_head", M, V, H, False, False, False),
              ("dgrad qkv", M, H, 3 * H, False, True, False), ("dgrad gate_up", M, H, 2 * I, False, True, False),
              ("dgrad down", M, I, H, False, True, False), ("dgrad lm_head", M, H, V, False, True, False),
              ("wgrad gate_up", 2 * I, H, M, True, True, False), ("wgrad down", H, I, M, True, True, False),
              ("wgrad lm_head", V, H, M, True, True, False)]
    print(f"{'GEMM (M x N x K)':44s} {'cuBLAS us':>10s} {'ours us':>9s} {'ratio':>6s} {'ours TFLOP/s':>13s}")
    for name, M_, N_, K_, a_mn, b_mn, add in shapes:
        a = rnd(K_, M_) if a_mn else rnd(M_, K_)
        b = rnd(K_, N_) if b_mn else rnd(N_, K_)
        out = torch.empty(M_, N_, device=dev, dtype=torch.bfloat16)
        res = rnd(M_, N_) if add else None
        a_op = a.t() if a_mn else a                   # logical [M, K]
        b_op = b if b_mn else b.t()                   # logical [K, N]

        def ref():
            torch.matmul(a_op, b_op, out=out)
            if add:
                out.add_(res)

        def ours():
            gemm_bf16(a, b, a_mn_major=a_mn, b_mn_major=b_mn, out=out, addend=res)
        t_ref = timer.time_us(ref, iters=iters)
        t_our = timer.time_us(ours, iters=iters)
        tag = f"{name} ({M_} x {N_} x {K_})"
        print(f"{tag:44s} {t_ref:10.1f} {t_our:9.1f} {t_ref / t_our:6.2f}x {2.0 * M_ * N_ * K_ / t_our / 1e6:13.1f}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--vs-reference", action="store_true",
                    help="time the reference's Triton attention / RoPE (baseline/_ref) next to ours")
    ap.add_argument("--vs-cublas", action="store_true",
                    help="time cuBLAS (torch.matmul) on every GEMM shape of the step next to ours")
    ap.add_argument("--only", default=None)
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--once", action="store_true", help="launch every selected kernel once, no timing (for ncu)")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    bw, fl, kind = peaks()
    if args.vs_reference:
        vs_reference(dev, Timer(dev), args.iters)
        return
    if args.vs_cublas:
        vs_cublas(dev, Timer(dev), args.iters, args.small)
        return
    cases = build_cases(dev, args.small)
    if args.only:
        cases = [c for c in cases if args.only in c[0]]
    if args.once:
        for name, fn, _, _ in cases:
            fn()
        torch.cuda.synchronize()
        print("launched", [c[0] for c in cases])
        return
    timer = Timer(dev)
    print(f"peaks ({kind}): copy {bw / 1e9:.0f} GB/s, bf16 GEMM {fl / 1e12:.0f} TFLOP/s")
    print(f"{'kernel':34s} {'us':>9s} {'TFLOP/s':>9s} {'GB/s':>8s}  fraction of {kind} peak")
    for name, fn, flops, byt in cases:
        us = timer.time_us(fn, iters=args.iters)
        tf = flops / us / 1e6 if flops else 0.0
        gbs = byt / us / 1e3
        frac = max(flops / (us * 1e-6) / fl if flops else 0.0, byt / (us * 1e-6) / bw)
        bound = "compute" if flops and flops / fl > byt / bw else "memory"
        print(f"{name:34s} {us:9.1f} {tf:9.1f} {gbs:8.0f}  {frac:5.2f} ({bound})")
    code, detail = _lib.read_status()
    print("device status", code, hex(detail))


if __name__ == "__main__":
    main()
