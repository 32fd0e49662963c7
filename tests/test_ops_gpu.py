"""Numerics of the single-GPU kernels against fp32 PyTorch references."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, atol, rtol=0.0, what=""):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = (err > tol)
    assert not bad.any(), f"{what}: max err {err.max().item():.4g} (tol {atol}), {int(bad.sum())} bad of {a.numel()}"


@pytest.mark.parametrize("B,nh,S,D", [(2, 2, 128, 64), (1, 3, 256, 64), (2, 2, 512, 128), (1, 2, 384, 128),
                                      (4, 12, 1024, 64), (1, 2, 2048, 64)])
def test_flash_attention_fwd_bwd(cuda_device, B, nh, S, D):
    from gpt_from_scratch_b200.ops.attention import apply_flash_attn, attention_reference
    g = torch.Generator(device="cuda").manual_seed(S + D)
    q, k, v = (torch.randn(B, nh, S, D, device=cuda_device, generator=g).bfloat16().requires_grad_() for _ in range(3))
    do = torch.randn(B, nh, S, D, device=cuda_device, generator=g).bfloat16()
    o = apply_flash_attn(q, k, v, True)
    o.backward(do)
    dq, dk, dv = q.grad.clone(), k.grad.clone(), v.grad.clone()
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    of = attention_reference(qf, kf, vf, True)
    of.backward(do.float())
    # the reference repository's own tolerances: 1e-2 forward, 5e-2 gradients
    _close(o, of, 1e-2, what="O")
    _close(dq, qf.grad, 5e-2, what="dQ")
    _close(dk, kf.grad, 5e-2, what="dK")
    _close(dv, vf.grad, 5e-2, what="dV")
    # and a tighter relative check on the aggregate error
    for name, a, b in (("O", o, of), ("dQ", dq, qf.grad), ("dK", dk, kf.grad), ("dV", dv, vf.grad)):
        rel = (a.float() - b).norm() / (b.norm() + 1e-12)
        assert rel < 2e-2, f"{name}: relative error {rel:.4g}"


def test_flash_attention_fp16_inputs_run_the_native_kernels(cuda_device):
    """fp16 in, fp16 out (the reference's self-test dtype): served by the bf16 kernels, never by the
    eager fallback; compared against the fp32 oracle with the reference's tolerances."""
    from gpt_from_scratch_b200.ops import _lib
    from gpt_from_scratch_b200.ops.attention import apply_flash_attn, attention_reference
    g = torch.Generator(device="cuda").manual_seed(77)
    B, nh, S, D = 2, 3, 256, 64
    q, k, v = (torch.randn(B, nh, S, D, device=cuda_device, generator=g).half().requires_grad_() for _ in range(3))
    do = torch.randn(B, nh, S, D, device=cuda_device, generator=g).half()
    before = _lib.launch_count()
    o = apply_flash_attn(q, k, v, True)
    o.backward(do)
    assert _lib.launch_count() - before >= 2 and o.dtype == torch.float16 and q.grad.dtype == torch.float16
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    of = attention_reference(qf, kf, vf, True)
    of.backward(do.float())
    _close(o, of, 2e-2, what="O")
    for name, a, b in (("O", o, of), ("dQ", q.grad, qf.grad), ("dK", k.grad, kf.grad), ("dV", v.grad, vf.grad)):
        _close(a, b, 5e-2, what=name)
        rel = (a.float() - b).norm() / (b.norm() + 1e-12)
        assert rel < 2e-2, f"{name}: relative error {rel:.4g}"
    with pytest.raises(ValueError):
        apply_flash_attn(q[..., :32], k[..., :32], v[..., :32], True)


@pytest.mark.parametrize("causal,D", [(True, 64), (False, 64), (True, 128)])
def test_flash_attention_growing_scores(cuda_device, causal, D):
    """Keys whose magnitude grows along the sequence: the row maximum rises by far more than 2^8
    from one key block to the next, so the head_dim-64 forward has to rescale the output it
    accumulates in tensor memory (with random-normal inputs the maximum settles in the first
    block and that path never runs). Some rows get a negative query, so their maximum stays."""
    from gpt_from_scratch_b200.ops.attention import apply_flash_attn, attention_reference
    g = torch.Generator(device="cuda").manual_seed(11)
    B, nh, S = 2, 3, 640
    q = torch.randn(B, nh, S, D, device=cuda_device, generator=g)
    k = torch.randn(B, nh, S, D, device=cuda_device, generator=g)
    v = torch.randn(B, nh, S, D, device=cuda_device, generator=g)
    ramp = torch.linspace(0.25, 6.0, S, device=cuda_device).view(1, 1, S, 1)
    k = k * ramp + 0.5 * ramp * torch.sign(q.mean(dim=2, keepdim=True))
    q[:, :, ::3] *= -1.0
    q, k, v = (t.bfloat16().requires_grad_() for t in (q, k, v))
    do = torch.randn(B, nh, S, D, device=cuda_device, generator=g).bfloat16()
    o = apply_flash_attn(q, k, v, causal)
    o.backward(do)
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    of = attention_reference(qf, kf, vf, causal)
    of.backward(do.float())
    _close(o, of, 2e-2, what="O")
    for name, a, b in (("O", o, of), ("dQ", q.grad, qf.grad), ("dK", k.grad, kf.grad), ("dV", v.grad, vf.grad)):
        rel = (a.float() - b).norm() / (b.norm() + 1e-12)
        assert rel < 3e-2, f"{name}: relative error {rel:.4g}"


def test_flash_attention_noncausal_and_ragged(cuda_device):
    from gpt_from_scratch_b200.ops.attention import apply_flash_attn, attention_reference
    g = torch.Generator(device="cuda").manual_seed(3)
    for S, causal in ((192, True), (320, False), (64, True)):
        q, k, v = (torch.randn(1, 2, S, 64, device=cuda_device, generator=g).bfloat16().requires_grad_()
                   for _ in range(3))
        do = torch.randn(1, 2, S, 64, device=cuda_device, generator=g).bfloat16()
        o = apply_flash_attn(q, k, v, causal)
        o.backward(do)
        qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
        of = attention_reference(qf, kf, vf, causal)
        of.backward(do.float())
        _close(o, of, 1e-2, what=f"O S={S}")
        _close(q.grad, qf.grad, 5e-2, what=f"dQ S={S}")
        _close(k.grad, kf.grad, 5e-2, what=f"dK S={S}")
        _close(v.grad, vf.grad, 5e-2, what=f"dV S={S}")


@pytest.mark.parametrize("S,B,nh,D", [(256, 2, 4, 64), (128, 1, 2, 128)])
def test_fused_rope_attention_matches_composition(cuda_device, S, B, nh, D):
    from gpt_from_scratch_b200.ops.attention import attention_reference, fused_rope_attention
    from gpt_from_scratch_b200.ops.rope import rope_reference
    g = torch.Generator(device="cuda").manual_seed(9)
    qkv = torch.randn(S * B, 3 * nh * D, device=cuda_device, generator=g).bfloat16()
    pos = torch.arange(S, device=cuda_device, dtype=torch.float32)
    freqs = 10000.0 ** (-torch.arange(0, D, 2, device=cuda_device, dtype=torch.float32) / D)
    ang = pos[:, None] * freqs[None, :]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    x = qkv.clone().requires_grad_()
    do = torch.randn(S * B, nh * D, device=cuda_device, generator=g).bfloat16()
    out = fused_rope_attention(x * 1, cos, sin, S, B, nh, D)
    out.backward(do)
    xf = qkv.float().requires_grad_()
    q, k, v = xf.view(S, B, 3, nh, D).unbind(2)
    qr, kr = rope_reference(q, cos, sin), rope_reference(k, cos, sin)
    of = attention_reference(qr.permute(1, 2, 0, 3), kr.permute(1, 2, 0, 3), v.permute(1, 2, 0, 3), True)
    of = of.permute(2, 0, 1, 3).reshape(S * B, nh * D)
    of.backward(do.float())
    _close(out, of, 1.5e-2, what="fused out")
    _close(x.grad, xf.grad, 6e-2, what="fused dqkv")
    rel = (x.grad.float() - xf.grad).norm() / xf.grad.norm()
    assert rel < 2e-2, rel


def test_rope_fwd_bwd(cuda_device):
    from gpt_from_scratch_b200.ops.rope import apply_rope, rope_reference
    S, B, nh, D = 96, 3, 5, 64
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(S, B, nh, D, device=cuda_device, generator=g).bfloat16().requires_grad_()
    ang = torch.rand(S, D // 2, device=cuda_device, generator=g) * 6.28
    cos, sin = ang.cos(), ang.sin()
    y = apply_rope(x, cos, sin)
    gy = torch.randn_like(y)
    y.backward(gy)
    xf = x.detach().float().requires_grad_()
    yf = rope_reference(xf, cos, sin)
    yf.backward(gy.float())
    _close(y, yf, 2e-2, what="rope y")
    _close(x.grad, xf.grad, 2e-2, what="rope dx")
    # strided input (an unbind view of a packed buffer) must give the same answer
    packed = torch.randn(S, B, 3, nh, D, device=cuda_device, generator=g).bfloat16()
    q = packed[:, :, 0]
    _close(apply_rope(q, cos, sin), rope_reference(q.float(), cos, sin), 2e-2, what="rope strided")


@pytest.mark.parametrize("rows,H", [(64, 768), (1000, 2048), (33, 4096), (17, 8192), (4096, 768)])
def test_rmsnorm_fwd_bwd(cuda_device, rows, H):
    from gpt_from_scratch_b200.ops.rmsnorm import rmsnorm, rmsnorm_reference
    g = torch.Generator(device="cuda").manual_seed(rows)
    x = (torch.randn(rows, H, device=cuda_device, generator=g) * 2).bfloat16().requires_grad_()
    w = (1 + 0.1 * torch.randn(H, device=cuda_device, generator=g)).bfloat16().requires_grad_()
    dy = torch.randn(rows, H, device=cuda_device, generator=g).bfloat16()
    y = rmsnorm(x, w, 1e-5)
    y.backward(dy)
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yf = rmsnorm_reference(xf, wf, 1e-5)
    yf.backward(dy.float())
    _close(y, yf, 3e-2, 1e-2, what="rmsnorm y")
    _close(x.grad, xf.grad, 3e-2, 2e-2, what="rmsnorm dx")
    rel = (w.grad.float() - wf.grad).norm() / wf.grad.norm()
    assert rel < 1e-2, f"rmsnorm dw rel {rel}"


def test_swiglu_fwd_bwd(cuda_device):
    from gpt_from_scratch_b200.ops.swiglu import swiglu, swiglu_reference
    g = torch.Generator(device="cuda").manual_seed(4)
    gu = torch.randn(300, 2 * 1408, device=cuda_device, generator=g).bfloat16().requires_grad_()
    da = torch.randn(300, 1408, device=cuda_device, generator=g).bfloat16()
    a = swiglu(gu)
    a.backward(da)
    gf = gu.detach().float().requires_grad_()
    af = swiglu_reference(gf)
    af.backward(da.float())
    _close(a, af, 2e-2, 1e-2, what="swiglu")
    _close(gu.grad, gf.grad, 2e-2, 1e-2, what="swiglu grad")


@pytest.mark.parametrize("M,H,I", [(256, 256, 384), (1000, 768, 704), (2048, 768, 3072)])
def test_fused_mlp_matches_unfused(cuda_device, M, H, I):
    """SwiGLU folded into the GEMM epilogues == separate GEMM / activation kernels."""
    from gpt_from_scratch_b200.ops.mlp_fused import _FusedMLP
    g = torch.Generator(device="cuda").manual_seed(M + I)
    x = torch.randn(M, H, device=cuda_device, generator=g).bfloat16()
    w_gu = (torch.randn(2 * I, H, device=cuda_device, generator=g) * 0.05).bfloat16()
    w_dn = (torch.randn(H, I, device=cuda_device, generator=g) * 0.05).bfloat16()
    res = torch.randn(M, H, device=cuda_device, generator=g).bfloat16()
    dout = torch.randn(M, H, device=cuda_device, generator=g).bfloat16()
    xa, wa, wb = x.clone().requires_grad_(), w_gu.clone().requires_grad_(), w_dn.clone().requires_grad_()
    ya = _FusedMLP.apply(xa, wa, wb, res, None, None)
    ya.backward(dout)
    xf, wf, wg = x.float().requires_grad_(), w_gu.float().requires_grad_(), w_dn.float().requires_grad_()
    gu = xf @ wf.t()
    act = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    yf = act @ wg.t() + res.float()
    yf.backward(dout.float())
    for name, a, b in (("y", ya, yf), ("dx", xa.grad, xf.grad), ("dW_gu", wa.grad, wf.grad), ("dW_down", wb.grad, wg.grad)):
        rel = (a.float() - b).norm() / (b.norm() + 1e-9)
        assert rel < 1.5e-2, f"{name}: relative error {rel:.4g}"


@pytest.mark.parametrize("M,H,I", [(512, 256, 384), (1000, 768, 704), (2048, 320, 1536)])
@pytest.mark.parametrize("pair", [False, True])
def test_swiglu_gemm_epilogues(cuda_device, M, H, I, pair):
    """SwiGLU forward / backward folded into the GEMM epilogue (single-CTA and CTA-pair kernels)
    against an fp32 reference of the same two steps."""
    from gpt_from_scratch_b200.ops import gemm as gemm_ops
    from gpt_from_scratch_b200.ops.mlp_fused import swiglu_gemm_bwd, swiglu_gemm_fwd
    g = torch.Generator(device="cuda").manual_seed(M + I + int(pair))
    x = torch.randn(M, H, device=cuda_device, generator=g).bfloat16()
    w_gu = (torch.randn(2 * I, H, device=cuda_device, generator=g) * 0.05).bfloat16()
    w_dn = (torch.randn(H, I, device=cuda_device, generator=g) * 0.05).bfloat16()
    dy = torch.randn(M, H, device=cuda_device, generator=g).bfloat16()
    with gemm_ops.pair_min_tiles(1 if pair else 10 ** 9):
        gu, act = swiglu_gemm_fwd(x, w_gu)
        dgu = swiglu_gemm_bwd(dy, w_dn, gu)
    gu_ref = x.float() @ w_gu.float().t()
    _close(gu, gu_ref, 2e-2, 2e-2, what="gate_up projection")
    guf = gu.float().requires_grad_()          # the kernels compute act and the gradient from the bf16 projection
    act_ref = torch.nn.functional.silu(guf[:, :I]) * guf[:, I:]
    _close(act, act_ref, 2e-2, 2e-2, what="act")
    dact = (dy.float() @ w_dn.float()).bfloat16().float()
    act_ref.backward(dact)
    _close(dgu, guf.grad, 3e-2, 3e-2, what="d_gate_up")


def test_dropout_residual_kernel(cuda_device):
    """Fused residual + dropout: keep rate, scaling, regenerated mask in the backward."""
    from gpt_from_scratch_b200.ops.dropout import dropout_add
    g = torch.Generator(device="cuda").manual_seed(11)
    x = (torch.rand(512, 768, device=cuda_device, generator=g) * 2 + 2).bfloat16().requires_grad_()   # in [2, 4]
    res = (torch.randn(512, 768, device=cuda_device, generator=g) * 0.25).bfloat16().requires_grad_()
    host_gen = torch.Generator().manual_seed(5)
    p = 0.25
    y = dropout_add(x, res, p, True, generator=host_gen)
    kept = (y.float() - res.float()).abs() > 0.5            # x is bounded away from zero
    rate = kept.float().mean().item()
    assert abs(rate - (1 - p)) < 0.01, rate
    expect = res.float() + torch.where(kept, x.float() / (1 - p), torch.zeros_like(x.float())).bfloat16().float()
    assert (y.float() - expect).abs().max() < 0.07
    dy = torch.randn_like(y)
    y.backward(dy)
    assert torch.equal(res.grad, dy)
    dx_expect = torch.where(kept, dy.float() / (1 - p), torch.zeros_like(dy.float()))
    assert (x.grad.float() - dx_expect).abs().max() < 0.05
    assert torch.equal(x.grad != 0, kept & (dy != 0))        # same mask in both directions
    # a different call draws a different mask; evaluation mode is the plain sum
    y2 = dropout_add(x.detach(), res.detach(), p, True, generator=host_gen)
    assert not torch.equal(y2, y.detach())
    assert torch.equal(dropout_add(x.detach(), res.detach(), p, False), res.detach() + x.detach())
