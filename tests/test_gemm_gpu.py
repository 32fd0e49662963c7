"""Numerics of the tcgen05 GEMM against an fp32 PyTorch reference (all operand layouts)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn, addend):
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    y = A @ B
    if addend is not None:
        y = y + addend.float()
    return y


def _check(out, ref, K):
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    # bf16 output rounding (2^-8 relative) plus accumulation-order noise
    assert err <= 1.5e-2 * scale + 1e-3, f"max err {err} vs scale {scale} (K={K})"


SHAPES = [
    (128, 256, 64), (128, 128, 128), (256, 512, 256), (384, 768, 768), (1000, 1384, 328),
    (130, 8, 72), (2048, 2304, 768), (96, 4096, 1024),
]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_layouts(cuda_device, M, N, K, a_mn, b_mn):
    from gpt_from_scratch_b200.ops.gemm import gemm_bf16
    if (a_mn and M % 8) or (b_mn and N % 8) or K % 8:
        pytest.skip("pitch must be a multiple of 8 elements")
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    a = torch.randn((K, M) if a_mn else (M, K), device=cuda_device, generator=g).bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device=cuda_device, generator=g).bfloat16()
    out = gemm_bf16(a, b, a_mn_major=a_mn, b_mn_major=b_mn)
    _check(out, _ref(a, b, a_mn, b_mn, None), K)


@pytest.mark.parametrize("split", [0, 1, 2, 5])
def test_gemm_splitk_and_addend(cuda_device, split):
    from gpt_from_scratch_b200.ops.gemm import gemm_bf16
    M, N, K = 768, 768, 4096
    g = torch.Generator(device="cuda").manual_seed(5)
    a = torch.randn((K, M), device=cuda_device, generator=g).bfloat16()
    b = torch.randn((K, N), device=cuda_device, generator=g).bfloat16()
    r = torch.randn((M, N), device=cuda_device, generator=g).bfloat16()
    out = r.clone()
    gemm_bf16(a, b, a_mn_major=True, b_mn_major=True, out=out, addend=out, force_split=split)
    _check(out, _ref(a, b, True, True, r), K)
    out2 = r.clone()
    gemm_bf16(a, b, a_mn_major=True, b_mn_major=True, out=out2, addend=out2, force_split=split)
    assert torch.equal(out, out2), "split-K must be deterministic"


def test_gemm_strided_views(cuda_device):
    """Operands and output that are column slices of wider buffers (pitch != width)."""
    from gpt_from_scratch_b200.ops.gemm import gemm_bf16
    g = torch.Generator(device="cuda").manual_seed(11)
    big_a = torch.randn((512, 1024), device=cuda_device, generator=g).bfloat16()
    big_b = torch.randn((640, 1024), device=cuda_device, generator=g).bfloat16()
    a = big_a[:, 256:768]
    b = big_b[:, 128:640]
    big_c = torch.zeros((512, 1280), device=cuda_device, dtype=torch.bfloat16)
    out = big_c[:, 640:]
    gemm_bf16(a, b, out=out)
    _check(out, a.float() @ b.float().t(), 512)
    assert big_c[:, :640].abs().max().item() == 0


def test_gemm_rope_epilogue(cuda_device):
    """Rotary embedding applied by the GEMM epilogue to the q and k thirds of a qkv projection."""
    from gpt_from_scratch_b200.ops.gemm import gemm_bf16
    from gpt_from_scratch_b200.ops.rope import rope_reference
    S, B, nh, D, K = 64, 3, 4, 64, 256
    g = torch.Generator(device="cuda").manual_seed(21)
    x = torch.randn(S * B, K, device=cuda_device, generator=g).bfloat16()
    w = (torch.randn(3 * nh * D, K, device=cuda_device, generator=g) * 0.05).bfloat16()
    ang = torch.rand(S, D // 2, device=cuda_device, generator=g) * 6.28
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    out = gemm_bf16(x, w, rope=(cos, sin, 2 * nh * D, D, B))
    ref = (x.float() @ w.float().t()).view(S, B, 3, nh, D)
    q, k, v = ref.unbind(2)
    ref = torch.stack((rope_reference(q, cos, sin), rope_reference(k, cos, sin), v), dim=2).view(S * B, -1)
    _check(out, ref, K)


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 256), (1024, 1280, 328), (2000, 520, 1024),
                                   (4096, 2304, 768)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
def test_gemm_cta_pair_kernel(cuda_device, M, N, K, a_mn, b_mn):
    """The cta_group::2 kernel (one 256x256 tile per CTA pair) against the fp32 reference."""
    from gpt_from_scratch_b200.ops.gemm import gemm_bf16
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn((K, M) if a_mn else (M, K), device=cuda_device, generator=g).bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device=cuda_device, generator=g).bfloat16()
    r = torch.randn((M, N), device=cuda_device, generator=g).bfloat16()
    out = gemm_bf16(a, b, a_mn_major=a_mn, b_mn_major=b_mn, pair=True)
    _check(out, _ref(a, b, a_mn, b_mn, None), K)
    out2 = r.clone()
    gemm_bf16(a, b, a_mn_major=a_mn, b_mn_major=b_mn, out=out2, addend=out2, pair=True)
    _check(out2, _ref(a, b, a_mn, b_mn, r), K)


def test_grouped_weight_gradients(cuda_device):
    """Several weight-gradient problems in one grouped launch (parked, then flushed) against
    the fp32 reference; one of them accumulates into an existing gradient."""
    from gpt_from_scratch_b200.ops import gemm as gemm_ops

    class Sink:  # the two methods of GradSink the GEMM layer uses, on a plain tensor
        def __init__(self, t, accumulate):
            self.t, self.acc, self.finished = t, accumulate, False

        def target(self):
            return self.t

        def consume_accumulate(self):
            return self.acc

        def done(self):
            self.finished = True

    g = torch.Generator(device="cuda").manual_seed(7)
    T = 1536  # tokens (the contraction)
    shapes = [(768, 768), (2304, 768), (768, 3072), (384, 264)]
    flat = torch.randn(sum(o * i for o, i in shapes), device=cuda_device, generator=g).bfloat16()
    before = flat.clone()
    sinks, operands, off = [], [], 0
    for n, (o, i) in enumerate(shapes):
        dy = torch.randn(T, o, device=cuda_device, generator=g).bfloat16()
        x = torch.randn(T, i, device=cuda_device, generator=g).bfloat16()
        sinks.append(Sink(flat[off:off + o * i].view(o, i), accumulate=(n == 1)))
        operands.append((dy, x))
        off += o * i
    with gemm_ops.pair_min_tiles(10 ** 6):   # park everything until the explicit flush
        for n, ((dy, x), sk) in enumerate(zip(operands, sinks)):
            gemm_ops.linear_wgrad_to_sink(dy, x, sk)
            if n == 2:
                assert not any(s_.finished for s_ in sinks)   # parked, nothing launched yet
        gemm_ops.flush_wgrad()   # (the fourth problem filled the group and launched it already)
    torch.cuda.synchronize()
    off = 0
    for n, ((dy, x), sk, (o, i)) in enumerate(zip(operands, sinks, shapes)):
        assert sk.finished
        ref = dy.float().t() @ x.float()
        if n == 1:
            ref = ref + before[off:off + o * i].view(o, i).float()
        _check(sk.t, ref, T)
        off += o * i
