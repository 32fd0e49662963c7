"""The allocation-free split-K GEMM entry point (``gfs_gemm_bf16_splitk_static``).

Some users of the library cannot allocate device memory at the point where they need a
GEMM (a serving thread that must not hit the allocator's device-wide synchronisation, a
host with no allocator of its own that only passes in its input and output buffers). For
them the library carries its split-K scratch inside its own image. This test calls that
entry point through its exported C symbol, exactly as such a caller would, and checks it
against the regular entry point on two consecutive calls (the second with different data,
so stale scratch contents from the first call would show up).

Collected last on purpose: the file name sorts after every other test file.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib_handle():
    from gpt_from_scratch_b200.ops import _lib
    handle = ctypes.CDLL(str(_lib.lib_path()))
    fn = handle.gfs_gemm_bf16_splitk_static
    vp, i = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [vp, vp, vp, vp, i, i, i, i, i, i, i, i, i, i, i, vp]
    fn.restype = i
    return fn


def _reference_entry(a, b, out, addend, M, N, K, a_mn, b_mn, splits):
    from gpt_from_scratch_b200.ops.gemm import gemm_bf16
    return gemm_bf16(a, b, a_mn_major=a_mn, b_mn_major=b_mn, out=out, addend=addend, force_split=splits)


def test_static_scratch_gemm_matches_regular_entry_point(cuda_device):
    fn = _lib_handle()
    stream = torch.cuda.current_stream().cuda_stream
    M, N, K, splits = 768, 512, 4096, 4          # wgrad-like: contraction over tokens
    g = torch.Generator(device="cuda").manual_seed(77)
    for call in range(2):                          # two calls in a row share the built-in scratch
        a = torch.randn(K, M, device=cuda_device, generator=g).bfloat16()
        b = torch.randn(K, N, device=cuda_device, generator=g).bfloat16()
        r = torch.randn(M, N, device=cuda_device, generator=g).bfloat16()
        out_static = r.clone()
        rc = fn(a.data_ptr(), b.data_ptr(), out_static.data_ptr(), out_static.data_ptr(), M, N, K,
                a.stride(0), b.stride(0), out_static.stride(0), out_static.stride(0), 1, 1, 1, splits, stream)
        assert rc == 0, f"call {call}: rc={rc}"
        out_regular = r.clone()
        _reference_entry(a, b, out_regular, out_regular, M, N, K, True, True, splits)
        torch.cuda.synchronize()
        ref = a.float().t() @ b.float() + r.float()
        scale = ref.abs().max().item()
        assert (out_static.float() - ref).abs().max().item() <= 1.5e-2 * scale + 1e-3
        assert (out_static.float() - out_regular.float()).abs().max().item() <= 1.5e-2 * scale + 1e-3
        assert torch.equal(out_static, out_regular), f"call {call}: results differ from the regular entry point"


@pytest.mark.parametrize("M,N,K,a_mn,b_mn,splits", [
    (256, 96, 1024, True, True, 4),      # N <= 128: the 128-column tile variants
    (200, 312, 1000, False, False, 2),   # K-major operands, K tail (1000 = 15 * 64 + 40), ragged M and N
    (384, 256, 520, False, True, 3),     # mixed layouts, K tail
    (136, 72, 2048, True, False, 8),     # small ragged output, deep contraction
])
def test_static_scratch_gemm_other_kernel_variants(cuda_device, M, N, K, a_mn, b_mn, splits):
    """Layouts, tile widths and ragged sizes beyond the weight-gradient case above, each against the
    regular entry point with the same split count; and the calls leave the amount of free device
    memory exactly as they found it (nothing is allocated or freed behind the caller's back)."""
    fn = _lib_handle()
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn((K, M) if a_mn else (M, K), device=cuda_device, generator=g).bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device=cuda_device, generator=g).bfloat16()
    out_regular = torch.empty(M, N, device=cuda_device, dtype=torch.bfloat16)
    _reference_entry(a, b, out_regular, None, M, N, K, a_mn, b_mn, splits)
    out_static = torch.empty(M, N, device=cuda_device, dtype=torch.bfloat16)
    fn(a.data_ptr(), b.data_ptr(), out_static.data_ptr(), None, M, N, K, a.stride(0), b.stride(0),
       out_static.stride(0), 0, int(a_mn), int(b_mn), 0, splits, stream)        # first call on the device: set-up
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(2):
        rc = fn(a.data_ptr(), b.data_ptr(), out_static.data_ptr(), None, M, N, K, a.stride(0), b.stride(0),
                out_static.stride(0), 0, int(a_mn), int(b_mn), 0, splits, stream)
        assert rc == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free entry point changed free device memory"
    af = a.float().t() if a_mn else a.float()
    bf = b.float() if b_mn else b.float().t()
    ref = af @ bf
    assert (out_static.float() - ref).abs().max().item() <= 1.5e-2 * ref.abs().max().item() + 1e-3
    assert torch.equal(out_static, out_regular)


def test_static_scratch_gemm_rejects_oversized_problems(cuda_device):
    fn = _lib_handle()
    stream = torch.cuda.current_stream().cuda_stream
    M, N, K = 2048, 2048, 1024                    # 2 splits x 2048 x 2048 x 4 B = 32 MiB > 16 MiB
    a = torch.zeros(M, K, device=cuda_device, dtype=torch.bfloat16)
    b = torch.zeros(N, K, device=cuda_device, dtype=torch.bfloat16)
    c = torch.zeros(M, N, device=cuda_device, dtype=torch.bfloat16)
    rc = fn(a.data_ptr(), b.data_ptr(), c.data_ptr(), None, M, N, K, K, K, N, 0, 0, 0, 0, 2, stream)
    assert rc == -4
    assert fn(a.data_ptr(), b.data_ptr(), c.data_ptr(), None, M, N, K, K, K, N, 0, 0, 0, 0, 1, stream) == -1
