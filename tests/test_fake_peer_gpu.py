"""The fused compute+collective kernels on ONE GPU, as rank 0 of a two-rank group whose second
rank is a set of plain buffers (``parallel/fake_peer.py``): what the absent rank would have pushed
is written into this rank's buffers beforehand and its flags are pre-set, so each kernel runs its
real code path (push, signal, wait, reduce) and is checked against an fp32 PyTorch restatement.
The last tests leave the peer's flags unset and give the wait two milliseconds: the kernel must
report the time-out in the status words and return, with the context still usable."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture()
def tp2(cuda_device):
    from gpt_from_scratch_b200.parallel import parallel_state as ps
    from gpt_from_scratch_b200.parallel.fake_peer import fake_peers
    ps.set_device(cuda_device)
    if not ps.model_parallel_is_initialized():
        ps.initialize_parallel_state(1)
    with fake_peers(2, 0) as groups:
        yield groups


def _rel(a, b):
    a, b = a.detach().float(), b.detach().float()
    return float((a - b).norm() / (b.norm() + 1e-9))


@pytest.mark.parametrize("Ms,K,N,pair", [(128, 256, 384, False), (256, 256, 512, True), (512, 320, 1000, True)])
def test_allgather_gemm_and_its_backward(tp2, cuda_device, Ms, K, N, pair):
    from gpt_from_scratch_b200.ops import gemm as gemm_ops
    from gpt_from_scratch_b200.parallel import fused_comm
    grp = tp2["tp"]
    g = torch.Generator(device="cuda").manual_seed(Ms + N)
    M = 2 * Ms
    x0 = torch.randn(Ms, K, device=cuda_device, generator=g).bfloat16().requires_grad_()
    x1 = torch.randn(Ms, K, device=cuda_device, generator=g).bfloat16()
    w = (torch.randn(N, K, device=cuda_device, generator=g) * 0.1).bfloat16().requires_grad_()
    dy = torch.randn(M, N, device=cuda_device, generator=g).bfloat16()
    p1 = torch.randn(Ms, K, device=cuda_device, generator=g).bfloat16()    # rank 1's partial dX for our rows
    # what rank 1 would have delivered: its shard in our gathered buffer, its partial in our staging
    gathered = grp.alloc(("ag", fused_comm._weight_site_key(w)), M * K, torch.bfloat16)
    gathered.tensor.view(M, K)[Ms:] = x1
    stage, _ = grp.pooled("rs", M * K, torch.bfloat16)
    stage.tensor.view(2, Ms, K)[1] = p1
    with gemm_ops.pair_min_tiles(1 if pair else 10 ** 9):
        y = fused_comm.allgather_linear(x0, w)
        y.backward(dy)
    torch.cuda.synchronize()
    xf = torch.cat([x0.detach(), x1]).float()
    ref = xf @ w.detach().float().t()
    assert _rel(y, ref) < 1e-2
    assert (y.float() - ref).abs().max() <= 2e-2 * ref.abs().max() + 1e-2
    # the push reached the fake peer's gathered buffer too (rows of rank 0)
    assert torch.equal(grp.rank_tensors(gathered)[1].view(M, K)[:Ms], x0.detach())
    dx_ref = (dy.float() @ w.detach().float())[:Ms] + p1.float()
    assert _rel(x0.grad, dx_ref) < 1e-2
    dw_ref = dy.float().t() @ xf
    assert _rel(w.grad, dw_ref) < 1e-2
    # and our partial for rank 1's rows went to ITS staging area, slot 0
    sent = grp.rank_tensors(stage)[1].view(2, Ms, K)[0]
    assert _rel(sent, (dy.float() @ w.detach().float())[Ms:]) < 1e-2


@pytest.mark.parametrize("Ms,Kp,N,pair,res", [(128, 192, 256, False, True), (256, 384, 768, True, True),
                                              (256, 256, 520, True, False)])
def test_gemm_reduce_scatter_and_its_backward(tp2, cuda_device, Ms, Kp, N, pair, res):
    from gpt_from_scratch_b200.ops import gemm as gemm_ops
    from gpt_from_scratch_b200.parallel import fused_comm
    grp = tp2["tp"]
    g = torch.Generator(device="cuda").manual_seed(Ms + N + 1)
    M = 2 * Ms
    x = torch.randn(M, Kp, device=cuda_device, generator=g).bfloat16().requires_grad_()
    w = (torch.randn(N, Kp, device=cuda_device, generator=g) * 0.1).bfloat16().requires_grad_()
    r = torch.randn(Ms, N, device=cuda_device, generator=g).bfloat16() if res else None
    part1 = torch.randn(Ms, N, device=cuda_device, generator=g).bfloat16()   # rank 1's partial of our rows
    dout0 = torch.randn(Ms, N, device=cuda_device, generator=g).bfloat16()
    dout1 = torch.randn(Ms, N, device=cuda_device, generator=g).bfloat16()   # rank 1's shard of dOut
    stage, _ = grp.pooled("rs", M * N, torch.bfloat16)
    stage.tensor.view(2, Ms, N)[1] = part1
    agb, _ = grp.pooled("agb", M * N, torch.bfloat16)
    agb.tensor.view(M, N)[Ms:] = dout1
    with gemm_ops.pair_min_tiles(1 if pair else 10 ** 9):
        y = fused_comm.linear_reduce_scatter(x, w, r)
        y.backward(dout0)
    torch.cuda.synchronize()
    full = x.detach().float() @ w.detach().float().t()
    ref = full[:Ms] + part1.float() + (r.float() if res else 0.0)
    assert _rel(y, ref) < 1e-2
    assert _rel(grp.rank_tensors(stage)[1].view(2, Ms, N)[0], full[Ms:]) < 1e-2
    dfull = torch.cat([dout0, dout1]).float()
    assert _rel(x.grad, dfull @ w.detach().float()) < 1e-2
    assert _rel(w.grad, dfull.t() @ x.detach().float()) < 1e-2


def test_swiglu_mlp_under_fused_comm(tp2, cuda_device):
    """gather -> gate|up GEMM with the SwiGLU epilogue -> down GEMM -> reduce-scatter (+ residual), and
    its backward (SwiGLU backward in the epilogue of the all-gather-fed dgrad), against fp32."""
    from gpt_from_scratch_b200.ops import gemm as gemm_ops
    from gpt_from_scratch_b200.parallel import fused_comm
    grp = tp2["tp"]
    g = torch.Generator(device="cuda").manual_seed(21)
    Ms, H, I = 256, 256, 384                   # I = this rank's share of the intermediate size
    M = 2 * Ms
    x0 = torch.randn(Ms, H, device=cuda_device, generator=g).bfloat16().requires_grad_()
    x1 = torch.randn(Ms, H, device=cuda_device, generator=g).bfloat16()
    w_gu = (torch.randn(2 * I, H, device=cuda_device, generator=g) * 0.08).bfloat16().requires_grad_()
    w_dn = (torch.randn(H, I, device=cuda_device, generator=g) * 0.08).bfloat16().requires_grad_()
    res = torch.randn(Ms, H, device=cuda_device, generator=g).bfloat16()
    part1 = torch.randn(Ms, H, device=cuda_device, generator=g).bfloat16()    # rank 1's partial of our output rows
    dout0 = torch.randn(Ms, H, device=cuda_device, generator=g).bfloat16()
    dout1 = torch.randn(Ms, H, device=cuda_device, generator=g).bfloat16()
    gathered = grp.alloc(("ag", fused_comm._weight_site_key(w_gu)), M * H, torch.bfloat16)
    gathered.tensor.view(M, H)[Ms:] = x1
    stage, _ = grp.pooled("rs", M * H, torch.bfloat16)
    agb, _ = grp.pooled("agb", M * H, torch.bfloat16)
    agb.tensor.view(M, H)[Ms:] = dout1
    with gemm_ops.pair_min_tiles(1):
        assert fused_comm.fused_mlp_eligible(x0, w_gu, w_dn)
        stage.tensor.view(2, Ms, H)[1] = part1
        y = fused_comm.swiglu_mlp(x0, w_gu, w_dn, res)
        torch.cuda.synchronize()
        stage.tensor.view(2, Ms, H)[1] = 0          # the backward's reduce-scatter reuses the staging buffer
        y.backward(dout0)
    torch.cuda.synchronize()
    xf = torch.cat([x0.detach(), x1]).float().requires_grad_()
    wg, wd = w_gu.detach().float().requires_grad_(), w_dn.detach().float().requires_grad_()
    gu = (xf @ wg.t())
    act = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    full = act @ wd.t()
    assert _rel(y, full[:Ms] + part1.float() + res.float()) < 1.5e-2
    full.backward(torch.cat([dout0, dout1]).float())
    assert _rel(x0.grad, xf.grad[:Ms]) < 2e-2
    assert _rel(w_gu.grad, wg.grad) < 2e-2
    assert _rel(w_dn.grad, wd.grad) < 2e-2


def test_lm_head_statistics_and_cross_entropy_exchange(tp2, cuda_device):
    """All-gather GEMM with the softmax statistics in its epilogue, then the exchange of (max,
    sum-exp, target logit) with the other vocabulary shard and the combine."""
    from gpt_from_scratch_b200.ops import gemm as gemm_ops
    from gpt_from_scratch_b200.ops import cross_entropy as ce_ops
    from gpt_from_scratch_b200.parallel import fused_comm
    grp = tp2["tp"]
    g = torch.Generator(device="cuda").manual_seed(5)
    Ms, K, Vp = 256, 256, 392
    M = 2 * Ms
    x0 = torch.randn(Ms, K, device=cuda_device, generator=g).bfloat16()
    x1 = torch.randn(Ms, K, device=cuda_device, generator=g).bfloat16()
    w0 = (torch.randn(Vp, K, device=cuda_device, generator=g) * 0.3).bfloat16()
    w1 = (torch.randn(Vp, K, device=cuda_device, generator=g) * 0.3).bfloat16()    # rank 1's vocabulary shard
    tgt = torch.randint(0, 2 * Vp, (M,), device=cuda_device, generator=g)
    gathered = grp.alloc(("ag", fused_comm._weight_site_key(w0)), M * K, torch.bfloat16)
    gathered.tensor.view(M, K)[Ms:] = x1
    with gemm_ops.pair_min_tiles(1):
        logits, partials = fused_comm.allgather_linear(x0, w0, ce_stats=True)
    assert partials is not None
    stats, _, _ = ce_ops.ce_stats_from_partials(partials, logits.view(M, Vp), tgt, 0, False)
    # rank 1's statistics, computed here in fp32 from its (bf16-rounded) logits
    xf = torch.cat([x0, x1]).float()
    l1 = (xf @ w1.float().t()).bfloat16().float()
    in1 = (tgt >= Vp)
    s1 = torch.stack([l1.max(-1)[0], (l1 - l1.max(-1, keepdim=True)[0]).exp().sum(-1),
                      torch.where(in1, l1.gather(1, (tgt - Vp).clamp(0, Vp - 1)[:, None])[:, 0],
                                  torch.zeros(M, device=cuda_device))], dim=-1)
    buf = grp.alloc(("ce", M), 2 * M * 3, torch.float32)
    buf.tensor.view(2, M, 3)[1] = s1
    lse, loss = fused_comm.ce_exchange_combine(stats)
    torch.cuda.synchronize()
    l0 = logits.view(M, Vp).float()
    both = torch.cat([l0, l1], dim=1)
    lse_ref = torch.logsumexp(both, dim=-1)
    loss_ref = lse_ref - both.gather(1, tgt[:, None])[:, 0]
    assert (lse - lse_ref).abs().max() < 2e-3
    assert (loss - loss_ref).abs().max() < 2e-3
    assert torch.equal(grp.rank_tensors(buf)[1].view(2, M, 3)[0], stats)     # our statistics reached rank 1


def test_embedding_scatter(tp2, cuda_device):
    from gpt_from_scratch_b200.parallel import fused_comm
    grp = tp2["tp"]
    g = torch.Generator(device="cuda").manual_seed(6)
    B, S, H, Vp = 3, 256, 128, 200
    ids = torch.randint(0, 2 * Vp, (B, S), device=cuda_device, generator=g)

    class Emb:
        weight = torch.randn(Vp, H, device=cuda_device, generator=g).bfloat16()
        vocab_start_index, vocab_end_index = 0, Vp
    out = fused_comm.embedding_reduce_scatter(ids, Emb)            # [S/2, B, H]: our sequence shard
    torch.cuda.synchronize()
    Ss = S // 2
    mine = ids < Vp
    ref = torch.nn.functional.embedding(ids.clamp(0, Vp - 1), Emb.weight) * mine[..., None]   # [B, S, H]
    ref = ref.transpose(0, 1)                                                                    # [S, B, H]
    assert torch.equal(out, ref[:Ss].contiguous())
    pool, _ = grp.pooled("emb", Ss * B * H, torch.bfloat16)
    assert torch.equal(grp.rank_tensors(pool)[1].view(Ss, B, H), ref[Ss:].contiguous())


def test_data_parallel_optimizer_kernels(cuda_device):
    """Per-bucket gradient push, sum of the staged contributions + norm, then clip + AdamW +
    parameter all-gather by peer stores, as DP rank 0 of 2 with two buckets (so the shard is the
    concatenation of one slice per bucket), against torch.optim.AdamW on the summed gradient."""
    from gpt_from_scratch_b200.parallel import fused_comm
    from gpt_from_scratch_b200.parallel import parallel_state as ps
    from gpt_from_scratch_b200.parallel.fake_peer import fake_peers
    ps.set_device(cuda_device)
    if not ps.model_parallel_is_initialized():
        ps.initialize_parallel_state(1)
    with fake_peers(2, 0) as groups:
        grp = groups["dp"]
        g = torch.Generator(device="cuda").manual_seed(7)
        n, shard = 40960, 20480
        cut, s0, s1 = 16384, 8192, 12288                 # bucket 0 = [0, cut), slices of s0; bucket 1: slices of s1
        dpc = fused_comm.DataParallelComm(n, shard, cuda_device, buckets=[(0, cut), (cut, n)])
        own = lambda t, r: torch.cat([t[r * s0:(r + 1) * s0], t[cut + r * s1:cut + (r + 1) * s1]])  # noqa: E731
        g0 = (torch.randn(n, device=cuda_device, generator=g) * 0.05).bfloat16()
        g1 = (torch.randn(n, device=cuda_device, generator=g) * 0.05).bfloat16()
        dpc.grad_buffer.copy_(g0)
        grp.rank_tensors(dpc._stage)[0].view(2, shard)[1] = own(g1, 0)       # what rank 1 pushed to us
        p0 = torch.randn(shard, device=cuda_device, generator=g)
        master, m, v = p0.clone(), torch.zeros_like(p0), torch.zeros_like(p0)
        other_sumsq = 3.25                                   # what rank 1 would publish for its shard
        grp.rank_tensors(dpc._norm)[0][1] = other_sumsq
        dpc.push_bucket(1)
        dpc.push_bucket(0)
        dpc.sum_and_norm()
        dpc.adam_and_gather(master, m, v, step=1, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                            clip=1.0, grad_scale=1.0)
        torch.cuda.synchronize()
        # our slices of rank 1's buckets went to ITS staging buffer, source slot 0
        assert torch.equal(grp.rank_tensors(dpc._stage)[1].view(2, shard)[0], own(g0, 1))
        red = (own(g0, 0).float() + own(g1, 0).float()).bfloat16()
        assert torch.equal(dpc.reduced, red)
        norm = (red.float().pow(2).sum() + other_sumsq).sqrt()
        assert abs(float(dpc.norm_out) - float(norm)) / float(norm) < 1e-4
        ref = p0.clone().requires_grad_()
        opt = torch.optim.AdamW([ref], lr=1e-2, weight_decay=0.1, betas=(0.9, 0.95))
        ref.grad = red.float() * (1.0 / (float(norm) + 1e-6) if norm > 1.0 else 1.0)
        opt.step()
        assert (master - ref.detach()).abs().max() < 2e-6
        # all-gather by peer stores: our shard landed, slice by slice, in both parameter buffers
        for buf in (dpc.param_buffer, grp.rank_tensors(dpc._param)[1]):
            assert torch.equal(own(buf, 0), master.bfloat16())
            assert float(own(buf, 1).abs().sum()) == 0.0      # rank 1's slices untouched


@pytest.mark.expects_status
def test_absent_peer_times_out_with_a_status(cuda_device, monkeypatch):
    """Nothing ever advances the absent rank's flag: barrier and all-gather give up after 2 ms,
    record status 6 with the waiting rank / source / slot in the detail word, and return."""
    from gpt_from_scratch_b200.ops import _lib
    from gpt_from_scratch_b200.parallel import fused_comm
    from gpt_from_scratch_b200.parallel import parallel_state as ps
    from gpt_from_scratch_b200.parallel.fake_peer import fake_peers
    ps.set_device(cuda_device)
    if not ps.model_parallel_is_initialized():
        ps.initialize_parallel_state(1)
    _lib.read_status(clear=True)
    monkeypatch.setattr(fused_comm, "WAIT_NS", 2_000_000)
    with fake_peers(2, 0, peers_ready=False) as groups:
        fused_comm.barrier("tp")
        code, detail = _lib.read_status(clear=True)
        assert code == 6, (code, hex(detail))
        slot0 = groups["tp"].site("barrier").slot0
        assert detail == (0xC0000000 | (slot0 << 8) | (1 << 4) | 0), hex(detail)   # source 1, waiting rank 0
        x = torch.arange(64 * 16, device=cuda_device, dtype=torch.float32).bfloat16().view(64, 16)
        out = fused_comm.allgather_rows(x, "probe")
        code, detail = _lib.read_status(clear=True)
        assert code == 6
        assert torch.equal(out[:64], x)                       # the kernel still did its own part
    # the context survived and the status words are clear again
    assert float(torch.ones(8, device=cuda_device).sum()) == 8.0
    assert _lib.read_status()[0] == 0
    # the same calls with the peer's flags set complete without a status
    with fake_peers(2, 0, peers_ready=True):
        fused_comm.barrier("tp")
        fused_comm.allgather_rows(x, "probe")
        assert _lib.read_status()[0] == 0
