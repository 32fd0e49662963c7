"""Loss / optimizer / end-to-end checks of the native path on one GPU."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_cross_entropy_kernels(cuda_device):
    from gpt_from_scratch_b200.parallel import parallel_state as ps
    from gpt_from_scratch_b200.parallel.loss import vocab_parallel_cross_entropy
    ps.set_device(cuda_device)
    if not ps.model_parallel_is_initialized():
        ps.initialize_parallel_state(1)
    g = torch.Generator(device="cuda").manual_seed(0)
    S, B, V = 48, 3, 1000
    logits = (torch.randn(S, B, V, device=cuda_device, generator=g) * 3).bfloat16()
    target = torch.randint(0, V, (S, B), device=cuda_device, generator=g)
    lf = logits.float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(lf.view(-1, V), target.view(-1), reduction="none").view(S, B)
    w = torch.rand(S, B, device=cuda_device, generator=g)
    (ref * w).sum().backward()
    lg = logits.clone().requires_grad_()
    loss = vocab_parallel_cross_entropy(lg * 1, target)
    (loss * w).sum().backward()
    assert (loss - ref).abs().max().item() < 2e-3
    assert (lg.grad.float() - lf.grad).abs().max().item() < 1e-2
    rel = (lg.grad.float() - lf.grad).norm() / lf.grad.norm()
    assert rel < 1e-2, rel


def test_embedding_kernels(cuda_device):
    from gpt_from_scratch_b200.ops.embedding import embedding_bwd_native, embedding_fwd_native
    g = torch.Generator(device="cuda").manual_seed(1)
    B, S, H, V = 3, 40, 128, 300
    ids = torch.randint(0, V, (B, S), device=cuda_device, generator=g)
    ids[0, :10] = 7  # repeated ids exercise the segmented sum
    W = torch.randn(100, H, device=cuda_device, generator=g).bfloat16()
    v0, v1 = 100, 200
    out = embedding_fwd_native(ids, W, v0, v1)
    mask = (ids >= v0) & (ids < v1)
    ref = torch.nn.functional.embedding((ids - v0).clamp(0, 99), W) * mask.unsqueeze(-1)
    assert torch.equal(out, ref.transpose(0, 1).contiguous())
    dout = torch.randn(S, B, H, device=cuda_device, generator=g).bfloat16()
    dW = torch.zeros_like(W)
    embedding_bwd_native(ids, dout, dW, v0, v1, accumulate=False)
    refd = torch.zeros(100, H, device=cuda_device)
    flat_ids = ids.t().reshape(-1)
    m = (flat_ids >= v0) & (flat_ids < v1)
    refd.index_add_(0, (flat_ids[m] - v0), dout.view(-1, H)[m].float())
    assert (dW.float() - refd).abs().max().item() < 5e-2
    dW2 = torch.zeros_like(W)
    embedding_bwd_native(ids, dout, dW2, v0, v1, accumulate=False)
    assert torch.equal(dW, dW2), "embedding backward must be deterministic"


def test_fused_adamw_matches_torch(cuda_device):
    from gpt_from_scratch_b200.ops import adam as adam_ops
    g = torch.Generator(device="cuda").manual_seed(2)
    n = 100003
    p0 = torch.randn(n, device=cuda_device, generator=g)
    ref_p = p0.clone().requires_grad_()
    opt = torch.optim.AdamW([ref_p], lr=1e-2, weight_decay=0.1, betas=(0.9, 0.95))
    master = p0.clone()
    m = torch.zeros_like(master)
    v = torch.zeros_like(master)
    out = torch.empty(n, dtype=torch.bfloat16, device=cuda_device)
    sumsq = torch.zeros(1, device=cuda_device)
    norm_out = torch.zeros(1, device=cuda_device)
    clip = 1.0
    for step in range(1, 4):
        grad = (torch.randn(n, device=cuda_device, generator=g) * 0.05).bfloat16()
        adam_ops.sumsq_bf16(grad, sumsq)
        ref_ss = grad.float().pow(2).sum()
        assert abs(sumsq.item() - ref_ss.item()) / ref_ss.item() < 1e-5
        adam_ops.adamw_step(grad, master, m, v, out, step=step, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8,
                            weight_decay=0.1, sumsq=sumsq, clip=clip, norm_out=norm_out)
        gf = grad.float()
        norm = gf.norm()
        if norm > clip:
            gf = gf * (clip / (norm + 1e-6))
        ref_p.grad = gf
        opt.step()
        assert abs(norm_out.item() - norm.item()) / norm.item() < 1e-4
        assert (master - ref_p.detach()).abs().max().item() < 2e-6
        assert torch.equal(out, master.bfloat16())


def test_wait_probe_reports_timeout_and_context_survives(cuda_device, request):
    """A device-side wait on a flag nothing sets must give up, record a status and return."""
    from gpt_from_scratch_b200.ops import _lib
    flag = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    rc = _lib.lib().gfs_wait_probe(flag.data_ptr(), 2_000_000, _lib.stream_ptr())  # 2 ms limit
    assert rc == 0
    code, _ = _lib.read_status(clear=True)
    assert code == 9
    # the context is still usable and the status is clear again
    x = torch.ones(16, device=cuda_device)
    assert float(x.sum()) == 16.0
    assert _lib.read_status()[0] == 0
    # and a wait whose flag IS set returns without a status
    flag.fill_(1)
    _lib.lib().gfs_wait_probe(flag.data_ptr(), 2_000_000, _lib.stream_ptr())
    assert _lib.read_status()[0] == 0


def test_training_matches_fp32_oracle(cuda_device):
    """Tiny GPT, 8 steps: the bf16 native path tracks the fp32 unsharded oracle."""
    from oracle import NaiveGPT, naive_step
    from gpt_from_scratch_b200.config import GPTConfig
    from gpt_from_scratch_b200.engine import TrainEngine
    from gpt_from_scratch_b200.ops import _lib
    from gpt_from_scratch_b200.parallel import parallel_state as ps
    ps.set_device(cuda_device)
    if not ps.model_parallel_is_initialized():
        ps.initialize_parallel_state(1)
    cfg = GPTConfig(vocab_size=512, hidden_size=256, num_layers=2, num_attention_heads=4,
                    max_position_embeddings=128, intermediate_size=512, init_method="normal")
    eng = TrainEngine(cfg, lr=1e-3, clip_grad=1.0, seed=5)
    full0 = {k: v.detach().float().cpu() for k, v in eng.model.state_dict().items()}
    oracle = NaiveGPT(cfg)
    oracle.load_state_dict(full0)
    opt = torch.optim.AdamW(oracle.parameters(), lr=1e-3, weight_decay=0.1, betas=(0.9, 0.95))
    before = _lib.launch_count()
    g = torch.Generator().manual_seed(3)
    ours, ref = [], []
    handles = []
    for i in range(8):
        t = torch.randint(0, 512, (4, 129), generator=g)
        x, y = t[:, :-1].contiguous(), t[:, 1:].contiguous()
        if i % 2:   # the asynchronous loss read (pinned buffer + event) must give the same numbers
            handles.append((i, eng.train_step_async(x.cuda(), y.cuda())))
            ours.append(None)
        else:
            ours.append(float(eng.train_step(x.cuda(), y.cuda())))
        ref.append(float(naive_step(oracle, opt, x, y, 1.0)))
    for i, h in handles:
        ours[i] = h.value()
    assert _lib.launch_count() - before > 100, "native kernels were not used"
    for a, b in zip(ours, ref):
        assert abs(a - b) < 3e-2, (ours, ref)
    sd = eng.model.state_dict()
    for k, v in oracle.state_dict().items():
        rel = (sd[k].float().cpu() - v).norm() / (v.norm() + 1e-9)
        assert rel < 2e-2, f"{k}: {rel}"


def test_training_with_bias_matches_fp32_oracle(cuda_device):
    """bias=True: the bias gradients come through plain autograd while the weight gradients go to
    gradient sinks; with the lazy gradient-buffer clearing both must still track the oracle."""
    from oracle import NaiveGPT, naive_step
    from gpt_from_scratch_b200.config import GPTConfig
    from gpt_from_scratch_b200.engine import TrainEngine
    from gpt_from_scratch_b200.parallel import parallel_state as ps
    ps.set_device(cuda_device)
    if not ps.model_parallel_is_initialized():
        ps.initialize_parallel_state(1)
    cfg = GPTConfig(vocab_size=512, hidden_size=256, num_layers=2, num_attention_heads=4,
                    max_position_embeddings=128, intermediate_size=512, init_method="normal", bias=True)
    eng = TrainEngine(cfg, lr=1e-3, clip_grad=1.0, seed=5)
    full0 = {k: v.detach().float().cpu() for k, v in eng.model.state_dict().items()}
    oracle = NaiveGPT(cfg)
    oracle.load_state_dict(full0)
    opt = torch.optim.AdamW(oracle.parameters(), lr=1e-3, weight_decay=0.1, betas=(0.9, 0.95))
    g = torch.Generator().manual_seed(3)
    for i in range(6):
        t = torch.randint(0, 512, (4, 129), generator=g)
        x, y = t[:, :-1].contiguous(), t[:, 1:].contiguous()
        a = float(eng.train_step(x.cuda(), y.cuda()))
        b = float(naive_step(oracle, opt, x, y, 1.0))
        assert abs(a - b) < 3e-2, (i, a, b)
    sd = eng.model.state_dict()
    for k, v in oracle.state_dict().items():
        if k.endswith(".bias"):
            # biases start at zero and Adam moves each element by about lr per step: compare the
            # direction and size of the movement. The key part of the qkv bias is left out: its
            # gradient is zero in exact arithmetic (softmax ignores a constant added to a row of
            # scores), so Adam only amplifies rounding noise there.
            ours = sd[k].float().cpu()
            if k.endswith("qkv_proj.bias"):
                H = cfg.hidden_size
                ours, v = torch.cat([ours[:H], ours[2 * H:]]), torch.cat([v[:H], v[2 * H:]])
            assert v.abs().max().item() > 1e-3, f"{k} did not train in the oracle"
            cos = float((ours * v).sum() / (ours.norm() * v.norm() + 1e-12))
            assert cos > 0.8, f"{k}: cosine {cos}"
            assert 0.7 < float(ours.norm() / v.norm()) < 1.3, f"{k}: norm ratio {float(ours.norm() / v.norm())}"


def test_checkpoint_roundtrip_gpu(cuda_device, tmp_path):
    from gpt_from_scratch_b200.checkpoint import load_checkpoint, save_checkpoint
    from gpt_from_scratch_b200.config import GPTConfig
    from gpt_from_scratch_b200.engine import TrainEngine
    from gpt_from_scratch_b200.parallel import parallel_state as ps
    ps.set_device(cuda_device)
    if not ps.model_parallel_is_initialized():
        ps.initialize_parallel_state(1)
    cfg = GPTConfig(vocab_size=256, hidden_size=128, num_layers=1, num_attention_heads=2,
                    max_position_embeddings=128, intermediate_size=256)
    g = torch.Generator().manual_seed(0)
    data = [torch.randint(0, 256, (2, 129), generator=g) for _ in range(6)]
    step = lambda e, t: float(e.train_step(t[:, :-1].contiguous().cuda(), t[:, 1:].contiguous().cuda()))  # noqa
    a = TrainEngine(cfg, lr=1e-3, seed=9)
    for t in data[:3]:
        step(a, t)
    save_checkpoint(str(tmp_path), 3, a.model, a.optimizer)
    tail_a = [step(a, t) for t in data[3:]]
    b = TrainEngine(cfg, lr=1e-3, seed=10)
    load_checkpoint(str(tmp_path), b.model, b.optimizer)
    tail_b = [step(b, t) for t in data[3:]]
    assert tail_a == tail_b, (tail_a, tail_b)


@pytest.mark.parametrize("M,K,N", [(512, 256, 1000), (1000, 320, 2048), (256, 768, 50304)])
def test_lm_head_epilogue_ce_statistics(cuda_device, M, K, N):
    """Softmax statistics produced by the LM-head GEMM epilogue == those of the separate pass
    over the same bf16 logits, and == an fp32 log-sum-exp of those logits."""
    from gpt_from_scratch_b200.ops import cross_entropy as ce_ops
    from gpt_from_scratch_b200.ops import gemm as gemm_ops
    g = torch.Generator(device="cuda").manual_seed(M + N)
    x = torch.randn(M, K, device=cuda_device, generator=g).bfloat16()
    w = (torch.randn(N, K, device=cuda_device, generator=g) * 0.2).bfloat16()
    tgt = torch.randint(0, N, (M,), device=cuda_device, generator=g)
    with gemm_ops.pair_min_tiles(1):
        logits, partials = gemm_ops.linear_fwd_ce(x, w)
    assert partials is not None
    ref_logits = x.float() @ w.float().t()
    assert (logits.float() - ref_logits).abs().max() <= 2e-2 * ref_logits.abs().max() + 1e-3
    stats_a, lse_a, loss_a = ce_ops.ce_stats_from_partials(partials, logits, tgt, 0, True)
    stats_b, lse_b, loss_b = ce_ops.ce_local_stats(logits, tgt, 0, True)
    lse_ref = torch.logsumexp(logits.float(), dim=-1)
    torch.cuda.synchronize()
    assert (lse_a - lse_ref).abs().max() < 2e-3, (lse_a - lse_ref).abs().max()
    assert (lse_a - lse_b).abs().max() < 2e-3
    assert (loss_a - loss_b).abs().max() < 2e-3
    assert torch.equal(stats_a[:, 2], stats_b[:, 2])      # target logits
    # vocabulary-parallel use: targets outside the local range contribute a zero target logit
    stats_c, _, _ = ce_ops.ce_stats_from_partials(partials, logits, tgt, N, False)
    assert float(stats_c[:, 2].abs().max()) == 0.0


def test_training_with_dropout(cuda_device):
    """dropout_prob > 0 takes the fused residual+dropout kernel in every block; the loss stays
    finite and decreases on a repeated batch."""
    from gpt_from_scratch_b200.config import GPTConfig
    from gpt_from_scratch_b200.engine import TrainEngine
    from gpt_from_scratch_b200.ops import _lib
    from gpt_from_scratch_b200.parallel import parallel_state as ps
    ps.set_device(cuda_device)
    if not ps.model_parallel_is_initialized():
        ps.initialize_parallel_state(1)
    cfg = GPTConfig(vocab_size=512, hidden_size=256, num_layers=2, num_attention_heads=4,
                    max_position_embeddings=128, intermediate_size=512, init_method="normal", dropout_prob=0.1)
    eng = TrainEngine(cfg, lr=2e-3, clip_grad=1.0, seed=6)
    t = torch.randint(0, 512, (4, 129), generator=torch.Generator().manual_seed(1))
    x, y = t[:, :-1].contiguous().cuda(), t[:, 1:].contiguous().cuda()
    losses = [float(eng.train_step(x, y)) for _ in range(12)]
    assert all(l == l and l < 20 for l in losses), losses
    assert losses[-1] < losses[0] - 0.5, losses
    assert _lib.read_status()[0] == 0


def test_gradients_complete_after_backward(cuda_device):
    """Weight gradients parked for a grouped launch are launched by the end of backward():
    every .grad is final before optimizer.step()."""
    from gpt_from_scratch_b200.config import GPTConfig
    from gpt_from_scratch_b200.engine import TrainEngine
    from gpt_from_scratch_b200.ops import gemm as gemm_ops
    from gpt_from_scratch_b200.parallel import parallel_state as ps
    ps.set_device(cuda_device)
    if not ps.model_parallel_is_initialized():
        ps.initialize_parallel_state(1)
    cfg = GPTConfig(vocab_size=512, hidden_size=256, num_layers=2, num_attention_heads=4,
                    max_position_embeddings=128, intermediate_size=512, init_method="normal")
    eng = TrainEngine(cfg, lr=1e-3, seed=8)
    t = torch.randint(0, 512, (4, 129), generator=torch.Generator().manual_seed(2))
    x, y = t[:, :-1].contiguous().cuda(), t[:, 1:].contiguous().cuda()
    eng.optimizer.zero_grad()
    eng.forward_loss(x, y).backward()
    assert not gemm_ops._wgrad_queue.items, "weight gradients still parked after backward()"
    torch.cuda.synchronize()
    for name, p in eng.model.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad.float()).all(), name
        if name.endswith("weight") and p.dim() == 2:
            assert float(p.grad.float().abs().max()) > 0, name


def test_training_is_bitwise_reproducible(cuda_device):
    """Two engines built from the same seed produce identical losses and weights: every kernel
    reduces in a fixed order (no atomics), and a missing fence or barrier-phase bug would
    show up as run-to-run differences."""
    from gpt_from_scratch_b200.config import GPTConfig
    from gpt_from_scratch_b200.engine import TrainEngine
    from gpt_from_scratch_b200.parallel import parallel_state as ps
    ps.set_device(cuda_device)
    if not ps.model_parallel_is_initialized():
        ps.initialize_parallel_state(1)
    cfg = GPTConfig(vocab_size=1024, hidden_size=256, num_layers=2, num_attention_heads=4,
                    max_position_embeddings=256, intermediate_size=768, init_method="normal")
    g = torch.Generator().manual_seed(12)
    batches = [torch.randint(0, 1024, (8, 257), generator=g) for _ in range(4)]
    runs = []
    for _ in range(2):
        eng = TrainEngine(cfg, lr=1e-3, clip_grad=1.0, seed=21)
        losses = [float(eng.train_step(t[:, :-1].contiguous().cuda(), t[:, 1:].contiguous().cuda())) for t in batches]
        runs.append((losses, {k: v.detach().clone() for k, v in eng.model.state_dict().items()}))
    assert runs[0][0] == runs[1][0], (runs[0][0], runs[1][0])
    for k, v in runs[0][1].items():
        assert torch.equal(v, runs[1][1][k]), k


def test_cuda_graph_step_matches_eager(cuda_device):
    """The step captured in a CUDA graph and replayed gives the eager loop's losses and weights
    (same seed, same batches); the optimizer's host-side step count keeps up with the replays."""
    from gpt_from_scratch_b200.config import GPTConfig
    from gpt_from_scratch_b200.engine import TrainEngine
    from gpt_from_scratch_b200.ops import _lib
    from gpt_from_scratch_b200.parallel import parallel_state as ps
    ps.set_device(cuda_device)
    if not ps.model_parallel_is_initialized():
        ps.initialize_parallel_state(1)
    cfg = GPTConfig(vocab_size=1024, hidden_size=256, num_layers=2, num_attention_heads=4,
                    max_position_embeddings=256, intermediate_size=768, init_method="normal")
    g = torch.Generator().manual_seed(12)
    batches = [torch.randint(0, 1024, (8, 257), generator=g) for _ in range(8)]
    runs = []
    for graph in (False, True):
        eng = TrainEngine(cfg, lr=1e-3, clip_grad=1.0, seed=21, cuda_graph=graph, graph_warmup=2)
        before = _lib.launch_count()
        losses = [float(eng.train_step(t[:, :-1].contiguous().cuda(), t[:, 1:].contiguous().cuda())) for t in batches]
        runs.append((losses, {k: v.detach().clone() for k, v in eng.model.state_dict().items()},
                     _lib.launch_count() - before, eng))
    eager, graphed = runs
    assert graphed[3]._graph is not None and graphed[3].launches_per_graph_step > 20
    assert graphed[2] == eager[2], "launch accounting of replays differs from the eager loop"
    assert graphed[3].optimizer._step_count == 8 == eager[3].optimizer._step_count
    for a, b in zip(eager[0], graphed[0]):
        assert abs(a - b) < 2e-3, (eager[0], graphed[0])
    for k, v in eager[1].items():
        rel = (graphed[1][k].float() - v.float()).norm() / (v.float().norm() + 1e-9)
        assert rel < 1e-3, f"{k}: {rel}"
    # an eager step after replays still works (the flag/step bookkeeping is shared)
    eng = graphed[3]
    t = batches[0][:4]
    loss = float(eng.train_step(t[:, :-1].contiguous().cuda(), t[:, 1:].contiguous().cuda()))   # other shape: eager
    assert loss == loss and eng.optimizer._step_count == 9
