"""Single-process CPU unit tests: group math, flat-buffer layout, resharding, data loading,
CLI, reference formulas of the operators, checkpoint round trip."""
import math
import os
import sys

import numpy as np
import pytest
import torch

from gpt_from_scratch_b200.config import GPTConfig
from gpt_from_scratch_b200.parallel import parallel_state as ps


@pytest.fixture(autouse=True)
def _cpu_state():
    ps.destroy_model_parallel()
    ps.set_device("cpu")
    ps.initialize_parallel_state(1)
    yield
    ps.destroy_model_parallel()


def test_parallel_state_single_process():
    assert ps.get_tensor_model_parallel_world_size() == 1
    assert ps.get_data_parallel_world_size() == 1
    assert ps.get_tensor_model_parallel_group() is None
    with pytest.raises(RuntimeError):
        ps.initialize_parallel_state(2)


def test_flops_and_param_count_of_the_three_model_shapes():
    cfg = GPTConfig()
    assert abs(cfg.flops_per_token(1024) / 1e9 - 0.968) < 1e-3
    assert abs(cfg.num_parameters() / 1e6 - 190.5) < 0.1
    big = GPTConfig(hidden_size=4096, num_layers=32, num_attention_heads=32, intermediate_size=11008)
    assert abs(big.flops_per_token(4096) / 1e9 - 43.3) < 0.1


def test_state_dict_layout_matches_reference_keys():
    from gpt_from_scratch_b200.models.gpt import GPTModel
    cfg = GPTConfig(vocab_size=64, hidden_size=32, num_layers=2, num_attention_heads=4,
                    max_position_embeddings=16, intermediate_size=48)
    sd = GPTModel(cfg).state_dict()
    expect = {"embedding.weight": (64, 32), "final_norm.weight": (32,), "output.weight": (64, 32)}
    for i in range(2):
        expect.update({
            f"layers.{i}.input_norm.weight": (32,),
            f"layers.{i}.attention.qkv_proj.weight": (96, 32),
            f"layers.{i}.attention.out_proj.weight": (32, 32),
            f"layers.{i}.attention.rotary_emb.freqs": (4,),
            f"layers.{i}.post_attention_norm.weight": (32,),
            f"layers.{i}.mlp.gate_up_proj.weight": (96, 32),
            f"layers.{i}.mlp.down_proj.weight": (32, 48),
        })
    assert {k: tuple(v.shape) for k, v in sd.items()} == expect


def test_reshard_roundtrip():
    from gpt_from_scratch_b200.utils.reshard import merge_state_dicts, shard_state_dict
    g = torch.Generator().manual_seed(0)
    H, I, V, nh = 16, 24, 32, 4
    full = {"embedding.weight": torch.randn(V, H, generator=g),
            "layers.0.attention.qkv_proj.weight": torch.randn(3 * H, H, generator=g),
            "layers.0.attention.out_proj.weight": torch.randn(H, H, generator=g),
            "layers.0.mlp.gate_up_proj.weight": torch.randn(2 * I, H, generator=g),
            "layers.0.mlp.down_proj.weight": torch.randn(H, I, generator=g),
            "layers.0.input_norm.weight": torch.randn(H, generator=g),
            "output.weight": torch.randn(V, H, generator=g)}
    for P in (2, 4):
        shards = [shard_state_dict(full, r, P) for r in range(P)]
        # q block of rank 1 = q rows [H/P, 2H/P) of the full tensor
        q1 = shards[1]["layers.0.attention.qkv_proj.weight"][: H // P]
        assert torch.equal(q1, full["layers.0.attention.qkv_proj.weight"][H // P: 2 * H // P])
        up0 = shards[0]["layers.0.mlp.gate_up_proj.weight"][I // P:]
        assert torch.equal(up0, full["layers.0.mlp.gate_up_proj.weight"][I: I + I // P])
        merged = merge_state_dicts(shards)
        for k in full:
            assert torch.equal(merged[k], full[k]), k


def test_optimizer_flat_buffer_layout_and_padding():
    from gpt_from_scratch_b200.models.gpt import GPTModel
    from gpt_from_scratch_b200.optimizer import DistributedOptimizer
    cfg = GPTConfig(vocab_size=64, hidden_size=32, num_layers=1, num_attention_heads=4,
                    max_position_embeddings=16, intermediate_size=48)
    model = GPTModel(cfg)
    names = [n for n, _ in model.named_parameters()]
    assert names == ["embedding.weight", "layers.0.input_norm.weight", "layers.0.attention.qkv_proj.weight",
                     "layers.0.attention.out_proj.weight", "layers.0.post_attention_norm.weight",
                     "layers.0.mlp.gate_up_proj.weight", "layers.0.mlp.down_proj.weight", "final_norm.weight",
                     "output.weight"]
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    opt = DistributedOptimizer(model, torch.optim.AdamW, {"lr": 1e-3}, dtype=torch.float32)
    off = 0
    for (n, p), o in zip(model.named_parameters(), opt.param_offsets):
        assert o == off and p.data_ptr() == opt.param_buffer[off:].data_ptr()
        assert p.grad.data_ptr() == opt.grad_buffer[off:].data_ptr()
        assert torch.equal(p.detach(), before[n])
        off += p.numel()
    assert opt.padded_numel % 8 == 0 and opt.padded_numel >= off
    assert torch.equal(opt.fp32_master_shard.detach(), opt.param_buffer)
    sd = opt.state_dict()
    assert set(sd) == {"state", "param_groups"}


def test_adamw_step_formula_and_clip():
    """One step of the optimizer == the closed-form AdamW update with the reference's clip rule."""
    lin = torch.nn.Linear(8, 8, bias=False)
    from gpt_from_scratch_b200.optimizer import DistributedOptimizer
    w0 = lin.weight.detach().clone()
    opt = DistributedOptimizer(lin, torch.optim.AdamW, {"lr": 0.1, "weight_decay": 0.1, "betas": (0.9, 0.95)},
                               clip_grad=1.0, dtype=torch.float32)
    opt.zero_grad()
    g = torch.full((8, 8), 0.5)
    lin.weight.grad.copy_(g)
    opt.step()
    norm = g.norm()
    gc = g * (1.0 / (norm + 1e-6))
    m = 0.1 * gc
    v = 0.05 * gc * gc
    expect = w0 * (1 - 0.1 * 0.1) - 0.1 * (m / 0.1) / ((v / 0.05).sqrt() + 1e-8)
    assert torch.allclose(lin.weight.detach(), expect, atol=1e-6)
    assert abs(float(opt.last_grad_norm) - float(norm)) < 1e-5


def test_rope_rmsnorm_swiglu_reference_formulas():
    from gpt_from_scratch_b200.ops.rmsnorm import rmsnorm_reference
    from gpt_from_scratch_b200.ops.rope import rope_reference
    from gpt_from_scratch_b200.ops.swiglu import swiglu_reference
    x = torch.arange(8, dtype=torch.float32).view(1, 1, 1, 8)
    ang = torch.tensor([[0.1, 0.2, 0.3, 0.4]])
    y = rope_reference(x, ang.cos(), ang.sin())
    for i in range(4):
        e, o = x[0, 0, 0, 2 * i], x[0, 0, 0, 2 * i + 1]
        assert abs(y[0, 0, 0, 2 * i] - (e * math.cos(ang[0, i]) - o * math.sin(ang[0, i]))) < 1e-5
        assert abs(y[0, 0, 0, 2 * i + 1] - (e * math.sin(ang[0, i]) + o * math.cos(ang[0, i]))) < 1e-5
    # rotation is orthogonal: inverse rotation restores the input
    back = rope_reference(y, ang.cos(), -ang.sin())
    assert torch.allclose(back, x, atol=1e-5)
    h = torch.randn(3, 16)
    w = torch.rand(16) + 0.5
    assert torch.allclose(rmsnorm_reference(h, w, 1e-5), h / (h.pow(2).mean(-1, keepdim=True) + 1e-5).sqrt() * w,
                          atol=1e-6)
    gu = torch.randn(4, 12)
    assert torch.allclose(swiglu_reference(gu), torch.nn.functional.silu(gu[:, :6]) * gu[:, 6:])


def test_vocab_parallel_ce_equals_torch_ce_on_one_rank():
    from gpt_from_scratch_b200.parallel.loss import _VocabParallelCrossEntropy
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(5, 2, 11, generator=g, requires_grad=True)
    tgt = torch.randint(0, 11, (5, 2), generator=g)
    loss = _VocabParallelCrossEntropy.apply(logits, tgt)
    ref = torch.nn.functional.cross_entropy(logits.detach().view(-1, 11), tgt.view(-1), reduction="none").view(5, 2)
    assert torch.allclose(loss, ref, atol=1e-5)
    loss.mean().backward()
    lf = logits.detach().clone().requires_grad_()
    torch.nn.functional.cross_entropy(lf.view(-1, 11), tgt.view(-1)).backward()
    assert torch.allclose(logits.grad, lf.grad, atol=1e-6)


def test_dataset_shift_and_sampler_sharding(tmp_path):
    from gpt_from_scratch_b200.data import DistributedDataset, create_distributed_dataloader, write_synthetic_tokens
    path = str(tmp_path / "tok.bin")
    write_synthetic_tokens(path, 8 * 10 + 1, vocab_size=100, seed=1)
    raw = np.fromfile(path, dtype=np.uint16)
    assert raw.max() < 100
    ds = DistributedDataset(path, 8)
    assert len(ds) == 10
    s = ds[3]
    assert s["input"].dtype == torch.int64
    assert s["input"].tolist() == raw[24:32].tolist() and s["label"].tolist() == raw[25:33].tolist()
    loader, sampler = create_distributed_dataloader(path, 8, 2, num_workers=0)
    sampler.set_epoch(0)
    batches = list(loader)
    assert len(batches) == 5 and batches[0]["input"].shape == (2, 8)
    with pytest.raises(FileNotFoundError):
        DistributedDataset(str(tmp_path / "missing.bin"), 8)


def test_cli_defaults_match_reference():
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import train
    a = train.parse_args([])
    assert (a.vocab_size, a.hidden_size, a.num_layers, a.num_attention_heads) == (50304, 768, 12, 12)
    assert (a.max_position_embeddings, a.intermediate_size, a.seq_len, a.batch_size) == (1024, 3072, 1024, 8)
    assert (a.num_workers, a.lr, a.weight_decay, a.max_steps, a.clip_grad, a.log_interval) == \
        (4, 3e-4, 0.1, 100000, 1.0, 10)
    assert a.tensor_model_parallel_size == 1
    cfg = train.build_config(train.parse_args(["--seq-len", "2048"]))
    assert cfg.max_position_embeddings == 2048      # no crash for seq_len > max positions


def test_rotary_cache_grows():
    from gpt_from_scratch_b200.models.position_embeddings import RotaryEmbedding
    r = RotaryEmbedding(8, max_position_embeddings=4)
    cos, sin = r(torch.zeros(1), 10)
    assert cos.shape == (10, 4)
    assert "freqs" in r.state_dict() and "cos_cached" not in r.state_dict()


def test_checkpoint_resume_is_exact_cpu(tmp_path):
    from gpt_from_scratch_b200.checkpoint import load_checkpoint, save_checkpoint
    from gpt_from_scratch_b200.engine import TrainEngine
    cfg = GPTConfig(vocab_size=64, hidden_size=32, num_layers=1, num_attention_heads=4,
                    max_position_embeddings=16, intermediate_size=48, attention_impl="torch")
    g = torch.Generator().manual_seed(0)
    data = [torch.randint(0, 64, (2, 17), generator=g) for _ in range(6)]
    step = lambda e, t: float(e.train_step(t[:, :-1].contiguous(), t[:, 1:].contiguous()))  # noqa: E731
    a = TrainEngine(cfg, lr=1e-2, dtype=torch.float32, seed=1)
    for t in data[:3]:
        step(a, t)
    save_checkpoint(str(tmp_path), 3, a.model, a.optimizer, {"epoch": 0})
    tail_a = [step(a, t) for t in data[3:]]
    b = TrainEngine(cfg, lr=1e-2, dtype=torch.float32, seed=2)
    payload = load_checkpoint(str(tmp_path), b.model, b.optimizer)
    assert payload["step"] == 3
    tail_b = [step(b, t) for t in data[3:]]
    assert tail_a == tail_b
    # a corrupted shard is detected
    bad = os.path.join(str(tmp_path), "step_00000003", "tp00_dp00.pt")
    with open(bad, "r+b") as f:
        f.seek(100)
        f.write(b"\0" * 64)
    with pytest.raises(Exception):
        load_checkpoint(str(tmp_path), b.model, b.optimizer)


def test_native_library_is_required_on_request(monkeypatch, tmp_path):
    from gpt_from_scratch_b200.ops import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "_LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(_lib.NativeLibraryError):
        _lib.lib()


def test_dropout_add_and_wgrad_queue_cpu_paths():
    """Host-side behaviour of two helpers whose kernels only exist on the GPU: the fused
    residual+dropout falls back to the composition off-GPU, and the weight-gradient queue
    never parks a problem it cannot serve natively."""
    import torch
    from gpt_from_scratch_b200.ops import gemm as gemm_ops
    from gpt_from_scratch_b200.ops.dropout import dropout_add
    x, r = torch.randn(4, 16), torch.randn(4, 16)
    assert torch.equal(dropout_add(x, r, 0.0, True), r + x)
    assert torch.equal(dropout_add(x, r, 0.3, False), r + x)
    torch.manual_seed(0)
    y = dropout_add(x, r, 0.5, True)
    kept = (y - r).abs() > 0
    assert torch.allclose((y - r)[kept], (2.0 * x)[kept])
    assert 0 < kept.float().mean() < 1

    class Sink:
        def __init__(self):
            self.t, self.finished = torch.zeros(8, 16), False

        def target(self):
            return self.t

        def consume_accumulate(self):
            return False

        def done(self):
            self.finished = True

    dy, xx, sk = torch.randn(32, 8), torch.randn(32, 16), Sink()
    gemm_ops.linear_wgrad_to_sink(dy, xx, sk)          # fp32 on CPU: computed at once, not parked
    assert sk.finished and torch.allclose(sk.t, dy.t() @ xx, atol=1e-5)
    gemm_ops.flush_wgrad()                              # nothing parked: a no-op


def test_train_step_async_cpu():
    import torch
    from gpt_from_scratch_b200.config import GPTConfig
    from gpt_from_scratch_b200.engine import TrainEngine
    from gpt_from_scratch_b200.parallel import parallel_state as ps
    ps.set_device(torch.device("cpu"))
    if not ps.model_parallel_is_initialized():
        ps.initialize_parallel_state(1)
    cfg = GPTConfig(vocab_size=64, hidden_size=32, num_layers=1, num_attention_heads=2, max_position_embeddings=16,
                    intermediate_size=64)
    eng = TrainEngine(cfg, lr=1e-3, dtype=torch.float32, seed=1)
    t = torch.randint(0, 64, (2, 17), generator=torch.Generator().manual_seed(0))
    h = eng.train_step_async(t[:, :-1].contiguous(), t[:, 1:].contiguous())
    assert h.ready() and 0 < h.value() < 10


def test_collective_site_keys_follow_program_order():
    """Keys of collectively allocated buffers come from a counter stored on the weight at its
    first use: a freed weight's key is never handed to a new tensor (``id()`` can be), so ranks
    that run the same program derive the same key sequence."""
    import torch
    from gpt_from_scratch_b200.parallel import fused_comm
    a, b = torch.zeros(2, 2), torch.zeros(2, 2)
    ka, kb = fused_comm._weight_site_key(a), fused_comm._weight_site_key(b)
    assert kb == ka + 1
    assert fused_comm._weight_site_key(a) == ka          # stable for the life of the tensor
    seen = {ka, kb}
    for _ in range(50):                                    # freed tensors: their ids get recycled, keys do not
        t = torch.zeros(2, 2)
        k = fused_comm._weight_site_key(t)
        assert k not in seen
        seen.add(k)
        del t
    p = torch.nn.Parameter(torch.zeros(2, 2))
    kp = fused_comm._weight_site_key(p)
    p.data = torch.ones(2, 2)                              # re-pointing the storage keeps the key
    assert fused_comm._weight_site_key(p) == kp


def test_lazy_zero_grad_clears_slices_written_by_plain_autograd():
    """With the kernel path's lazy ``zero_grad`` (no memset) a gradient that arrives through plain
    autograd must not be added onto the previous step's values."""
    from gpt_from_scratch_b200.optimizer import DistributedOptimizer
    lin = torch.nn.Linear(4, 3, bias=True)
    opt = DistributedOptimizer(lin, torch.optim.AdamW, {"lr": 1e-3}, dtype=torch.float32, fused=True)
    x = torch.ones(2, 4)
    for _ in range(3):
        opt.zero_grad()
        lin(x).sum().backward()
        assert torch.equal(lin.bias.grad, torch.full((3,), 2.0))
        assert torch.equal(lin.weight.grad, torch.full((3, 4), 2.0))
        opt._materialise_unwritten()                      # what step() does before it reads the buffer
        assert torch.equal(lin.bias.grad, torch.full((3,), 2.0))
    # a parameter nothing wrote in a step reads as zero
    opt.zero_grad()
    opt._materialise_unwritten()
    assert float(lin.bias.grad.abs().sum()) == 0.0


def test_gradient_buckets_cover_the_flat_buffer_in_aligned_pieces():
    """The bucket cut of the data-parallel gradient reduction: whole buffer covered once, every
    bucket a multiple of 8 x DP size long (so each rank's slice is a whole number of 16-byte
    vectors), boundaries at (rounded) parameter boundaries, and a bucket count that stays small."""
    from gpt_from_scratch_b200.optimizer import DistributedOptimizer

    class Stub:
        NUM_BUCKETS = DistributedOptimizer.NUM_BUCKETS
        _make_buckets = DistributedOptimizer._make_buckets

    for dp, sizes in ((8, [50304 * 768] + [768, 2304 * 768, 768 * 768, 768, 6144 * 768, 768 * 3072] * 12 +
                          [768, 50304 * 768]),
                      (2, [1000, 24, 7, 4096, 333]),
                      (4, [64])):
        st = Stub()
        st.dp_world_size = dp
        st.params = [torch.empty(n) for n in sizes]
        total = sum(sizes)
        align = dp * 8
        st.padded_numel = (total + align - 1) // align * align
        buckets = st._make_buckets()
        assert buckets[0][0] == 0 and buckets[-1][1] == st.padded_numel
        assert all(a1 == b0 for (_, a1), (b0, _) in zip(buckets[:-1], buckets[1:]))
        assert all((b - a) % align == 0 and b > a for a, b in buckets)
        assert len(buckets) <= DistributedOptimizer.NUM_BUCKETS + 1
    # the 124M model at DP8: the LM head, whose gradient the backward pass produces first, is a
    # bucket of its own (it can leave at once)
    st = Stub()
    st.dp_world_size = 8
    sizes = [50304 * 768] + [768, 2304 * 768, 768 * 768, 768, 6144 * 768, 768 * 3072] * 12 + [768, 50304 * 768]
    st.params = [torch.empty(1).expand(n) for n in sizes]
    st.padded_numel = sum(sizes)
    b = st._make_buckets()
    assert b[-1] == (sum(sizes) - 50304 * 768, sum(sizes)), b
    assert b[0] == (0, 50304 * 768), b     # and the embedding table, produced last, another


def test_pending_flag_counts_are_folded_into_the_base_words():
    """Launches made outside a captured step advance the per-site host counts; before the next
    replay they must move into the base words (the captured waits start from those) and restart
    at zero. The bookkeeping is plain host code: exercised here on a group object without any
    symmetric memory behind it."""
    import ctypes
    from gpt_from_scratch_b200.parallel import symm

    grp = symm.SymmGroup.__new__(symm.SymmGroup)        # no CUDA, no rendezvous
    grp.world, grp.rank, grp.device = 2, 0, torch.device("cpu")
    grp._sites, grp._next_slot = {}, 0
    grp._target_store = (ctypes.c_uint * symm.NUM_FLAG_SLOTS)()
    grp._target_view = np.frombuffer(grp._target_store, dtype=np.uint32)
    grp.base = torch.zeros(symm.NUM_FLAG_SLOTS, dtype=torch.int32)
    grp.per_step = torch.zeros(symm.NUM_FLAG_SLOTS, dtype=torch.int32)
    a, b = grp.site("a"), grp.site("b")
    assert (a.slot0, b.slot0) == (0, 2) and grp.site("a") is a
    assert not grp._target_view.any()
    a.target.value += 3                                  # what a launcher does through byref(site.target)
    ctypes.cast(ctypes.byref(b.target), ctypes.POINTER(ctypes.c_uint))[0] += 5
    assert grp._target_view.any() and b.target.value == 5
    saved = dict(symm._groups)
    symm._groups.clear()
    symm._groups["dp"] = grp
    try:
        symm.fold_pending()
        assert grp.base[:4].tolist() == [3, 3, 5, 5] and int(grp.base[4:].abs().sum()) == 0
        assert a.target.value == 0 and b.target.value == 0 and not grp._target_view.any()
        symm.fold_pending()                              # nothing pending: nothing changes
        assert grp.base[:4].tolist() == [3, 3, 5, 5]
        # a capture: counts of the captured step become the per-step increments of the epilogue
        a.target.value += 2
        grp.record_per_step()
        assert grp.per_step[:4].tolist() == [2, 2, 0, 0] and a.target.value == 0
        symm.graph_epilogue()
        assert grp.base[:4].tolist() == [5, 5, 5, 5]
    finally:
        symm._groups.clear()
        symm._groups.update(saved)
