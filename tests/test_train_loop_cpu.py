"""The training script itself on CPU/gloo ranks: a run resumed in the middle of an epoch repeats
the uninterrupted run's losses (checkpoint carries the position inside the epoch), and a rank that
leaves between steps is reported by the heartbeat before the next collective is launched."""
import json
import os
import sys

import pytest
import torch

from dist_utils import run_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

MODEL = ["--vocab-size", "128", "--hidden-size", "32", "--num-layers", "1", "--num-attention-heads", "4",
         "--intermediate-size", "48", "--seq-len", "16", "--max-position-embeddings", "16", "--batch-size", "2",
         "--num-workers", "0", "--device", "cpu", "--backend", "gloo", "--attention-impl", "torch",
         "--log-interval", "1", "--lr", "1e-2", "--seed", "7"]


def _losses(path):
    return [json.loads(l)["loss"] for l in open(path)]


def _train_worker(rank, world, workdir, tag, extra):
    sys.path.insert(0, ROOT)
    import train
    log = os.path.join(workdir, f"{tag}.jsonl")
    train.main(MODEL + ["--data-path", os.path.join(workdir, "tokens.bin"), "--log-jsonl", log] + extra)
    return _losses(log) if rank == 0 else None


def test_resume_inside_an_epoch_replays_no_data(tmp_path):
    from gpt_from_scratch_b200.data import write_synthetic_tokens
    wd = str(tmp_path)
    # 16 samples of 16 tokens, 2 DP ranks x batch 2 -> 4 batches per epoch
    write_synthetic_tokens(os.path.join(wd, "tokens.bin"), 16 * 16 + 1, 128, seed=3)
    ck = os.path.join(wd, "ck")
    run = lambda tag, extra: run_ranks(_train_worker, 2, args=(wd, tag, extra), tmp_path=tmp_path, init=False)[0]  # noqa
    full = run("full", ["--max-steps", "7"])
    run("head", ["--max-steps", "2", "--save-dir", ck, "--save-interval", "2"])
    tail = run("tail", ["--max-steps", "7", "--load", ck])
    assert len(full) == 7 and len(tail) == 5
    # steps 3..7 of the uninterrupted run: the rest of epoch 0 (2 batches) and 3 batches of epoch 1
    assert tail == full[2:], (full, tail)


class _Leave(Exception):
    pass


def _heartbeat_worker(rank, world, workdir):
    sys.path.insert(0, ROOT)
    import train
    import torch.distributed as dist
    from gpt_from_scratch_b200.engine import TrainEngine
    from gpt_from_scratch_b200.utils.health import PeerFailure
    if rank == 1:
        real = TrainEngine.train_step
        calls = {"n": 0}

        def leaving_step(self, x, y):
            out = real(self, x, y)
            calls["n"] += 1
            if calls["n"] == 3:      # the third step completes (no collective in flight), then the rank
                raise _Leave()       # is gone before it reports it
            return out
        TrainEngine.train_step = leaving_step
    argv = MODEL + ["--synthetic-data", "--data-path", os.path.join(workdir, f"tok.bin"), "--max-steps", "50",
                    "--heartbeat-timeout", "1.5"]
    outcome = "finished"
    try:
        train.main(argv)
    except _Leave:
        outcome = "left"
    except PeerFailure as e:
        outcome = ("peer failure", e.rank, e.last_step)
    if dist.is_initialized():
        # no collective here: the other rank is gone
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass
    return outcome


def test_rank_leaving_between_steps_raises_peer_failure(tmp_path):
    res = run_ranks(_heartbeat_worker, 2, args=(str(tmp_path),), tmp_path=tmp_path, init=False)
    assert res[1] == "left"
    assert res[0] == ("peer failure", 1, 2), res
