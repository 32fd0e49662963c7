"""Token-file data loading.

File format and sampling follow the reference (core/data.py:8-70): a flat ``uint16`` token
file read through ``np.memmap``; sample ``i`` is tokens ``[i*S, i*S+S+1)`` split into
``input = chunk[:-1]`` and ``label = chunk[1:]``; ``num_samples = (len-1)//S``; samples
are sharded over the data-parallel group by a ``DistributedSampler`` (shuffle, drop_last)
so tensor-parallel peers read identical batches.

Additions: :class:`PrefetchLoader` moves batches to the GPU from pinned memory with
non-blocking copies one step ahead (the reference does blocking ``.cuda()`` copies of
int64 tensors, train.py:168-169), and :func:`write_synthetic_tokens` produces the seeded
uniform-random token files used by the benchmarks.
"""
from __future__ import annotations

import os

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset
from torch.utils.data.distributed import DistributedSampler

from .parallel import parallel_state as ps


class DistributedDataset(Dataset):
    def __init__(self, data_path: str, seq_len: int):
        if not os.path.exists(data_path):
            raise FileNotFoundError(data_path)
        self.data_path = data_path
        self.seq_len = seq_len
        self.data = np.memmap(data_path, dtype=np.uint16, mode="r")
        self.total_tokens = len(self.data)
        self.num_samples = (self.total_tokens - 1) // seq_len
        if self.num_samples <= 0:
            raise ValueError(f"{data_path}: {self.total_tokens} tokens is less than one sample of {seq_len}+1")

    def __len__(self):
        return self.num_samples

    def __getitem__(self, idx):
        start = idx * self.seq_len
        chunk = torch.from_numpy(self.data[start:start + self.seq_len + 1].astype(np.int64))
        return {"input": chunk[:-1], "label": chunk[1:]}


class ResumableDistributedSampler(DistributedSampler):
    """``DistributedSampler`` that can start an epoch part-way: ``skip_samples(n)`` drops the
    first ``n`` indices of the NEXT iteration only, so a run resumed in the middle of an epoch
    continues with the batch the interrupted run would have read next."""

    _skip = 0

    def skip_samples(self, n: int) -> None:
        self._skip = int(n)

    def __iter__(self):
        it = super().__iter__()
        skip, self._skip = self._skip, 0
        for _ in range(skip):
            next(it, None)
        return it


def create_distributed_dataloader(data_path: str, seq_len: int, batch_size: int, num_workers: int = 4,
                                  seed: int = 0, pin_memory: bool | None = None):
    """Returns ``(dataloader, sampler)``; call ``sampler.set_epoch(epoch)`` every epoch (and
    ``sampler.skip_samples(batches_done * batch_size)`` before iterating to resume inside one)."""
    dataset = DistributedDataset(data_path, seq_len)
    sampler = ResumableDistributedSampler(dataset, num_replicas=ps.get_data_parallel_world_size(),
                                 rank=ps.get_data_parallel_group_rank(), shuffle=True, drop_last=True, seed=seed)
    if pin_memory is None:
        pin_memory = torch.cuda.is_available()
    loader = DataLoader(dataset, batch_size=batch_size, sampler=sampler, num_workers=num_workers,
                        pin_memory=pin_memory, drop_last=True, persistent_workers=num_workers > 0)
    return loader, sampler


class PrefetchLoader:
    """Wraps a loader of ``{'input','label'}`` CPU batches; yields device tensors whose
    host-to-device copies were issued on a side stream while the previous step computed."""

    def __init__(self, loader, device: torch.device):
        self.loader = loader
        self.device = device
        self.stream = torch.cuda.Stream(device) if device.type == "cuda" else None

    def __len__(self):
        return len(self.loader)

    def _to_device(self, batch):
        if self.stream is None:
            return {k: v.to(self.device) for k, v in batch.items()}
        with torch.cuda.stream(self.stream):
            out = {k: (v if v.is_pinned() else v.pin_memory()).to(self.device, non_blocking=True)
                   for k, v in batch.items()}
        return out

    def __iter__(self):
        it = iter(self.loader)
        try:
            nxt = self._to_device(next(it))
        except StopIteration:
            return
        while nxt is not None:
            if self.stream is not None:
                torch.cuda.current_stream(self.device).wait_stream(self.stream)
                for v in nxt.values():
                    v.record_stream(torch.cuda.current_stream(self.device))
            cur = nxt
            try:
                nxt = self._to_device(next(it))
            except StopIteration:
                nxt = None
            yield cur


def write_synthetic_tokens(path: str, num_tokens: int, vocab_size: int = 50257, seed: int = 1234) -> str:
    """Seeded uniform-random ``uint16`` token ids in ``[0, vocab_size)`` written with ``tofile``
    (the format tools/preprocess_data.py produces)."""
    assert vocab_size <= 65536
    rng = np.random.default_rng(seed)
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    rng.integers(0, vocab_size, size=num_tokens, dtype=np.uint16).tofile(path)
    return path
