"""Optional bridge to ``torch.utils.data.DataLoader``: wraps a windowed token dataset as an iterable dataset whose
workers (spawn start method only — forking a process that owns a CUDA context is unsafe) each take a strided share
of the batch sequence, and yields ``LMTokenBatch`` objects in pinned memory.
Parity: ``cppmega_mlx/data/dataloader_bridge.py:72``."""
from __future__ import annotations

from typing import Iterator

import torch
from torch.utils.data import DataLoader, IterableDataset, get_worker_info

from .batch import LMTokenBatch


class _BatchStream(IterableDataset):
    def __init__(self, dataset, *, epoch: int = 0, resume_batch: int = 0, loop: bool = False):
        self.dataset, self.epoch, self.resume_batch, self.loop = dataset, epoch, resume_batch, loop

    def __iter__(self) -> Iterator[dict]:
        info = get_worker_info()
        wid, nw = (info.id, info.num_workers) if info is not None else (0, 1)
        self.dataset.pin_memory = False  # pinning happens in the parent process
        for i, b in enumerate(self.dataset.iter_batches(resume_batch=self.resume_batch, epoch=self.epoch, loop=self.loop)):
            if i % nw == wid:
                yield b.as_dict()


def make_dataloader(dataset, *, num_workers: int = 0, epoch: int = 0, resume_batch: int = 0, loop: bool = False,
                    prefetch_factor: int | None = None, pin_memory: bool | None = None) -> DataLoader:
    if num_workers < 0:
        raise ValueError("num_workers must be non-negative")
    pin = torch.cuda.is_available() if pin_memory is None else pin_memory
    kw = {}
    if num_workers > 0:
        kw.update(multiprocessing_context="spawn", persistent_workers=False)
        if prefetch_factor is not None:
            kw["prefetch_factor"] = prefetch_factor
    return DataLoader(_BatchStream(dataset, epoch=epoch, resume_batch=resume_batch, loop=loop), batch_size=None,
                      num_workers=num_workers, pin_memory=pin, collate_fn=None, **kw)


def iterate_lm_batches(loader: DataLoader) -> Iterator[LMTokenBatch]:
    for d in loader:
        yield LMTokenBatch(**d)
