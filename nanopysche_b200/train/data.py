"""Token datasets and loaders (reference: train/data.py:33-158).

``DistributedDataset`` cuts a flat token array into fixed-length ``(input_ids, labels)`` pairs (``Batch``: unpacks as a
pair and indexes by the reference's keys). Labels
are the *same* window as the inputs (the model shifts by one internally); the reference pre-shifts
them in the dataset and the model shifts again. ``DistributedDataLoader`` is an iterator (the
reference's is only iterable although its Trainer calls ``next`` on it), shards over the
data-parallel coordinates rather than the whole world, pins host memory when CUDA is present and
restarts with a new epoch seed when exhausted.
"""
from __future__ import annotations

from collections import namedtuple
from typing import Iterator, Optional

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset, DistributedSampler, RandomSampler


class Batch(namedtuple("Batch", ("input_ids", "labels"))):
    """One sample or batch. A pair - ``input_ids, labels = batch`` - that also reads like the reference's mapping:
    ``batch["input_ids"]``, ``batch.get("labels")``, ``batch.keys()`` (train/data.py:63-71 returns a dict). A named tuple
    keeps its type through ``default_collate`` and the DataLoader's memory pinning."""

    __slots__ = ()

    def __getitem__(self, key):
        if isinstance(key, str):
            try:
                return tuple.__getitem__(self, self._fields.index(key))
            except ValueError:
                raise KeyError(key) from None
        return tuple.__getitem__(self, key)

    def __contains__(self, key):
        return key in self._fields if isinstance(key, str) else any(key is v for v in self)

    def get(self, key, default=None):
        return self[key] if key in self._fields else default

    def keys(self):
        return list(self._fields)

    def values(self):
        return list(self)

    def items(self):
        return list(zip(self._fields, self))


class DistributedDataset(Dataset):
    def __init__(self, tokens=None, seq_len: Optional[int] = None, *, data_source=None, sequence_length: Optional[int] = None):
        """``tokens`` / ``seq_len``, or by the reference's names ``data_source`` / ``sequence_length``
        (train/data.py, default length 2048)."""
        tokens = tokens if tokens is not None else data_source
        seq_len = seq_len if seq_len is not None else (sequence_length if sequence_length is not None else 2048)
        if torch.is_tensor(tokens):
            tokens = tokens.cpu().numpy()
        self.tokens = tokens
        self.seq_len = seq_len
        self.n = max((len(tokens) - 1) // seq_len, 0)

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        s = i * self.seq_len
        window = np.asarray(self.tokens[s:s + self.seq_len]).astype(np.int64)
        ids = torch.from_numpy(window)
        return Batch(ids, ids.clone())


class DistributedDataLoader:
    """Batches of ``(input_ids, labels)`` for this rank's data-parallel index. Which index that is - the position
    among the ranks that read *different* batches (dp x ep of the world mesh; tensor-, context- and pipeline-parallel
    peers read the same batch) - is resolved at the first batch, not at construction: the CLI builds its loaders before
    the mesh exists. Without a mesh every rank is its own data-parallel index (plain DDP)."""

    def __init__(self, dataset: Dataset, batch_size: int, num_workers: int = 0, pin_memory: Optional[bool] = None,
                 drop_last: bool = True, *, seed: int = 0, dp_rank: Optional[int] = None,
                 dp_world: Optional[int] = None, shuffle: bool = True):
        """The first five arguments in the reference's order (train/data.py:87-94). Defaults that differ: no worker
        processes (the reference starts four per loader) and pinning only when CUDA is present."""
        self.dataset, self.batch_size, self.seed = dataset, batch_size, seed
        self.epoch = 0
        self._args = dict(num_workers=num_workers, dp_rank=dp_rank, dp_world=dp_world, shuffle=shuffle,
                          pin_memory=pin_memory, drop_last=drop_last)
        self.sampler = None
        self._loader: Optional[DataLoader] = None
        self._it: Optional[Iterator] = None
        self.batches_served = 0

    @property
    def loader(self) -> DataLoader:
        if self._loader is None:
            a = self._args
            dp_rank, dp_world = a["dp_rank"], a["dp_world"]
            if dp_world is None:
                from ..parallel.mesh import data_parallel_coords, get_world_mesh

                if get_world_mesh() is not None:
                    dp_rank, dp_world = data_parallel_coords()
                elif torch.distributed.is_available() and torch.distributed.is_initialized():
                    dp_rank, dp_world = torch.distributed.get_rank(), torch.distributed.get_world_size()
                else:
                    dp_rank, dp_world = 0, 1
            self.dp_rank, self.dp_world = dp_rank, dp_world
            if dp_world > 1:
                self.sampler = DistributedSampler(self.dataset, num_replicas=dp_world, rank=dp_rank,
                                                  shuffle=a["shuffle"], seed=self.seed)
                self.sampler.set_epoch(self.epoch)
            else:
                gen = torch.Generator().manual_seed(self.seed)
                self.sampler = RandomSampler(self.dataset, generator=gen) if a["shuffle"] else None
            pin = torch.cuda.is_available() if a["pin_memory"] is None else a["pin_memory"]
            self._loader = DataLoader(self.dataset, batch_size=self.batch_size, sampler=self.sampler,
                                      num_workers=a["num_workers"], pin_memory=pin, drop_last=a["drop_last"],
                                      persistent_workers=a["num_workers"] > 0)
        return self._loader

    def set_epoch(self, epoch: int):
        self.epoch = epoch
        if isinstance(self.sampler, DistributedSampler):
            self.sampler.set_epoch(epoch)

    def __len__(self):
        return len(self.loader)

    def __iter__(self):
        self._it = iter(self.loader)
        return self

    def __next__(self):
        if self._it is None:
            self._it = iter(self.loader)
        try:
            b = next(self._it)
        except StopIteration:
            self.set_epoch(self.epoch + 1)
            self._it = iter(self.loader)
            b = next(self._it)
        self.batches_served += 1
        return b

    def state_dict(self):
        return {"epoch": self.epoch, "batches_served": self.batches_served, "seed": self.seed}

    def load_state_dict(self, sd):
        self.set_epoch(sd.get("epoch", 0))
        self.batches_served = sd.get("batches_served", 0)


def create_distributed_loader(data_source, batch_size: int, sequence_length: int = 2048, num_workers: int = 0,
                              **kw) -> DistributedDataLoader:
    return DistributedDataLoader(DistributedDataset(data_source, sequence_length), batch_size,
                                 num_workers=num_workers, **kw)
