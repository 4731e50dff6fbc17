"""Data loading for the trainers: a stateful loader over in-memory datasets and the factory the entry scripts use.

``StatefulListLoader`` shards a list-like dataset over the data-parallel ranks, shuffles per epoch with a seed
that every rank shares, and can be checkpointed in the middle of an epoch: its state is the epoch and the number
of batches already handed out, and a restored loader continues with the next batch of the same permutation (the
role of torchdata's ``StatefulDataLoader`` + ``DistributedSampler`` in areal/utils/dataloader.py).

Training loaders (``drop_last=True``) give every rank the same number of batches, dropping the tail that does
not divide. Evaluation loaders (``drop_last=False``) hand out every sample exactly once: ranks may differ by one
sample and nothing is padded or repeated, so metrics are not biased by duplicates (``EvalDistributedSampler`` in
the reference).
"""

from __future__ import annotations

from typing import Any, Callable, Sequence

import torch


class StatefulListLoader:
    auto_epoch = True  # a full pass moves on to the next epoch by itself (``cycle_dataloader`` relies on it)

    def __init__(self, dataset: Sequence[Any], batch_size: int, shuffle: bool = True, seed: int = 0, rank: int = 0,
                 world: int = 1, drop_last: bool = True, collate_fn: Callable[[list], Any] | None = None):
        if batch_size < 1:
            raise ValueError("batch_size must be positive")
        self.dataset, self.batch_size, self.shuffle = dataset, int(batch_size), shuffle
        self.seed, self.rank, self.world, self.drop_last = seed, rank, world, drop_last
        self.collate_fn = collate_fn
        self.epoch = 0
        self.position = 0  # batches of the current epoch already handed out
        self.sampler = self  # ``loader.sampler.set_epoch`` of the torch idiom lands here

    # ------------------------------------------------------------------ order
    def indices(self, epoch: int | None = None) -> list[int]:
        """This rank's sample indices for ``epoch`` (default: the current one)."""
        n = len(self.dataset)
        idx = list(range(n))
        if self.shuffle:
            g = torch.Generator().manual_seed(self.seed + (self.epoch if epoch is None else epoch))
            idx = torch.randperm(n, generator=g).tolist()
        if self.drop_last:
            idx = idx[: n - n % self.world]  # every rank gets the same count
        return idx[self.rank::self.world]

    def __len__(self) -> int:
        n = len(self.indices(0)) if not self.drop_last else len(self.dataset) // self.world
        return n // self.batch_size if self.drop_last else -(-n // self.batch_size)

    def set_epoch(self, epoch: int) -> None:
        if epoch != self.epoch:
            self.epoch, self.position = int(epoch), 0

    def __iter__(self):
        idx = self.indices()
        stop = len(idx) - (self.batch_size - 1 if self.drop_last else 0)
        starts = list(range(0, max(stop, 0), self.batch_size))
        for k in range(self.position, len(starts)):
            self.position = k + 1
            items = [self.dataset[j] for j in idx[starts[k]:starts[k] + self.batch_size]]
            yield self.collate_fn(items) if self.collate_fn is not None else items
        self.epoch += 1
        self.position = 0

    # ------------------------------------------------------------------ state
    def state_dict(self) -> dict[str, int]:
        return {"epoch": self.epoch, "position": self.position}

    def load_state_dict(self, state: dict[str, int]) -> None:
        self.epoch = int(state.get("epoch", 0))
        self.position = int(state.get("position", 0))


def create_dataloader(dataset, rank: int, world_size: int, dataset_config, collate_fn: Callable | None = None,
                      seed: int = 0) -> StatefulListLoader:
    """The loader of one data-parallel rank for ``dataset_config`` (``batch_size`` is the GLOBAL batch and must
    divide by ``world_size``). A validation config (no ``shuffle`` requested and ``drop_last`` off, or an instance
    of ``ValidDatasetConfig``) gets the exact, unpadded evaluation split."""
    bs = int(dataset_config.batch_size)
    if bs % world_size != 0:
        raise ValueError(f"batch size ({bs}) must be divisible by world_size ({world_size})")
    is_valid = type(dataset_config).__name__.startswith("Valid")
    drop_last = bool(getattr(dataset_config, "drop_last", True)) and not is_valid
    return StatefulListLoader(dataset, bs // world_size, shuffle=bool(getattr(dataset_config, "shuffle", not is_valid)),
                              seed=seed, rank=rank, world=world_size, drop_last=drop_last, collate_fn=collate_fn)
