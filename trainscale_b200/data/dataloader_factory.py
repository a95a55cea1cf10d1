"""DataLoader construction (fluent builder + one-call helpers).

After data_pipeline/data/dataloader_factory.py:45-372: `DataLoaderBuilder` with `_create_sampler`
(DistributedSampler(seed, drop_last) | seeded RandomSampler | SequentialSampler), `build_dataloader`, and
`build_distributed_dataloaders` (every rank's loader in one process, for tests).
"""
from __future__ import annotations

from typing import Callable

import torch
from torch.utils.data import DataLoader, DistributedSampler, IterableDataset, RandomSampler, SequentialSampler

from ..core.errors import DataLoadingError


class DataLoaderBuilder:
    def __init__(self, dataset=None):
        self.dataset = dataset
        self._batch_size, self._shuffle, self._seed = 8, False, 42
        self._num_workers, self._pin, self._drop_last = 0, False, False
        self._prefetch, self._persistent = None, False
        self._collate: Callable | None = None
        self._dist, self._rank, self._world = False, 0, 1

    def batch_size(self, n: int):
        if n <= 0:
            raise DataLoadingError("batch_size must be positive", batch_size=n)
        self._batch_size = n
        return self

    def shuffle(self, on: bool = True, seed: int = 42):
        self._shuffle, self._seed = on, seed
        return self

    def workers(self, n: int, prefetch_factor: int | None = None, persistent: bool = False):
        self._num_workers, self._prefetch, self._persistent = n, prefetch_factor, persistent
        return self

    def pin_memory(self, on: bool = True):
        self._pin = on
        return self

    def drop_last(self, on: bool = True):
        self._drop_last = on
        return self

    def collate(self, fn: Callable):
        self._collate = fn
        return self

    def distributed(self, rank: int, world_size: int):
        self._dist, self._rank, self._world = world_size > 1, rank, world_size
        return self

    # ---- `with_*` spelling of the reference's builder (data_pipeline/data/dataloader_factory.py:89-176)
    def with_dataset(self, dataset):
        self.dataset = dataset
        return self

    def with_batch_size(self, batch_size: int):
        return self.batch_size(batch_size)

    def with_shuffle(self, shuffle: bool):
        self._shuffle = bool(shuffle)
        return self

    def with_seed(self, seed: int):
        self._seed = int(seed)
        return self

    def with_num_workers(self, num_workers: int):
        self._num_workers = int(num_workers)
        return self

    def with_pin_memory(self, pin_memory: bool):
        return self.pin_memory(pin_memory)

    def with_drop_last(self, drop_last: bool):
        return self.drop_last(drop_last)

    def with_distributed(self, rank: int, world_size: int):
        return self.distributed(rank, world_size)

    def with_collate_fn(self, collate_fn: Callable):
        return self.collate(collate_fn)

    def with_sampler(self, sampler):
        """A sampler given here wins over the shuffle / distributed settings."""
        self._sampler = sampler
        return self

    def with_padding(self, pad_token_id: int, label_pad_token_id: int = -100, padding_side: str = "right",
                     max_length: int | None = None):
        """Pad batches with the framework collate function (`data.collate.create_collate_fn`) unless a collate function
        is set explicitly."""
        self._padding = dict(pad_token_id=pad_token_id, label_pad_token_id=label_pad_token_id,
                             padding_side=padding_side, max_length=max_length)
        return self

    def with_output_schema(self, schema):
        self._schema = schema
        return self

    def with_config(self, config):
        """Take batch size, workers, pinning, drop_last, shuffle, prefetch and worker persistence from a loader
        configuration object (attributes missing on it keep their current values)."""
        g = lambda name, cur: getattr(config, name, cur)      # noqa: E731
        self._batch_size, self._num_workers = g("batch_size", self._batch_size), g("num_workers", self._num_workers)
        self._pin, self._drop_last = g("pin_memory", self._pin), g("drop_last", self._drop_last)
        self._shuffle, self._prefetch = g("shuffle", self._shuffle), g("prefetch_factor", self._prefetch)
        self._persistent = g("persistent_workers", self._persistent)
        return self

    def _padding_collate(self):
        pad = getattr(self, "_padding", None)
        if pad is None:
            return None
        from .collate import create_collate_fn
        import inspect
        accepted = set(inspect.signature(create_collate_fn).parameters)
        kw = {k: v for k, v in pad.items() if k in accepted and v is not None}
        if getattr(self, "_schema", None) is not None and "output_schema" in accepted:
            kw["output_schema"] = self._schema
        return create_collate_fn(**kw)

    def _create_sampler(self):
        if getattr(self, "_sampler", None) is not None:
            return self._sampler
        if isinstance(self.dataset, IterableDataset):
            return None
        if self._dist:
            return DistributedSampler(self.dataset, num_replicas=self._world, rank=self._rank, shuffle=self._shuffle,
                                      seed=self._seed, drop_last=self._drop_last)
        if self._shuffle:
            return RandomSampler(self.dataset, generator=torch.Generator().manual_seed(self._seed))
        return SequentialSampler(self.dataset)

    def build(self) -> DataLoader:
        kw = dict(batch_size=self._batch_size, sampler=self._create_sampler(), num_workers=self._num_workers,
                  pin_memory=self._pin and torch.cuda.is_available(), drop_last=self._drop_last,
                  collate_fn=self._collate if self._collate is not None else self._padding_collate())
        if self._num_workers > 0:
            if self._prefetch:
                kw["prefetch_factor"] = self._prefetch
            kw["persistent_workers"] = self._persistent
        return DataLoader(self.dataset, **kw)


def build_dataloader(dataset, batch_size: int = 8, shuffle: bool = False, seed: int = 42, num_workers: int = 0,
                     pin_memory: bool = False, drop_last: bool = False, collate_fn=None, distributed: bool = False,
                     rank: int = 0, world_size: int = 1, prefetch_factor=None, persistent_workers=False, *,
                     pad_token_id: int | None = None, label_pad_token_id: int = -100, padding_side: str = "right",
                     max_length: int | None = None, output_schema=None, config=None) -> DataLoader:
    """One call for a loader.  `pad_token_id` (with `label_pad_token_id`, `padding_side`, `max_length`) selects the
    padding collate function unless `collate_fn` is given; `output_schema` filters / casts the batch's keys; `config`
    (a loader configuration object) supplies batch size, workers, pinning and the like
    (data_pipeline/data/dataloader_factory.py:225-300)."""
    b = (DataLoaderBuilder(dataset).batch_size(batch_size).shuffle(shuffle, seed)
         .workers(num_workers, prefetch_factor, persistent_workers).pin_memory(pin_memory).drop_last(drop_last))
    if config is not None:
        b.with_config(config)
    if pad_token_id is not None:
        b.with_padding(pad_token_id, label_pad_token_id, padding_side, max_length)
    if output_schema is not None:
        b.with_output_schema(output_schema)
    if collate_fn is not None:
        b.collate(collate_fn)
    if distributed:
        b.distributed(rank, world_size)
    return b.build()


def build_distributed_dataloaders(dataset, world_size: int, **kw) -> list[DataLoader]:
    return [build_dataloader(dataset, distributed=True, rank=r, world_size=world_size, **kw) for r in range(world_size)]
