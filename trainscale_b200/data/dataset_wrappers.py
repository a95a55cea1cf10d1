"""Map-style and streaming datasets that run the prompt engine per item.

After data_pipeline/data/dataset_wrappers.py:41-377 (`PreprocessedDataset` with a per-index cache, column mapping
and tensor conversion; `StreamingPreprocessedDataset` sharded per DataLoader worker and rank, `skip_errors`).
"""
from __future__ import annotations

from typing import Any, Callable, Iterable, Mapping

import torch
from torch.utils.data import Dataset, IterableDataset, get_worker_info

from ..core.errors import PipelineError
from ..utils.refargs import ANY, reference_kwargs


def _to_tensors(d: Mapping[str, Any]) -> dict:
    out = {}
    for k, v in d.items():
        if isinstance(v, (list, tuple)) and v and isinstance(v[0], (int, bool)):
            out[k] = torch.tensor(v, dtype=torch.long)
        elif isinstance(v, (list, tuple)) and v and isinstance(v[0], float):
            out[k] = torch.tensor(v, dtype=torch.float32)
        elif isinstance(v, bool):
            out[k] = torch.tensor(int(v))
        elif isinstance(v, (int, float)):
            out[k] = torch.tensor(v)
        else:
            try:
                out[k] = torch.tensor(v)
            except (ValueError, TypeError, RuntimeError):
                out[k] = v
    return out


class PreprocessedDataset(Dataset):
    @reference_kwargs(hf_dataset="dataset", prompt_engine="engine", cache_enabled="cache")
    def __init__(self, dataset, engine, column_mapping: Mapping[str, str] | None = None, cache: bool = True,
                 max_cache_items: int = 1 << 20, transform: Callable | None = None):
        """`transform(item) -> item` runs on every processed example (after tensor conversion, before caching)."""
        self.transform = transform
        self.dataset, self.engine, self.mapping = dataset, engine, dict(column_mapping or {})
        self.cache = {} if cache else None
        self.max_cache_items = max_cache_items

    def __len__(self):
        return len(self.dataset)

    def _apply_mapping(self, row: Mapping[str, Any]) -> dict:
        row = dict(row)
        for src, dst in self.mapping.items():
            if src in row:
                row[dst] = row[src]
        return row

    def __getitem__(self, i):
        if self.cache is not None and i in self.cache:
            return self.cache[i]
        ex = self.engine.process(self._apply_mapping(self.dataset[i]))
        item = _to_tensors(ex.to_dict())
        if getattr(self, "transform", None) is not None:
            item = self.transform(item)
        if self.cache is not None and len(self.cache) < self.max_cache_items:
            self.cache[i] = item
        return item

    def clear_cache(self) -> None:
        if self.cache is not None:
            self.cache.clear()

    @property
    def features(self):
        """Feature description of the wrapped dataset (None when it has none)."""
        return getattr(self.dataset, "features", None)

    def select(self, indices) -> "PreprocessedDataset":
        """The same preprocessing over a subset of rows (data_pipeline/data/dataset_wrappers.py:179-196)."""
        indices = list(indices)
        sub = self.dataset.select(indices) if hasattr(self.dataset, "select") else [self.dataset[i] for i in indices]
        return PreprocessedDataset(sub, self.engine, self.mapping, self.cache is not None, self.max_cache_items,
                                   getattr(self, "transform", None))


class _BufferShuffle:
    """Iterable that yields the rows of `source` through a buffer of `buffer_size` rows, picking a random one each
    time (the usual approximate shuffle of a stream); a fresh pass re-seeds, so every pass has the same order."""

    def __init__(self, source, buffer_size: int, seed: int = 0):
        self.source, self.buffer_size, self.seed = source, max(1, buffer_size), seed

    def __iter__(self):
        import random
        rng, buf = random.Random(self.seed), []
        for row in self.source:
            if len(buf) < self.buffer_size:
                buf.append(row)
                continue
            i = rng.randrange(len(buf))
            yield buf[i]
            buf[i] = row
        rng.shuffle(buf)
        yield from buf


class StreamingPreprocessedDataset(IterableDataset):
    @reference_kwargs(hf_iterable="iterable", prompt_engine="engine")
    def __init__(self, iterable: Iterable, engine, column_mapping: Mapping[str, str] | None = None, rank: int = 0,
                 world_size: int = 1, skip_errors: bool = True, max_items: int | None = None,
                 buffer_size: int | None = None, transform: Callable | None = None):
        """`buffer_size`: shuffle the stream through a buffer of that many rows (see `shuffle`); `transform(item)` runs
        on every processed example."""
        self.transform = transform
        if buffer_size:
            iterable = iterable.shuffle(buffer_size=buffer_size) if hasattr(iterable, "shuffle") \
                else _BufferShuffle(iterable, buffer_size)
        self.iterable, self.engine, self.mapping = iterable, engine, dict(column_mapping or {})
        self.rank, self.world, self.skip_errors, self.max_items = rank, world_size, skip_errors, max_items
        self.num_errors = 0

    def shuffle(self, buffer_size: int = 1000, seed: int = 0) -> "StreamingPreprocessedDataset":
        """The same stream in shuffled order: the source's own `shuffle(buffer_size=..., seed=...)` when it has one
        (HuggingFace iterable datasets), else a reservoir of `buffer_size` rows drawn from at random."""
        src = self.iterable
        if hasattr(src, "shuffle"):
            shuffled = src.shuffle(buffer_size=buffer_size, seed=seed)
        else:
            shuffled = _BufferShuffle(src, buffer_size, seed)
        return StreamingPreprocessedDataset(shuffled, self.engine, self.mapping, self.rank, self.world, self.skip_errors,
                                            self.max_items)

    def __iter__(self):
        info = get_worker_info()
        nw, wid = (info.num_workers, info.id) if info else (1, 0)
        shard, nshards = self.rank * nw + wid, self.world * nw
        src = self.iterable
        if hasattr(src, "shard") and nshards > 1:
            try:
                src, shard, nshards = src.shard(num_shards=nshards, index=shard), 0, 1
            except Exception:   # noqa: BLE001 - not every iterable dataset can shard itself
                pass
        n = 0
        for idx, row in enumerate(src):
            if idx % nshards != shard:
                continue
            row = dict(row)
            for s, d in self.mapping.items():
                if s in row:
                    row[d] = row[s]
            try:
                ex = self.engine.process(row)
            except PipelineError:
                self.num_errors += 1
                if self.skip_errors:
                    continue
                raise
            item = _to_tensors(ex.to_dict())
            yield self.transform(item) if getattr(self, "transform", None) is not None else item
            n += 1
            if self.max_items is not None and n >= self.max_items:
                return


def create_preprocessed_dataset(dataset, engine, streaming: bool = False, **kw):
    if streaming or not hasattr(dataset, "__len__"):
        return StreamingPreprocessedDataset(dataset, engine, **kw)
    kw.pop("rank", None)
    kw.pop("world_size", None)
    kw.pop("skip_errors", None)
    kw.pop("max_items", None)
    return PreprocessedDataset(dataset, engine, **kw)
