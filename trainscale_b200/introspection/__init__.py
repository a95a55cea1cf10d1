"""Dataset discovery and column mapping.

After data_pipeline/introspection/introspector.py:83-511 (`DatasetMetadata`, `DatasetIntrospector.discover`,
`get_default_split`, `levenshtein_distance`) and column_mapper.py:180-356 (`ColumnMapper.map_columns` with fuzzy
matching).  Local files / in-memory datasets are introspected directly; hub datasets go through `datasets` when it
is importable and the network is reachable.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Mapping, Sequence

from ..core.errors import ColumnNotFoundError, DatasetNotFoundError, SplitNotFoundError
from ..core.types import Err, Ok, Result


def levenshtein_distance(a: str, b: str) -> int:
    if a == b:
        return 0
    if not a or not b:
        return len(a) or len(b)
    prev = list(range(len(b) + 1))
    for i, ca in enumerate(a, 1):
        cur = [i]
        for j, cb in enumerate(b, 1):
            cur.append(min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (ca != cb)))
        prev = cur
    return prev[-1]


@dataclass
class DatasetMetadata:
    name: str
    configs: list[str] = field(default_factory=list)
    splits: dict[str, int | None] = field(default_factory=dict)     # split -> rows (None if unknown)
    columns: dict[str, str] = field(default_factory=dict)           # column -> dtype name
    source: str = "memory"


class DatasetIntrospector:
    SPLIT_PREFERENCE = ("train", "train_sft", "training", "validation", "valid", "dev", "test")

    def __init__(self, token: str | None = None):
        self.token = token

    def discover(self, name_or_data, config_name: str | None = None) -> Result:
        try:
            if isinstance(name_or_data, Mapping):   # {"split": rows}
                return Ok(self._from_memory("memory", dict(name_or_data)))
            if isinstance(name_or_data, (list, tuple)):
                return Ok(self._from_memory("memory", {"train": list(name_or_data)}))
            p = Path(str(name_or_data))
            if p.exists():
                return Ok(self._from_path(p))
            return Ok(self._from_hub(str(name_or_data), config_name))
        except DatasetNotFoundError as e:
            return Err(e)

    @staticmethod
    def _columns_of(rows: Sequence[Mapping[str, Any]]) -> dict[str, str]:
        cols = {}
        for r in rows[:16]:
            for k, v in r.items():
                cols.setdefault(k, type(v).__name__)
        return cols

    def _from_memory(self, name, splits) -> DatasetMetadata:
        first = next(iter(splits.values()), [])
        return DatasetMetadata(name, [], {k: len(v) for k, v in splits.items()}, self._columns_of(list(first)), "memory")

    def _from_path(self, p: Path) -> DatasetMetadata:
        from ..data.local_datasets import load_local_dataset
        files = [p] if p.is_file() else sorted(q for q in p.iterdir() if q.suffix in (".json", ".jsonl", ".csv", ".txt", ".parquet"))
        if not files:
            raise DatasetNotFoundError(f"no data files under {p}")
        splits = {f.stem: load_local_dataset(f) for f in files}
        md = self._from_memory(str(p), splits)
        md.source = "local"
        return md

    def _from_hub(self, name: str, config_name) -> DatasetMetadata:
        try:
            import datasets
            configs = datasets.get_dataset_config_names(name, token=self.token)
            cfg = config_name or (configs[0] if configs else None)
            infos = datasets.get_dataset_split_names(name, cfg, token=self.token)
            return DatasetMetadata(name, list(configs), {s: None for s in infos}, {}, "hub")
        except Exception as e:   # noqa: BLE001
            raise DatasetNotFoundError(f"dataset {name!r} not found locally and the hub is unreachable", cause=e)

    def get_default_split(self, md: DatasetMetadata) -> Result:
        for s in self.SPLIT_PREFERENCE:
            if s in md.splits:
                return Ok(s)
        if md.splits:
            return Ok(next(iter(md.splits)))
        return Err(SplitNotFoundError(f"dataset {md.name} has no splits"))


class ColumnMapper:
    """Map the columns a template needs onto the columns a dataset has (exact, alias, then fuzzy)."""

    ALIASES = {"text": ("content", "document", "body", "passage"), "prompt": ("question", "query", "instruction", "input"),
               "completion": ("answer", "response", "output", "target"), "chosen": ("preferred", "winner", "accepted"),
               "rejected": ("dispreferred", "loser", "refused"), "messages": ("conversation", "conversations", "dialog")}

    def __init__(self, max_distance: int = 2, case_sensitive: bool = False):
        self.max_distance, self.case_sensitive = max_distance, case_sensitive

    def _norm(self, s: str) -> str:
        return s if self.case_sensitive else s.lower()

    def _find_best_match(self, wanted: str, available: Sequence[str]) -> str | None:
        w = self._norm(wanted)
        for a in available:
            if self._norm(a) == w:
                return a
        for alias in self.ALIASES.get(w, ()):
            for a in available:
                if self._norm(a) == alias:
                    return a
        best, best_d = None, self.max_distance + 1
        for a in available:
            d = levenshtein_distance(w, self._norm(a))
            if d < best_d:
                best, best_d = a, d
        return best if best_d <= self.max_distance else None

    def map_columns(self, required: Sequence[str], available: Sequence[str], explicit: Mapping[str, str] | None = None
                    ) -> Result:
        out, missing = {}, []
        for r in required:
            if explicit and r in explicit:
                if explicit[r] not in available:
                    return Err(ColumnNotFoundError(f"mapped column {explicit[r]!r} does not exist", available=list(available)))
                out[r] = explicit[r]
                continue
            m = self._find_best_match(r, available)
            if m is None:
                missing.append(r)
            else:
                out[r] = m
        if missing:
            return Err(ColumnNotFoundError(f"no column matches {missing}", available=list(available)))
        return Ok(out)
