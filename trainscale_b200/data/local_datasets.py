"""Readers for local dataset files (jsonl / json / csv / txt / parquet) returning lists of row dicts."""
from __future__ import annotations

import csv
import json
from pathlib import Path

from ..core.errors import DataLoadingError


def load_local_dataset(path) -> list[dict]:
    p = Path(path)
    try:
        if p.suffix == ".jsonl":
            return [json.loads(l) for l in p.read_text().splitlines() if l.strip()]
        if p.suffix == ".json":
            data = json.loads(p.read_text())
            return data if isinstance(data, list) else data.get("data", [data])
        if p.suffix == ".csv":
            with open(p, newline="") as f:
                return list(csv.DictReader(f))
        if p.suffix == ".txt":
            return [{"text": l} for l in p.read_text().splitlines() if l.strip()]
        if p.suffix == ".parquet":
            import pyarrow.parquet as pq
            return pq.read_table(p).to_pylist()
    except (OSError, ValueError) as e:
        raise DataLoadingError(f"cannot read {p}", cause=e)
    raise DataLoadingError(f"unsupported dataset file type {p.suffix!r}")
