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
from ..utils.refargs import ANY, reference_kwargs


@reference_kwargs(s1="a", s2="b")
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
    default_config: str | None = None

    def get_config(self, name: str) -> "ConfigInfo | None":
        """Typed record of one configuration ("default" names the only one of a dataset without configurations)."""
        if name in self.configs or (not self.configs and name == "default"):
            return ConfigInfo(name, tuple(SplitInfo(k, v) for k, v in self.splits.items()))
        return None

    def get_all_splits(self, config: str | None = None) -> list[str]:
        """Split names in their declared order.  Splits are recorded for the configuration that was discovered, so an
        unknown `config` yields an empty list."""
        if config is not None and self.get_config(config) is None:
            return []
        return list(self.splits)


class DatasetIntrospector:
    SPLIT_PREFERENCE = ("train", "train_sft", "training", "validation", "valid", "dev", "test")

    def __init__(self, token: str | None = None):
        self.token = token
        self._cache: dict = {}

    def clear_cache(self) -> None:
        self._cache.clear()

    @reference_kwargs({"trust_remote_code": ANY}, dataset_id="name_or_data")
    def discover(self, name_or_data, config_name: str | None = None) -> Result:
        """Metadata of rows in memory, of a local file / directory, or of a hub dataset.  Hub and path look-ups are
        cached per (name, config) until `clear_cache()`."""
        key = (str(name_or_data), config_name) if isinstance(name_or_data, (str, Path)) else None
        if key is not None and key in self._cache:
            return Ok(self._cache[key])
        r = self._discover(name_or_data, config_name)
        if key is not None and r.is_ok():
            self._cache[key] = r.unwrap()
        return r

    def _discover(self, name_or_data, config_name: str | None = None) -> Result:
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

    def get_default_split(self, md: "DatasetMetadata | str | None" = None, config: str | None = None, *,
                          dataset_id=None) -> Result:
        """Preferred split of discovered metadata, or of a dataset given by id / path / rows (discovered first)."""
        md = md if md is not None else dataset_id
        if not isinstance(md, DatasetMetadata):
            r = self.discover(md, config)
            if r.is_err():
                return r
            md = r.unwrap()
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

    def __init__(self, max_distance: int = 2, case_sensitive: bool = False,
                 custom_patterns: Mapping[str, Sequence[str]] | None = None, min_fuzzy_score: float | None = None):
        """`custom_patterns`: extra aliases {wanted column: (accepted names...)}; `min_fuzzy_score` in [0, 1]: a fuzzy
        match must have at least this normalised similarity (in addition to the edit-distance bound)."""
        self.max_distance, self.case_sensitive, self.min_fuzzy_score = max_distance, case_sensitive, min_fuzzy_score
        if custom_patterns:
            self.ALIASES = {**self.ALIASES}
            for k, names in custom_patterns.items():
                self.ALIASES[k] = tuple(self.ALIASES.get(k, ())) + tuple(n.lower() for n in names)

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
        if best is not None and self.min_fuzzy_score is not None and \
                normalized_similarity(wanted, best) < self.min_fuzzy_score:
            return None
        return best if best_d <= self.max_distance else None

    def map_columns(self, required: Sequence[str] | None = None, available: Sequence[str] | None = None,
                    explicit: Mapping[str, str] | None = None, *, source_columns: Sequence[str] | None = None,
                    target_schema: Sequence[str] | None = None, explicit_mapping: Mapping[str, str] | None = None) -> Result:
        """{wanted column: dataset column}.  `map_columns(required, available, explicit)`; the reference names the same
        three things `target_schema`, `source_columns`, `explicit_mapping` and passes the SOURCE columns first."""
        if source_columns is not None or target_schema is not None:
            required = target_schema if target_schema is not None else available
            available = source_columns if source_columns is not None else required
        explicit = explicit if explicit is not None else explicit_mapping
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

    STANDARD_SCHEMA = ("text", "prompt", "completion", "chosen", "rejected", "messages")

    def suggest_mappings(self, source_columns: Sequence[str], target_schema: Sequence[str] | None = None) -> list:
        """`ColumnMatch` for every target column (the standard training columns by default) that some source column
        matches; nothing is required, so an unknown dataset can be explored
        (data_pipeline/introspection/column_mapper.py:305-330)."""
        return match_columns(source_columns, list(target_schema or self.STANDARD_SCHEMA))


# ------------------------------------------------------------------------------------------------ reference surface
@dataclass(frozen=True)
class FeatureInfo:
    """One column: name, dtype name, whether its values are lists and whether they nest mappings."""
    name: str
    dtype: str
    is_list: bool = False
    is_nested: bool = False

    @classmethod
    def of(cls, name: str, value: Any) -> "FeatureInfo":
        is_list = isinstance(value, (list, tuple))
        inner = value[0] if is_list and value else value
        return cls(name, type(inner).__name__ if is_list else type(value).__name__, is_list, isinstance(inner, Mapping))


@dataclass(frozen=True)
class SplitInfo:
    name: str
    num_examples: int | None = None
    num_bytes: int | None = None


@dataclass(frozen=True)
class ConfigInfo:
    name: str
    splits: tuple = ()
    description: str | None = None


@dataclass(frozen=True)
class ColumnMatch:
    """How a required column was matched: exact name, known alias ("pattern") or edit distance ("fuzzy")."""
    source: str
    target: str
    confidence: float
    match_type: str


def normalized_similarity(s1: str, s2: str) -> float:
    """1 - edit distance / longer length, case-insensitive; 1.0 for two empty strings."""
    if not s1 and not s2:
        return 1.0
    if not s1 or not s2:
        return 0.0
    return 1.0 - levenshtein_distance(s1.lower(), s2.lower()) / max(len(s1), len(s2))


def describe_dataset(md: DatasetMetadata, sample_row: Mapping[str, Any] | None = None) -> tuple[ConfigInfo, ...]:
    """`DatasetMetadata` as typed records: one `ConfigInfo` per configuration (a single "default" one when the dataset
    has none), each with its `SplitInfo`s."""
    splits = tuple(SplitInfo(k, v) for k, v in md.splits.items())
    return tuple(ConfigInfo(c, splits) for c in (md.configs or ["default"]))


def describe_features(rows: Sequence[Mapping[str, Any]]) -> tuple[FeatureInfo, ...]:
    seen: dict[str, FeatureInfo] = {}
    for r in rows[:16]:
        for k, v in r.items():
            seen.setdefault(k, FeatureInfo.of(k, v))
    return tuple(seen.values())


def match_columns(source_columns: Sequence[str], target_schema: Sequence[str], min_score: float = 0.7) -> list[ColumnMatch]:
    """Best source column for every target column with how it was found; targets without a match above `min_score`
    are left out."""
    mapper = ColumnMapper(max_distance=10 ** 6)
    out = []
    for t in target_schema:
        exact = next((s for s in source_columns if s.lower() == t.lower()), None)
        if exact is not None:
            out.append(ColumnMatch(exact, t, 1.0, "exact"))
            continue
        alias = next((s for s in source_columns if s.lower() in mapper.ALIASES.get(t.lower(), ())), None)
        if alias is not None:
            out.append(ColumnMatch(alias, t, 0.9, "pattern"))
            continue
        best = max(source_columns, key=lambda s: normalized_similarity(s, t), default=None)
        if best is not None and normalized_similarity(best, t) >= min_score:
            out.append(ColumnMatch(best, t, normalized_similarity(best, t), "fuzzy"))
    return out


def fuzzy_match_columns(source_columns: Sequence[str], target_schema: Sequence[str],
                        explicit_mapping: Mapping[str, str] | None = None, min_score: float = 0.7) -> Result:
    """{target column: source column} as a Result; explicit mappings win, every other target needs a match of at least
    `min_score` (data_pipeline/introspection/column_mapper.py:337)."""
    out: dict[str, str] = {}
    for t, s in (explicit_mapping or {}).items():
        if s not in source_columns:
            return Err(ColumnNotFoundError(f"mapped column {s!r} does not exist", available=list(source_columns)))
        out[t] = s
    rest = [t for t in target_schema if t not in out]
    found = {m.target: m.source for m in match_columns(source_columns, rest, min_score)}
    missing = [t for t in rest if t not in found]
    if missing:
        return Err(ColumnNotFoundError(f"no column matches {missing}", available=list(source_columns)))
    out.update(found)
    return Ok(out)


_INTROSPECTOR: list = [None]


def get_introspector(token: str | None = None) -> DatasetIntrospector:
    if _INTROSPECTOR[0] is None:
        _INTROSPECTOR[0] = DatasetIntrospector(token=token)
    return _INTROSPECTOR[0]


def discover_dataset(dataset_id, token: str | None = None) -> Result:
    return get_introspector(token).discover(dataset_id)


def get_default_split(dataset_id, config: str | None = None, token: str | None = None) -> Result:
    """Preferred split (train first) of a dataset given by id, path, rows or an already discovered `DatasetMetadata`."""
    intro = get_introspector(token)
    if isinstance(dataset_id, DatasetMetadata):
        return intro.get_default_split(dataset_id)
    md = intro.discover(dataset_id, config)
    return md if md.is_err() else intro.get_default_split(md.unwrap())


# ---- column-role patterns as compiled expressions (data_pipeline/introspection/column_mapper.py), built from the
# alias table `ColumnMapper` matches with, and the split / config preferences of the introspector
import re as _re  # noqa: E402


def _role_patterns(*names: str) -> tuple:
    return tuple(_re.compile(f"^{_re.escape(n)}$", _re.I) for n in names)


INSTRUCTION_PATTERNS = _role_patterns("instruction", "prompt", *ColumnMapper.ALIASES["prompt"], "user_input", "user_message", "human")
INPUT_PATTERNS = _role_patterns("input", "context", "text", *ColumnMapper.ALIASES["text"], "source")
OUTPUT_PATTERNS = _role_patterns("output", "completion", *ColumnMapper.ALIASES["completion"], "assistant", "generated")
LABEL_PATTERNS = _role_patterns("label", "labels", "class", "category", "target")
STANDARD_SCHEMA = {"instruction": INSTRUCTION_PATTERNS, "input": INPUT_PATTERNS, "output": OUTPUT_PATTERNS,
                   "label": LABEL_PATTERNS}
DEFAULT_SPLIT_PRIORITY = DatasetIntrospector.SPLIT_PREFERENCE
DEFAULT_CONFIG_NAMES = frozenset({"default", "plain_text", "en", "english"})
