"""Token budgets: smart truncation, per-column budget distribution, padding-length policies, dynamic collate.

Behaviour after data_pipeline/preprocessing/length_manager.py:92-1765:
  * SMART truncation cascade - cut at a sentence end if that keeps >= 50 % of the budget, else a clause end
    (>= 40 %), else a word end (>= 30 %), else hard cut (:446-546);
  * TokenEstimator at 3.8 characters per token (:556);
  * TokenAwareContentDistributor modes EQUAL / RATIO / PROPORTIONAL / PRIORITY / ADAPTIVE (:816-1134; ADAPTIVE gives
    label columns a 60 % floor, weights 1/(priority+1), label columns x1.5);
  * padding strategies DO_NOT_PAD / LONGEST / MAX_LENGTH / BUCKET (bisect over boundaries) / POWER_OF_TWO (:1375-1449);
  * special-token budget of 10 and buckets (64 ... 4096) as defaults (:260).
"""
from __future__ import annotations

import bisect
import math
import re
from dataclasses import dataclass, field
from typing import Callable, Mapping, Sequence

import torch

from ..utils.refargs import ANY, reference_kwargs

from ..config.data_schema import ContentDistributionMode, PaddingStrategy, TruncationStrategy

DEFAULT_BUCKETS = (64, 128, 256, 512, 1024, 2048, 4096)
CHARS_PER_TOKEN = 3.8
INT_MAX = 2 ** 31 - 1


def checked_add(a: int, b: int) -> int:
    r = a + b
    if r > INT_MAX or r < -INT_MAX:
        raise OverflowError(f"length arithmetic overflow: {a} + {b}")
    return r


def checked_mul(a: int, b: int) -> int:
    r = a * b
    if abs(r) > INT_MAX:
        raise OverflowError(f"length arithmetic overflow: {a} * {b}")
    return r


@dataclass
class ColumnContentConfig:
    name: str
    priority: int = 0              # 0 = most important
    ratio: float | None = None
    min_tokens: int = 0
    max_tokens: int | None = None
    is_label: bool = False
    truncation: TruncationStrategy = TruncationStrategy.SMART


@dataclass
class ColumnLengthConfig:
    """Limits of one text column (data_pipeline/preprocessing/length_manager.py:231-257).  `max_length` and
    `max_tokens` are the same limit in tokens; `max_chars` is a hard limit in characters and wins over both."""
    name: str = ""
    max_length: int | None = None
    truncation: TruncationStrategy = TruncationStrategy.RIGHT
    max_chars: int | None = None
    max_tokens: int | None = None
    preserve_ratio: float = 0.0
    priority: int = 0

    def __post_init__(self):
        if self.max_tokens is None:
            self.max_tokens = self.max_length
        elif self.max_length is None:
            self.max_length = self.max_tokens
        if not 0.0 <= self.preserve_ratio <= 1.0:
            raise ValueError("preserve_ratio must lie in [0, 1]")


@dataclass
class LengthManagerConfig:
    max_total_length: int = 2048
    padding_strategy: PaddingStrategy = PaddingStrategy.MAX_LENGTH
    truncation_strategy: TruncationStrategy = TruncationStrategy.RIGHT
    bucket_boundaries: tuple[int, ...] = DEFAULT_BUCKETS
    special_tokens_budget: int = 10
    chars_per_token: float = CHARS_PER_TOKEN
    per_column: Mapping[str, ColumnLengthConfig] = field(default_factory=dict)
    pad_to_multiple_of: int | None = None

    # the reference's field names for the same settings
    @property
    def total_max_length(self) -> int:
        return self.max_total_length

    @property
    def default_truncation(self) -> TruncationStrategy:
        return self.truncation_strategy

    @property
    def chars_per_token_estimate(self) -> float:
        return self.chars_per_token


_SENT = re.compile(r"[.!?]['\")\]]*\s")
_CLAUSE = re.compile(r"[,;:]\s|\s[-–—]\s")
_WORD = re.compile(r"\s")


def _last_boundary(text: str, pattern: re.Pattern, limit: int) -> int:
    pos = -1
    for m in pattern.finditer(text, 0, limit):
        pos = m.end()
    return pos


@reference_kwargs(max_chars="limit")
def find_sentence_boundary(text: str, limit: int) -> int:
    return _last_boundary(text, _SENT, limit)


@reference_kwargs(max_chars="limit")
def find_clause_boundary(text: str, limit: int) -> int:
    return _last_boundary(text, _CLAUSE, limit)


@reference_kwargs(max_chars="limit")
def find_word_boundary(text: str, limit: int) -> int:
    return _last_boundary(text, _WORD, limit)


def smart_truncate(text: str, max_chars: int, strategy: TruncationStrategy = TruncationStrategy.SMART,
                   ellipsis: str = "") -> str:
    """Truncate `text` to at most max_chars characters."""
    strategy = TruncationStrategy(strategy)
    if max_chars <= 0:
        return ""
    if len(text) <= max_chars or strategy == TruncationStrategy.NONE:
        return text
    if strategy == TruncationStrategy.LEFT:
        return text[-max_chars:]
    if strategy == TruncationStrategy.MIDDLE:
        head = max_chars // 2
        return text[:head] + text[len(text) - (max_chars - head):]
    if strategy == TruncationStrategy.RIGHT:
        return text[:max_chars]
    budget = max_chars - len(ellipsis)
    for finder, frac in ((find_sentence_boundary, 0.5), (find_clause_boundary, 0.4), (find_word_boundary, 0.3)):
        cut = finder(text, budget)
        if cut >= frac * budget:
            return text[:cut].rstrip() + ellipsis
    return text[:budget] + ellipsis


class TokenEstimator:
    """Cheap token counts: exact when a tokenizer is given and `exact`, else len(text)/chars_per_token."""

    def __init__(self, tokenizer=None, chars_per_token: float = CHARS_PER_TOKEN, exact: bool = False):
        self.tokenizer, self.cpt, self.exact = tokenizer, chars_per_token, exact

    def estimate(self, text: str) -> int:
        if not text:
            return 0
        if self.exact and self.tokenizer is not None:
            return self.tokenizer.count_tokens(text)
        return max(1, int(len(text) / self.cpt + 0.5))

    def chars_for(self, tokens: int) -> int:
        return int(tokens * self.cpt)

    def estimate_tokens(self, text: str) -> int:
        """Token count of `text`: the tokenizer's when one is attached (any of count_tokens / encode / __call__),
        else the characters-per-token estimate."""
        if not text:
            return 0
        tk = self.tokenizer
        if tk is not None:
            try:
                if hasattr(tk, "count_tokens"):
                    return max(1, int(tk.count_tokens(text)))
                if hasattr(tk, "encode"):
                    ids = tk.encode(text)
                    return max(1, len(ids["input_ids"] if isinstance(ids, dict) else ids))
            except Exception:   # noqa: BLE001 - an unusable tokenizer falls back to the estimate
                pass
        return max(1, int(len(text) / self.cpt + 0.5))

    def tokens_to_chars(self, tokens: int) -> int:
        return 0 if tokens <= 0 else int(math.ceil(tokens * self.cpt))


class TokenAwareContentDistributor:
    """Split a total token budget over text columns and truncate each column to its share."""

    @reference_kwargs(total_max_tokens="max_length", distribution_mode="mode")
    def __init__(self, mode: ContentDistributionMode = ContentDistributionMode.PROPORTIONAL, max_length: int = 2048,
                 columns: Sequence[ColumnContentConfig] = (), special_tokens_budget: int = 10, tokenizer=None,
                 chars_per_token: float = CHARS_PER_TOKEN, exact: bool = False, *,
                 column_ratios: Mapping[str, float] | None = None,
                 column_configs: Mapping[str, ColumnContentConfig] | None = None,
                 default_truncation: TruncationStrategy | str | None = None):
        """`column_ratios` ({name: share}) and `column_configs` ({name: ColumnContentConfig}) are the reference's
        mapping forms of `columns`; `default_truncation` applies to columns that come from ratios alone."""
        if isinstance(mode, int) and not isinstance(mode, ContentDistributionMode):      # (total_max_tokens, mode, ...)
            mode, max_length = (max_length if not isinstance(max_length, int) else ContentDistributionMode.PROPORTIONAL), mode
        self.mode = ContentDistributionMode(getattr(mode, "value", mode))
        self.max_length, self.special = max_length, special_tokens_budget
        trunc = TruncationStrategy(default_truncation) if default_truncation is not None else TruncationStrategy.SMART
        cols = {c.name: c for c in columns}
        for n, r in (column_ratios or {}).items():
            cols.setdefault(n, ColumnContentConfig(n, ratio=r, truncation=trunc))
        for n, c in (column_configs or {}).items():
            cols[n] = c if c.name == n else ColumnContentConfig(**{**c.__dict__, "name": n})
        self.columns = cols
        self.estimator = TokenEstimator(tokenizer, chars_per_token, exact)

    def _cfg(self, name: str) -> ColumnContentConfig:
        return self.columns.get(name) or ColumnContentConfig(name)

    @property
    def available_tokens(self) -> int:
        """Token budget left for content once the special tokens' headroom is taken out."""
        return max(0, self.max_length - self.special)

    def allocate(self, lengths: Mapping[str, int]) -> dict[str, int]:
        """lengths: estimated tokens per column -> allotted tokens per column (sum <= budget)."""
        budget = max(0, self.max_length - self.special)
        names = list(lengths)
        if not names:
            return {}
        if sum(lengths.values()) <= budget:
            return dict(lengths)
        fn = {ContentDistributionMode.EQUAL: self._allocate_equal, ContentDistributionMode.RATIO: self._allocate_ratio,
              ContentDistributionMode.PROPORTIONAL: self._allocate_proportional,
              ContentDistributionMode.PRIORITY: self._allocate_priority,
              ContentDistributionMode.ADAPTIVE: self._allocate_adaptive}[self.mode]
        alloc = fn(lengths, budget)
        for n in names:   # clamp to configured limits and to what the column needs
            c = self._cfg(n)
            a = min(alloc.get(n, 0), lengths[n])
            if c.max_tokens is not None:
                a = min(a, c.max_tokens)
            alloc[n] = max(0, a)
        self._redistribute_slack(alloc, lengths, budget)
        return alloc

    @staticmethod
    def _redistribute_slack(alloc, lengths, budget):
        slack = budget - sum(alloc.values())
        while slack > 0:
            hungry = [n for n in alloc if alloc[n] < lengths[n]]
            if not hungry:
                break
            share = max(1, slack // len(hungry))
            moved = 0
            for n in hungry:
                give = min(share, lengths[n] - alloc[n], slack - moved)
                alloc[n] += give
                moved += give
                if moved >= slack:
                    break
            if moved == 0:
                break
            slack -= moved

    def _allocate_equal(self, lengths, budget):
        share = budget // len(lengths)
        return {n: share for n in lengths}

    def _allocate_ratio(self, lengths, budget):
        ratios = {n: (self._cfg(n).ratio if self._cfg(n).ratio is not None else 0.0) for n in lengths}
        unset = [n for n, r in ratios.items() if r <= 0]
        rest = max(0.0, 1.0 - sum(ratios.values()))
        for n in unset:
            ratios[n] = rest / len(unset) if unset else 0.0
        tot = sum(ratios.values()) or 1.0
        return {n: int(budget * ratios[n] / tot) for n in lengths}

    def _allocate_proportional(self, lengths, budget):
        tot = sum(lengths.values()) or 1
        return {n: int(budget * lengths[n] / tot) for n in lengths}

    def _allocate_priority(self, lengths, budget):
        alloc, left = {}, budget
        for n in sorted(lengths, key=lambda k: self._cfg(k).priority):
            alloc[n] = min(lengths[n], left)
            left -= alloc[n]
        return alloc

    def _allocate_adaptive(self, lengths, budget):
        labels = [n for n in lengths if self._cfg(n).is_label]
        alloc = {n: 0 for n in lengths}
        left = budget
        if labels:   # labels first: up to 60 % of the budget is reserved for them
            floor = int(0.6 * budget)
            need = sum(lengths[n] for n in labels)
            give = min(need, floor)
            for n in labels:
                alloc[n] = int(give * lengths[n] / max(need, 1))
            left -= sum(alloc[n] for n in labels)
        weights = {n: (1.0 / (self._cfg(n).priority + 1)) * (1.5 if self._cfg(n).is_label else 1.0) for n in lengths}
        want = {n: max(0, lengths[n] - alloc[n]) for n in lengths}
        wsum = sum(weights[n] for n in lengths if want[n] > 0) or 1.0
        for n in lengths:
            if want[n] > 0:
                alloc[n] += min(want[n], int(left * weights[n] / wsum))
        return alloc

    @reference_kwargs(text_columns="columns")
    def distribute(self, example: Mapping[str, str], columns: Sequence[str] | None = None,
                   label_column: str | None = None) -> dict[str, str]:
        """Truncate the text columns of `example` so that together they fit the budget.  `label_column` is treated as
        a label for this call (labels are served first in the adaptive mode) and is included in the columns."""
        if label_column is not None and label_column in example:
            import dataclasses
            cur = self._cfg(label_column)
            if not cur.is_label:
                self.columns = {**self.columns, label_column: dataclasses.replace(cur, is_label=True)}
            if columns is not None and label_column not in columns:
                columns = list(columns) + [label_column]
        cols = [c for c in (columns or example.keys()) if isinstance(example.get(c), str)]
        lengths = {c: self.estimator.estimate(example[c]) for c in cols}
        alloc = self.allocate(lengths)
        out = dict(example)
        for c in cols:
            if alloc[c] < lengths[c]:
                out[c] = smart_truncate(example[c], self.estimator.chars_for(alloc[c]), self._cfg(c).truncation)
        return out


class LengthManager:
    def __init__(self, config: LengthManagerConfig | None = None, tokenizer=None):
        self.config = config or LengthManagerConfig()
        self.estimator = TokenEstimator(tokenizer, self.config.chars_per_token)
        self._column_configs: dict[str, ColumnLengthConfig] = dict(self.config.per_column)

    @property
    def max_length(self) -> int:
        return self.config.max_total_length

    @property
    def padding_strategy(self) -> PaddingStrategy:
        return self.config.padding_strategy

    def get_column_config(self, column: str | None) -> ColumnLengthConfig:
        """The column's limits; defaults for a column that has none."""
        if column is None or column not in self._column_configs:
            return ColumnLengthConfig(column or "", truncation=self.config.truncation_strategy)
        return self._column_configs[column]

    def set_column_config(self, column: str, config: ColumnLengthConfig) -> None:
        self._column_configs[column] = config

    def preprocess_text(self, text: str, column: str | None = None, max_chars: int | None = None) -> str:
        """Truncate one field.  The limit is the first of: `max_chars`, the column's max_chars, the column's
        max_tokens in characters, the total length in characters."""
        if not text:
            return ""
        cc = self.get_column_config(column)
        if max_chars is None:
            max_chars = cc.max_chars if cc.max_chars is not None else self.estimator.tokens_to_chars(
                cc.max_tokens if cc.max_tokens is not None else self.config.max_total_length)
        return smart_truncate(text, max_chars, cc.truncation)

    def preprocess_example(self, example: Mapping[str, str], text_columns: Sequence[str] | None = None) -> dict[str, str]:
        """Per-column limits first, then priority trimming until the total fits.  `text_columns` restricts both steps
        to those columns (the others pass through untouched)."""
        if text_columns is not None:
            part = self.preprocess_example({k: example[k] for k in text_columns if k in example})
            return {**example, **part}
        out = dict(example)
        for name, cc in self._column_configs.items():
            if isinstance(out.get(name), str) and (cc.max_length is not None or cc.max_chars is not None):
                out[name] = self.preprocess_text(out[name], name)
        return self._priority_trim(out)

    def _priority_trim(self, example: dict) -> dict:
        budget = self.config.max_total_length - self.config.special_tokens_budget
        cols = [c for c, v in example.items() if isinstance(v, str)]
        total = sum(self.estimator.estimate(example[c]) for c in cols)
        if total <= budget or not cols:
            return example
        # trim the longest columns first
        for c in sorted(cols, key=lambda k: -self.estimator.estimate(example[k])):
            over = total - budget
            if over <= 0:
                break
            have = self.estimator.estimate(example[c])
            keep = max(have - over, have // 4)
            example[c] = smart_truncate(example[c], self.estimator.chars_for(keep), self.config.truncation_strategy)
            total -= have - self.estimator.estimate(example[c])
        return example

    def get_bucket(self, length: int) -> int:
        b = self.config.bucket_boundaries
        i = bisect.bisect_left(b, length)
        return b[i] if i < len(b) else self.config.max_total_length

    @staticmethod
    def _next_power_of_two(n: int) -> int:
        return 1 if n <= 1 else 1 << (n - 1).bit_length()

    @reference_kwargs(batch_lengths="lengths")
    def get_effective_max_length(self, lengths: Sequence[int]) -> int:
        """Padded length of a batch under the configured padding strategy."""
        longest = max(lengths) if lengths else 0
        cap = self.config.max_total_length
        s = PaddingStrategy(self.config.padding_strategy)
        if s == PaddingStrategy.MAX_LENGTH:
            n = cap
        elif s == PaddingStrategy.BUCKET:
            n = min(cap, self.get_bucket(longest))
        elif s == PaddingStrategy.POWER_OF_TWO:
            n = min(cap, self._next_power_of_two(longest))
        else:
            n = min(cap, longest)
        m = self.config.pad_to_multiple_of
        if m:
            n = min(max(cap, m), (n + m - 1) // m * m)
        return n


@reference_kwargs(label_pad_token_id="label_pad")
def create_dynamic_collate_fn(length_manager: LengthManager, pad_token_id: int = 0, label_pad: int = -100,
                              padding_side: str = "right", additional_pad_keys: Mapping[str, int] | None = None) -> Callable:
    """Collate that pads (or crops) every `*input_ids / *attention_mask / *labels` key to the batch's effective length;
    `additional_pad_keys` = {key: fill value} for other sequence-valued keys (e.g. token_type_ids)."""
    extra = dict(additional_pad_keys or {})

    def pad_value(key: str) -> int:
        if key in extra:
            return extra[key]
        if key.endswith("labels"):
            return label_pad
        if key.endswith("attention_mask"):
            return 0
        return pad_token_id

    def collate(batch: Sequence[Mapping[str, torch.Tensor]]):
        out = {}
        for key in batch[0]:
            vals = [torch.as_tensor(b[key]) for b in batch]
            if vals[0].dim() == 0:
                out[key] = torch.stack(vals)
                continue
            if key.endswith("attention_mask") or key.endswith("input_ids") or key.endswith("labels"):
                mk = key.replace("input_ids", "attention_mask").replace("labels", "attention_mask")
                real = [int(torch.as_tensor(b[mk]).sum()) if mk in b else len(torch.as_tensor(b[key])) for b in batch]
            else:
                real = [len(v) for v in vals]
            width = length_manager.get_effective_max_length(real)
            rows = []
            for v in vals:
                v = v[:width] if padding_side == "right" else v[-width:]
                if len(v) < width:
                    fill = torch.full((width - len(v),), pad_value(key), dtype=v.dtype)
                    v = torch.cat((v, fill)) if padding_side == "right" else torch.cat((fill, v))
                rows.append(v)
            out[key] = torch.stack(rows)
        return out

    return collate


def create_length_manager(max_total_length: int = 2048, padding_strategy="max_length", truncation_strategy="right",
                          per_column_limits: Mapping[str, int] | None = None, tokenizer=None, **kw) -> LengthManager:
    per = {k: ColumnLengthConfig(k, v, TruncationStrategy(truncation_strategy)) for k, v in (per_column_limits or {}).items()}
    cfg = LengthManagerConfig(max_total_length=max_total_length, padding_strategy=PaddingStrategy(padding_strategy),
                              truncation_strategy=TruncationStrategy(truncation_strategy), per_column=per, **kw)
    return LengthManager(cfg, tokenizer)


@reference_kwargs(distribution_mode="mode")
def create_content_distributor(mode="proportional", max_length: int = 2048, column_ratios: Mapping[str, float] | None = None,
                               label_columns: Sequence[str] = (), priorities: Mapping[str, int] | None = None,
                               special_tokens_budget: int = 10, tokenizer=None,
                               column_configs: Mapping[str, ColumnContentConfig] | None = None,
                               default_truncation: TruncationStrategy | str | None = None,
                               chars_per_token: float = CHARS_PER_TOKEN) -> TokenAwareContentDistributor:
    """`column_configs` ({name: ColumnContentConfig}) gives full per-column settings and wins over the short forms
    (ratios, label columns, priorities); `default_truncation` applies to columns built from the short forms.
    `create_content_distributor(max_length, distribution_mode, ...)` (the length first, as in
    data_pipeline/preprocessing/length_manager.py) is taken as well."""
    if isinstance(mode, int) and not isinstance(mode, bool):
        mode, max_length = (max_length if not isinstance(max_length, int) else "proportional"), mode
    names = set(column_ratios or {}) | set(label_columns) | set(priorities or {})
    trunc = TruncationStrategy(default_truncation) if default_truncation is not None else TruncationStrategy.SMART
    cols = {n: ColumnContentConfig(n, priority=(priorities or {}).get(n, 0), ratio=(column_ratios or {}).get(n),
                                   is_label=n in label_columns, truncation=trunc) for n in names}
    for n, c in (column_configs or {}).items():
        cols[n] = c if c.name == n else ColumnContentConfig(**{**c.__dict__, "name": n})
    mode = getattr(mode, "value", mode)
    return TokenAwareContentDistributor(ContentDistributionMode(mode), max_length, list(cols.values()),
                                        special_tokens_budget, tokenizer, chars_per_token)


def saturating_sub(a: int, b: int) -> int:
    """a - b, never below zero."""
    return a - b if a > b else 0


def clamp(value: int, lo: int, hi: int) -> int:
    return lo if value < lo else hi if value > hi else value


class TokenizerProtocol:
    """What token estimation needs of a tokenizer: `encode(text, add_special_tokens=False) -> list[int]`
    (structural: any object with that method qualifies, see `is_tokenizer`)."""

    def encode(self, text: str, *, add_special_tokens: bool = False) -> list:
        raise NotImplementedError


def is_tokenizer(obj) -> bool:
    return callable(getattr(obj, "encode", None))
