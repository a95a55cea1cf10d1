"""Data half of the unified YAML file: enums, frozen dataclasses and `load_config -> Result[PipelineConfig]`.

Keys follow data_pipeline/core/config_schema.py:52-805 (`type: data_module`, `version`, `dataset{name, config_name,
streaming, revision, splits|stages, column_mapping, columns}`, `tokenizer{...}`, `prompt_engine{...}`,
`prompt_template{...}`, `output_schema{...}`, `dataloader{...}`; required keys type/version/dataset/tokenizer).
Unlike the reference, the `prompt_engine` sub-sections (fim / packing / span_corruption / multi_turn / rl) and the
`preprocessing{length_manager, content_distribution, packing}` block ARE parsed, and the packing / FIM fields that
the reference's processors read but its schema never defined exist here.  Training-half keys are ignored.
"""
from __future__ import annotations

import dataclasses
import os
import re
from dataclasses import dataclass, field
from enum import Enum
from pathlib import Path
from typing import Any, Dict, List, Mapping, Optional, Tuple

import yaml

from ..utils.refargs import ANY, reference_kwargs

from ..core.errors import ConfigurationError, SchemaValidationError, YAMLParseError
from ..core.types import Err, Ok, Result


class TrainingStage(str, Enum):
    PRE_TRAINING = "pre_training"
    FINE_TUNING = "fine_tuning"
    POST_TRAINING = "post_training"


class PreTrainingFormat(str, Enum):
    CAUSAL_LM = "causal_lm"
    FILL_IN_MIDDLE = "fill_in_middle"
    SPAN_CORRUPTION = "span_corruption"


class FineTuningFormat(str, Enum):
    CHAT = "chat"
    COMPLETION = "completion"
    INSTRUCTION = "instruction"
    MULTI_TURN = "multi_turn"
    CUSTOM = "custom"


class RLAlgorithm(str, Enum):
    DPO = "dpo"
    PPO = "ppo"
    KTO = "kto"
    ORPO = "orpo"
    GRPO = "grpo"
    REWARD_MODEL = "reward_model"


class FIMMode(str, Enum):
    PSM = "psm"
    SPM = "spm"


class PackingStrategy(str, Enum):
    GREEDY = "greedy"
    FFD = "ffd"
    SINGLE = "single"


class TruncationStrategy(str, Enum):
    RIGHT = "right"
    LEFT = "left"
    MIDDLE = "middle"
    SMART = "smart"
    NONE = "none"


class ContentDistributionMode(str, Enum):
    EQUAL = "equal"
    RATIO = "ratio"
    PROPORTIONAL = "proportional"
    PRIORITY = "priority"
    ADAPTIVE = "adaptive"


class PaddingStrategy(str, Enum):
    DO_NOT_PAD = "do_not_pad"
    LONGEST = "longest"
    MAX_LENGTH = "max_length"
    BUCKET = "bucket"
    POWER_OF_TWO = "power_of_two"


@dataclass(frozen=True)
class SplitSpec:
    name: str
    alias: Optional[str] = None
    sample_size: Optional[int] = None
    shuffle: bool = False
    seed: int = 42


@dataclass(frozen=True)
class StageConfig:
    name: str
    splits: Mapping[str, SplitSpec] = field(default_factory=dict)
    weight: float = 1.0

    def get_split(self, name: str) -> Optional[SplitSpec]:
        return self.splits.get(name)

    def all_splits(self) -> Dict[str, SplitSpec]:
        """train / test / eval first (when present), then the other splits in their declared order."""
        head = {k: self.splits[k] for k in ("train", "test", "eval") if k in self.splits}
        return {**head, **{k: v for k, v in self.splits.items() if k not in head}}

    @property
    def train(self) -> Optional[SplitSpec]:
        return self.splits.get("train")

    @property
    def test(self) -> Optional[SplitSpec]:
        return self.splits.get("test")

    @property
    def eval(self) -> Optional[SplitSpec]:
        return self.splits.get("eval")


@dataclass(frozen=True)
class DatasetConfig:
    name: str
    config_name: Optional[str] = None
    streaming: bool = False
    revision: Optional[str] = None
    splits: Mapping[str, SplitSpec] = field(default_factory=dict)
    stages: Mapping[str, StageConfig] = field(default_factory=dict)
    column_mapping: Mapping[str, str] = field(default_factory=dict)
    columns: Tuple[str, ...] = ()
    data_files: Optional[Any] = None
    path: Optional[str] = None          # local json/jsonl/parquet/csv/txt file or directory

    def is_staged(self) -> bool:
        """True when the dataset is configured as named stages (curriculum) rather than one set of splits."""
        return bool(self.stages)

    def get_split_spec(self, split_name: str, stage_name: Optional[str] = None) -> Optional[SplitSpec]:
        if stage_name is not None:
            stage = self.stages.get(stage_name)
            return stage.get_split(split_name) if stage is not None else None
        return self.splits.get(split_name)


@dataclass(frozen=True)
class TokenizerConfig:
    name_or_path: str
    max_length: int = 2048
    padding: str = "max_length"
    truncation: bool = True
    padding_side: str = "right"
    truncation_side: str = "right"
    special_tokens: Mapping[str, Any] = field(default_factory=dict)
    add_special_tokens: bool = True
    use_fast: bool = True


@dataclass(frozen=True)
class PromptTemplate:
    format_type: str = "custom"
    template: Optional[str] = None
    system_message: Optional[str] = None
    user_template: Optional[str] = None
    assistant_template: Optional[str] = None
    input_columns: Tuple[str, ...] = ()
    label_column: Optional[str] = None
    mask_input: bool = True
    add_bos: bool = False
    add_eos: bool = True

    def get_required_columns(self) -> List[str]:
        """Input columns plus the label column, each once, in that order."""
        cols = list(self.input_columns)
        if self.label_column and self.label_column not in cols:
            cols.append(self.label_column)
        return cols


@dataclass(frozen=True)
class FIMConfig:
    enabled: bool = False
    fim_rate: float = 0.5
    mode: FIMMode = FIMMode.PSM
    spm_rate: float = 0.0
    max_middle_ratio: float = 0.5
    prefix_token: str = "<fim_prefix>"
    suffix_token: str = "<fim_suffix>"
    middle_token: str = "<fim_middle>"
    seed: int = 0


@dataclass(frozen=True)
class PackingConfig:
    enabled: bool = False
    strategy: PackingStrategy = PackingStrategy.GREEDY
    max_packed_length: Optional[int] = None
    separator_tokens: Tuple[int, ...] = ()
    add_eos_separator: bool = True
    drop_remainder: bool = False
    min_fill_ratio: float = 0.0
    use_vsl: bool = True                 # emit cu_seqlens for the variable-length attention kernel
    max_sequences_per_pack: int = 0
    add_position_ids: bool = True


@dataclass(frozen=True)
class SpanCorruptionConfig:
    enabled: bool = False
    noise_density: float = 0.15
    mean_span_len: float = 3.0
    num_sentinels: int = 100
    sentinel_start: Optional[int] = None   # first sentinel id; default = vocab_size - 1 counting down
    seed: int = 0


@dataclass(frozen=True)
class PreTrainingConfig:
    format: PreTrainingFormat = PreTrainingFormat.CAUSAL_LM
    text_column: str = "text"
    fim: FIMConfig = field(default_factory=FIMConfig)
    packing: PackingConfig = field(default_factory=PackingConfig)
    span_corruption: SpanCorruptionConfig = field(default_factory=SpanCorruptionConfig)
    add_bos: bool = False
    add_eos: bool = True


@dataclass(frozen=True)
class MultiTurnConfig:
    messages_column: str = "messages"
    role_key: str = "role"
    content_key: str = "content"
    train_on_roles: Tuple[str, ...] = ("assistant",)
    system_message: Optional[str] = None


@dataclass(frozen=True)
class FineTuningConfig:
    format: FineTuningFormat = FineTuningFormat.CUSTOM
    instruction_column: str = "instruction"
    input_column: str = "input"
    output_column: str = "output"
    prompt_column: str = "prompt"
    completion_column: str = "completion"
    mask_prompt: bool = True
    multi_turn: MultiTurnConfig = field(default_factory=MultiTurnConfig)


@dataclass(frozen=True)
class RLColumnMapping:
    prompt: str = "prompt"
    chosen: str = "chosen"
    rejected: str = "rejected"
    response: str = "response"
    responses: str = "responses"
    label: str = "label"
    reward: str = "reward"
    scores: str = "scores"


@dataclass(frozen=True)
class RLConfig:
    algorithm: RLAlgorithm = RLAlgorithm.DPO
    columns: RLColumnMapping = field(default_factory=RLColumnMapping)
    max_prompt_length: Optional[int] = None
    max_response_length: Optional[int] = None
    num_generations: int = 4
    desirable_weight: float = 1.0
    undesirable_weight: float = 1.0


@dataclass(frozen=True)
class PromptEngineConfig:
    stage: TrainingStage = TrainingStage.FINE_TUNING
    max_length: int = 2048
    column_mapping: Mapping[str, str] = field(default_factory=dict)
    per_column_limits: Mapping[str, int] = field(default_factory=dict)
    truncation_strategy: TruncationStrategy = TruncationStrategy.RIGHT
    pre_training: PreTrainingConfig = field(default_factory=PreTrainingConfig)
    fine_tuning: FineTuningConfig = field(default_factory=FineTuningConfig)
    rl: RLConfig = field(default_factory=RLConfig)
    pad_to_max_length: bool = True


@dataclass(frozen=True)
class TensorSpec:
    dtype: str = "long"
    pad_value: int = 0
    requires_grad: bool = False


@dataclass(frozen=True)
class OutputSchema:
    tensors: Mapping[str, TensorSpec] = field(default_factory=lambda: {
        "input_ids": TensorSpec("long", 0), "attention_mask": TensorSpec("long", 0), "labels": TensorSpec("long", -100)})


@dataclass(frozen=True)
class DataLoaderConfig:
    batch_size: int = 8
    num_workers: int = 0
    pin_memory: bool = True
    drop_last: bool = False
    shuffle: bool = True
    prefetch_factor: Optional[int] = None
    persistent_workers: bool = False
    seed: int = 42


@dataclass(frozen=True)
class LengthManagerSection:
    enabled: bool = False
    max_total_length: Optional[int] = None
    padding_strategy: PaddingStrategy = PaddingStrategy.MAX_LENGTH
    truncation_strategy: TruncationStrategy = TruncationStrategy.RIGHT
    per_column_limits: Mapping[str, int] = field(default_factory=dict)


@dataclass(frozen=True)
class ContentDistributionSection:
    enabled: bool = False
    mode: ContentDistributionMode = ContentDistributionMode.PROPORTIONAL
    column_ratios: Mapping[str, float] = field(default_factory=dict)
    special_tokens_budget: int = 10


@dataclass(frozen=True)
class PreprocessingConfig:
    length_manager: LengthManagerSection = field(default_factory=LengthManagerSection)
    content_distribution: ContentDistributionSection = field(default_factory=ContentDistributionSection)
    packing: PackingConfig = field(default_factory=PackingConfig)


@dataclass(frozen=True)
class PipelineConfig:
    type: str
    version: str
    dataset: DatasetConfig
    tokenizer: TokenizerConfig
    prompt: PromptTemplate = field(default_factory=PromptTemplate)
    prompt_engine: Optional[PromptEngineConfig] = None
    output_schema: OutputSchema = field(default_factory=OutputSchema)
    dataloader: DataLoaderConfig = field(default_factory=DataLoaderConfig)
    preprocessing: PreprocessingConfig = field(default_factory=PreprocessingConfig)
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    def __post_init__(self):
        if self.type != "data_module":
            raise SchemaValidationError(f"type must be 'data_module', got {self.type!r}")


_ENV = re.compile(r"\$\{([A-Za-z_][A-Za-z0-9_]*)(?::-([^}]*))?\}")


@reference_kwargs(value="obj")
def interpolate_env_vars(obj):
    """${VAR} / ${VAR:-default} interpolation inside strings (data_pipeline/trainer/core/config.py:54)."""
    if isinstance(obj, str):
        return _ENV.sub(lambda m: os.environ.get(m.group(1), m.group(2) if m.group(2) is not None else m.group(0)), obj)
    if isinstance(obj, dict):
        return {k: interpolate_env_vars(v) for k, v in obj.items()}
    if isinstance(obj, list):
        return [interpolate_env_vars(v) for v in obj]
    return obj


def _build(cls, d: Optional[Mapping[str, Any]], where: str, lenient: bool = True):
    """Dataclass from a mapping with enum / nested / tuple coercion. Unknown keys are ignored when `lenient`
    (the shared `tokenizer` section carries the other half's keys), else rejected."""
    if d is None:
        return cls()
    if not isinstance(d, Mapping):
        raise SchemaValidationError(f"{where} must be a mapping", got=type(d).__name__)
    fields = {f.name: f for f in dataclasses.fields(cls)}
    kw = {}
    for k, v in d.items():
        if k not in fields:
            if lenient:
                continue
            raise SchemaValidationError(f"unknown key {k!r} in {where}")
        f = fields[k]
        default = f.default if f.default is not dataclasses.MISSING else (
            f.default_factory() if f.default_factory is not dataclasses.MISSING else None)
        try:
            if isinstance(default, Enum) and v is not None:
                v = type(default)(v)
            elif dataclasses.is_dataclass(default) and isinstance(v, Mapping):
                v = _build(type(default), v, f"{where}.{k}", lenient)
            elif isinstance(default, tuple) and isinstance(v, (list, tuple)):
                v = tuple(v)
        except ValueError as e:
            raise SchemaValidationError(f"invalid value for {where}.{k}: {v!r}", cause=e)
        kw[k] = v
    try:
        return cls(**kw)
    except TypeError as e:
        raise SchemaValidationError(f"invalid {where} section", cause=e)


def _parse_split(name: str, v) -> SplitSpec:
    if isinstance(v, str):
        return SplitSpec(name=v, alias=name)
    v = dict(v or {})
    v.setdefault("name", name)
    v.setdefault("alias", name)
    return _build(SplitSpec, v, f"dataset.splits.{name}")


def _parse_dataset(d: Mapping[str, Any]) -> DatasetConfig:
    if "name" not in d and "path" not in d:
        raise SchemaValidationError("dataset.name (or dataset.path) is required")
    splits = {k: _parse_split(k, v) for k, v in (d.get("splits") or {}).items()}
    stages = {}
    for sname, sv in (d.get("stages") or {}).items():
        sv = sv or {}
        stages[sname] = StageConfig(name=sname, weight=float(sv.get("weight", 1.0)),
                                    splits={k: _parse_split(k, v) for k, v in (sv.get("splits") or {}).items()})
    rest = {k: v for k, v in d.items() if k not in ("splits", "stages")}
    rest.setdefault("name", d.get("path", ""))
    if "columns" in rest and rest["columns"] is not None:
        rest["columns"] = tuple(rest["columns"])
    base = _build(DatasetConfig, rest, "dataset")
    return dataclasses.replace(base, splits=splits, stages=stages)


def _parse_output_schema(d) -> OutputSchema:
    if not d:
        return OutputSchema()
    return OutputSchema({k: _build(TensorSpec, v or {}, f"output_schema.{k}") for k, v in d.items()})


def parse_config(raw: Mapping[str, Any]) -> PipelineConfig:
    raw = interpolate_env_vars(dict(raw or {}))
    missing = [k for k in ("type", "version", "dataset", "tokenizer") if k not in raw]
    if missing:
        raise SchemaValidationError(f"missing required keys: {missing}")
    tok = dict(raw["tokenizer"] or {})
    if not tok.get("name_or_path"):
        raise SchemaValidationError("tokenizer.name_or_path is required")
    pe = raw.get("prompt_engine")
    return PipelineConfig(
        type=str(raw["type"]), version=str(raw["version"]), dataset=_parse_dataset(raw["dataset"] or {}),
        tokenizer=_build(TokenizerConfig, tok, "tokenizer"),
        prompt=_build(PromptTemplate, raw.get("prompt_template") or raw.get("prompt"), "prompt_template"),
        prompt_engine=_build(PromptEngineConfig, pe, "prompt_engine") if pe is not None else None,
        output_schema=_parse_output_schema(raw.get("output_schema")),
        dataloader=_build(DataLoaderConfig, raw.get("dataloader"), "dataloader"),
        preprocessing=_build(PreprocessingConfig, raw.get("preprocessing"), "preprocessing"), raw=raw)


def load_config(path) -> Result:
    """YAML file -> Ok(PipelineConfig) | Err(ConfigurationError)."""
    p = Path(path)
    if not p.exists():
        return Err(ConfigurationError(f"config file not found: {p}"))
    try:
        raw = yaml.safe_load(p.read_text())
    except yaml.YAMLError as e:
        return Err(YAMLParseError(f"cannot parse {p}", cause=e))
    if not isinstance(raw, dict):
        return Err(SchemaValidationError("top level of the config must be a mapping"))
    try:
        return Ok(parse_config(raw))
    except ConfigurationError as e:
        return Err(e)


def load_config_dict(raw: Mapping[str, Any]) -> Result:
    try:
        return Ok(parse_config(raw))
    except ConfigurationError as e:
        return Err(e)


# ---- value sets of the schema, by the names of data_pipeline/core/config_schema.py
PADDING_STRATEGIES = frozenset({"max_length", "longest", "do_not_pad"})
PROMPT_FORMAT_TYPES = frozenset({"chat", "completion", "custom"})
TENSOR_DTYPES = frozenset({"long", "int", "float", "half", "bfloat16", "bool"})
