"""Legacy argument objects: pydantic `TrainingArguments` with `${ENV}` interpolation, `load_training_config`,
`merge_configs`, and the plain-dataclass `TrainingConfig` with presets.

After data_pipeline/trainer/core/config.py:54-539, data_pipeline/trainer/core/types.py:88-920 (ParallelMode, ZeROStage,
CheckpointConfig, LoggingConfig, frozen TrainingState, TrainerEvent) and data_pipeline/trainer/training_config.py:30-292.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field, replace
from enum import Enum
from pathlib import Path
from typing import Any, Dict, List, Optional

import yaml
from pydantic import BaseModel, Field, field_validator, model_validator

from ..utils.refargs import ANY, reference_kwargs
from .data_schema import interpolate_env_vars


class ParallelMode(str, Enum):
    NONE = "none"
    DDP = "ddp"
    FSDP = "fsdp"
    TENSOR = "tensor"
    PIPELINE = "pipeline"
    CONTEXT = "context"
    EXPERT = "expert"
    HYBRID = "hybrid"


class ZeROStage(int, Enum):
    DISABLED = 0
    OPTIMIZER = 1
    GRADIENTS = 2
    PARAMETERS = 3


class TrainerEvent(str, Enum):
    INIT_END = "on_init_end"
    TRAIN_BEGIN = "on_train_begin"
    TRAIN_END = "on_train_end"
    EPOCH_BEGIN = "on_epoch_begin"
    EPOCH_END = "on_epoch_end"
    STEP_BEGIN = "on_step_begin"
    STEP_END = "on_step_end"
    EVALUATE = "on_evaluate"
    SAVE = "on_save"
    LOG = "on_log"
    PREDICTION_STEP = "on_prediction_step"


class CheckpointConfig(BaseModel):
    save_strategy: str = "steps"
    save_steps: int = 500
    save_total_limit: Optional[int] = 3
    save_safetensors: bool = True
    load_best_model_at_end: bool = False
    metric_for_best_model: str = "eval_loss"
    greater_is_better: bool = False


class LoggingConfig(BaseModel):
    logging_steps: int = 10
    logging_first_step: bool = True
    report_to: List[str] = Field(default_factory=lambda: ["console"])
    logging_dir: Optional[str] = None


class TrainingArguments(BaseModel):
    output_dir: str = "./outputs"
    num_train_epochs: float = 3.0
    max_steps: int = -1
    per_device_train_batch_size: int = 8
    per_device_eval_batch_size: int = 8
    gradient_accumulation_steps: int = 1
    learning_rate: float = 5e-5
    weight_decay: float = 0.0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_epsilon: float = 1e-8
    max_grad_norm: float = 1.0
    lr_scheduler_type: str = "linear"
    warmup_steps: int = 0
    warmup_ratio: float = 0.0
    optim: str = "adamw"
    bf16: bool = True
    fp16: bool = False
    seed: int = 42
    parallel_mode: ParallelMode = ParallelMode.NONE
    zero_stage: ZeROStage = ZeROStage.DISABLED
    gradient_checkpointing: bool = False
    eval_strategy: str = "no"
    eval_steps: Optional[int] = None
    detect_anomaly: bool = False
    dataloader_num_workers: int = 0
    dataloader_pin_memory: bool = True
    dataloader_drop_last: bool = False
    world_size: int = 1
    overwrite_output_dir: bool = False
    push_to_hub: bool = False
    hub_model_id: Optional[str] = None
    checkpoint: CheckpointConfig = Field(default_factory=CheckpointConfig)
    logging: LoggingConfig = Field(default_factory=LoggingConfig)

    @field_validator("learning_rate")
    @classmethod
    def _lr_positive(cls, v):
        if v <= 0:
            raise ValueError("learning_rate must be positive")
        return v

    @field_validator("gradient_accumulation_steps", "per_device_train_batch_size")
    @classmethod
    def _at_least_one(cls, v):
        if v < 1:
            raise ValueError("must be >= 1")
        return v

    @property
    def effective_batch_size(self) -> int:
        """per-device batch x accumulation steps x world size (data_pipeline/trainer/core/config.py:312-323)."""
        return self.per_device_train_batch_size * self.gradient_accumulation_steps * max(1, self.world_size)

    @property
    def per_device_batch_size(self) -> int:
        return self.per_device_train_batch_size

    @property
    def output_path(self) -> Path:
        return Path(self.output_dir)

    @model_validator(mode="after")
    def validate_arguments(self) -> "TrainingArguments":
        """Cross-field checks: a hub upload needs its repository name; bf16 and fp16 exclude each other."""
        if self.push_to_hub and not self.hub_model_id:
            raise ValueError("hub_model_id is required when push_to_hub=True")
        if self.bf16 and self.fp16:
            raise ValueError("bf16 and fp16 are mutually exclusive")
        return self

    def to_sota_dict(self) -> Dict[str, Any]:
        """The same settings expressed in the SOTAConfig key schema."""
        strat = {ParallelMode.DDP: "ddp", ParallelMode.FSDP: "fsdp2", ParallelMode.PIPELINE: "pipeline",
                 ParallelMode.CONTEXT: "context_parallel", ParallelMode.TENSOR: "tp"}.get(self.parallel_mode, "ddp")
        if self.zero_stage in (ZeROStage.GRADIENTS, ZeROStage.PARAMETERS):
            strat = "fsdp2"
        return {"optimizer": {"type": "adamw" if self.optim.startswith("adam") else self.optim,
                              "learning_rate": self.learning_rate, "weight_decay": self.weight_decay,
                              "betas": [self.adam_beta1, self.adam_beta2], "eps": self.adam_epsilon,
                              "max_grad_norm": self.max_grad_norm},
                "scheduler": {"type": self.lr_scheduler_type, "warmup_steps": self.warmup_steps, "warmup_ratio": self.warmup_ratio},
                "distributed": {"enabled": self.parallel_mode != ParallelMode.NONE, "strategy": strat,
                                "gradient_checkpointing": self.gradient_checkpointing},
                "hardware": {"precision": "bf16" if self.bf16 else ("fp16" if self.fp16 else "fp32")},
                "training": {"output_dir": self.output_dir, "num_train_epochs": int(self.num_train_epochs),
                             "max_steps": self.max_steps, "per_device_train_batch_size": self.per_device_train_batch_size,
                             "per_device_eval_batch_size": self.per_device_eval_batch_size,
                             "gradient_accumulation_steps": self.gradient_accumulation_steps, "seed": self.seed,
                             "eval_strategy": self.eval_strategy, "eval_steps": self.eval_steps or 100,
                             "save_strategy": self.checkpoint.save_strategy, "save_steps": self.checkpoint.save_steps,
                             "save_total_limit": self.checkpoint.save_total_limit or 0,
                             "logging_steps": self.logging.logging_steps}}


@reference_kwargs(overrides="override")
def merge_configs(base: Dict[str, Any], override: Dict[str, Any]) -> Dict[str, Any]:
    out = copy.deepcopy(base)
    for k, v in (override or {}).items():
        if isinstance(v, dict) and isinstance(out.get(k), dict):
            out[k] = merge_configs(out[k], v)
        else:
            out[k] = copy.deepcopy(v)
    return out


@reference_kwargs(yaml_path="path")
def load_training_config(path, overrides: Dict[str, Any] | None = None, config_key: str = "training_arguments",
                         interpolate_env: bool = True) -> TrainingArguments:
    """`TrainingArguments` from the `config_key` section of a YAML file (the whole file when it has no such section),
    with ${VAR} / ${VAR:-default} interpolation unless `interpolate_env=False`."""
    raw = yaml.safe_load(Path(path).read_text()) or {}
    raw = raw.get(config_key, raw) if config_key else raw
    if interpolate_env:
        raw = interpolate_env_vars(raw)
    return TrainingArguments(**merge_configs(raw, overrides or {}))


class TrainingMode(str, Enum):
    """What is trained (data_pipeline/trainer/training_config.py)."""
    FULL_FINETUNE = "full"
    LORA = "lora"
    QLORA = "qlora"
    PRETRAINING = "pretrain"
    RL = "rl"


@dataclass
class TrainingConfig:
    """Flat, script-friendly training configuration with the reference's field names
    (data_pipeline/trainer/training_config.py:40-224) plus the short spellings this framework's presets use
    (`model_name`, `batch_size`, `num_epochs`, `use_lora`, `precision`, `strategy`), which are kept in step with their
    long forms.  `to_sota_dict()` turns it into the nested dictionary `SOTAConfig.from_dict` reads."""
    output_dir: str = "./outputs"
    model_name_or_path: str = ""
    training_mode: TrainingMode | None = None
    num_train_epochs: int = 3
    max_steps: int = -1
    per_device_train_batch_size: int = 4
    per_device_eval_batch_size: int = 4
    gradient_accumulation_steps: int = 4
    learning_rate: float = 2e-5
    weight_decay: float = 0.01
    warmup_ratio: float = 0.1
    warmup_steps: int = 0
    max_seq_length: int = 4096
    load_in_4bit: bool = False
    load_in_8bit: bool = False
    load_in_fp8: bool = False
    bnb_4bit_quant_type: str = "nf4"
    bnb_4bit_compute_dtype: str = "bfloat16"
    bnb_4bit_use_double_quant: bool = True
    lora_r: int = 16
    lora_alpha: int = 32
    lora_dropout: float = 0.0
    lora_target_modules: list = field(default_factory=lambda: ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj",
                                                               "up_proj", "down_proj"])
    use_rslora: bool = False
    use_dora: bool = False
    pack_sequences: bool = False
    padding_free: bool = True
    fp16: bool = False
    bf16: bool = True
    tf32: bool = True
    gradient_checkpointing: bool = True
    use_flash_attention: bool = True
    use_triton_kernels: bool = False
    optim: str = "adamw"
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_epsilon: float = 1e-8
    max_grad_norm: float = 1.0
    lr_scheduler_type: str = "cosine"
    logging_steps: int = 10
    save_steps: int = 500
    eval_steps: int = 500
    save_total_limit: int = 3
    report_to: str = "tensorboard"
    push_to_hub: bool = False
    hub_model_id: str | None = None
    distributed_strategy: str = "ddp"
    num_pipeline_stages: int = 4
    num_microbatches: int = 8
    pipeline_memory_limit_gb: float = 4.0
    seed: int = 42
    data_seed: int = 42
    # short spellings (None = take the long form)
    model_name: str | None = None
    batch_size: int | None = None
    num_epochs: int | None = None
    use_lora: bool | None = None
    precision: str | None = None
    strategy: str | None = None

    def __post_init__(self):
        if isinstance(self.training_mode, str):
            self.training_mode = TrainingMode(self.training_mode)
        if self.model_name is not None:
            self.model_name_or_path = self.model_name
        if self.batch_size is not None:
            self.per_device_train_batch_size = self.batch_size
        if self.num_epochs is not None:
            self.num_train_epochs = self.num_epochs
        if self.strategy is not None:
            self.distributed_strategy = self.strategy
        if self.precision is not None:
            self.bf16, self.fp16 = self.precision == "bf16", self.precision == "fp16"
            self.load_in_fp8 = self.load_in_fp8 or self.precision.startswith("fp8")
        if self.training_mode is None:
            self.training_mode = (TrainingMode.QLORA if self.load_in_4bit else TrainingMode.LORA) if self.use_lora \
                else TrainingMode.FULL_FINETUNE
        if self.use_lora is None:
            self.use_lora = self.training_mode in (TrainingMode.LORA, TrainingMode.QLORA)
        if self.training_mode is TrainingMode.QLORA:
            self.load_in_4bit = True
        elif self.training_mode is TrainingMode.FULL_FINETUNE:
            self.load_in_4bit = self.load_in_8bit = False
        elif self.training_mode is TrainingMode.PRETRAINING:
            self.pack_sequences = self.gradient_checkpointing = True
        self.model_name, self.batch_size = self.model_name_or_path, self.per_device_train_batch_size
        self.num_epochs, self.strategy = self.num_train_epochs, self.distributed_strategy
        self.precision = self.precision or ("bf16" if self.bf16 else "fp16" if self.fp16 else "fp32")

    @property
    def compute_dtype(self) -> "torch.dtype":
        import torch
        return {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}.get(
            self.bnb_4bit_compute_dtype, torch.bfloat16)

    @property
    def effective_batch_size(self) -> int:
        return self.per_device_train_batch_size * self.gradient_accumulation_steps

    def to_lora_config(self):
        from ..lora import LoraConfig
        return LoraConfig(r=self.lora_r, lora_alpha=self.lora_alpha, lora_dropout=self.lora_dropout,
                          target_modules=list(self.lora_target_modules), use_rslora=self.use_rslora,
                          use_dora=self.use_dora)

    def to_quant_config(self):
        from ..quantization import QuantizationConfig
        return QuantizationConfig(load_in_4bit=self.load_in_4bit, load_in_8bit=self.load_in_8bit,
                                  load_in_fp8=self.load_in_fp8, bnb_4bit_quant_type=self.bnb_4bit_quant_type,
                                  bnb_4bit_compute_dtype=self.compute_dtype,
                                  bnb_4bit_use_double_quant=self.bnb_4bit_use_double_quant)

    def to_dict(self) -> Dict[str, Any]:
        return {k: (v.value if isinstance(v, Enum) else v) for k, v in self.__dict__.items()}

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "TrainingConfig":
        known = {f for f in cls.__dataclass_fields__}
        return cls(**{k: v for k, v in d.items() if k in known})

    def to_sota_dict(self) -> Dict[str, Any]:
        mode = {TrainingMode.FULL_FINETUNE: "full", TrainingMode.LORA: "lora", TrainingMode.QLORA: "qlora",
                TrainingMode.PRETRAINING: "pretrain", TrainingMode.RL: "rl"}[self.training_mode]
        return {"training_mode": mode, "model": {"name_or_path": self.model_name_or_path},
                "lora": {"enabled": bool(self.use_lora), "r": self.lora_r, "lora_alpha": self.lora_alpha,
                         "lora_dropout": self.lora_dropout, "target_modules": list(self.lora_target_modules),
                         "use_rslora": self.use_rslora},
                "optimizer": {"learning_rate": self.learning_rate, "weight_decay": self.weight_decay,
                              "max_grad_norm": self.max_grad_norm, "betas": [self.adam_beta1, self.adam_beta2],
                              "eps": self.adam_epsilon},
                "scheduler": {"type": self.lr_scheduler_type, "warmup_ratio": self.warmup_ratio,
                              "warmup_steps": self.warmup_steps},
                "distributed": {"strategy": self.distributed_strategy, "gradient_checkpointing": self.gradient_checkpointing},
                "hardware": {"precision": self.precision}, "data": {"max_seq_length": self.max_seq_length,
                                                                    "packing": self.pack_sequences},
                "training": {"output_dir": self.output_dir, "num_train_epochs": self.num_train_epochs,
                             "max_steps": self.max_steps,
                             "per_device_train_batch_size": self.per_device_train_batch_size,
                             "gradient_accumulation_steps": self.gradient_accumulation_steps,
                             "logging_steps": self.logging_steps, "save_steps": self.save_steps,
                             "save_total_limit": self.save_total_limit, "seed": self.seed}}


def get_quick_test_config() -> TrainingConfig:
    return TrainingConfig(batch_size=2, gradient_accumulation_steps=1, num_epochs=1, max_seq_length=256)


def get_memory_efficient_config() -> TrainingConfig:
    return TrainingConfig(use_lora=True, batch_size=1, gradient_accumulation_steps=16, strategy="fsdp2")


def get_high_throughput_config() -> TrainingConfig:
    return TrainingConfig(batch_size=8, gradient_accumulation_steps=1, strategy="fsdp2", gradient_checkpointing=False)


def get_qlora_config(model_name: str, r: int = 16, max_seq_length: int = 2048) -> TrainingConfig:
    """Adapters of rank r (alpha 2r) on a quantised base, packed sequences
    (data_pipeline/trainer/training_config.py:230)."""
    return TrainingConfig(model_name=model_name, training_mode=TrainingMode.QLORA, lora_r=r, lora_alpha=2 * r,
                          max_seq_length=max_seq_length, learning_rate=2e-4, strategy="ddp", pack_sequences=True)


def get_full_finetune_config(model_name: str, max_seq_length: int = 2048) -> TrainingConfig:
    return TrainingConfig(model_name=model_name, training_mode=TrainingMode.FULL_FINETUNE, max_seq_length=max_seq_length,
                          learning_rate=1e-5, precision="bf16", strategy="fsdp2", gradient_checkpointing=True)


def get_pretraining_config(model_name: str, max_seq_length: int = 4096) -> TrainingConfig:
    return TrainingConfig(model_name=model_name, training_mode=TrainingMode.PRETRAINING, max_seq_length=max_seq_length,
                          learning_rate=3e-4, warmup_ratio=0.01, precision="bf16", strategy="fsdp2")


def load_training_config_from_dict(config_dict: Dict[str, Any], *, interpolate_env: bool = True) -> TrainingArguments:
    """Validated `TrainingArguments` from a dictionary; `${VAR}` / `${VAR:default}` strings are replaced from the
    environment first.  Validation problems are raised as one ValueError that lists every offending field."""
    raw = interpolate_env_vars(config_dict) if interpolate_env else config_dict
    raw = raw.get("training_arguments", raw)
    try:
        return TrainingArguments(**raw)
    except Exception as e:    # noqa: BLE001 - pydantic's ValidationError, re-worded
        details = getattr(e, "errors", None)
        if callable(details):
            lines = [f"{'.'.join(str(p) for p in d.get('loc', ()))}: {d.get('msg')}" for d in details()]
            raise ValueError("invalid training configuration:\n  " + "\n  ".join(lines)) from e
        raise


import re as _re  # noqa: E402

ENV_VAR_PATTERN = _re.compile(r"\$\{([^}]+)\}")           # ${VAR} / ${VAR:-default}, what `interpolate_env_vars` replaces
