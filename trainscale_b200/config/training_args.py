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
from pydantic import BaseModel, Field, field_validator

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


def merge_configs(base: Dict[str, Any], override: Dict[str, Any]) -> Dict[str, Any]:
    out = copy.deepcopy(base)
    for k, v in (override or {}).items():
        if isinstance(v, dict) and isinstance(out.get(k), dict):
            out[k] = merge_configs(out[k], v)
        else:
            out[k] = copy.deepcopy(v)
    return out


def load_training_config(path, overrides: Dict[str, Any] | None = None) -> TrainingArguments:
    raw = yaml.safe_load(Path(path).read_text()) or {}
    raw = interpolate_env_vars(raw.get("training_arguments", raw))
    return TrainingArguments(**merge_configs(raw, overrides or {}))


@dataclass
class TrainingConfig:
    model_name: str = ""
    output_dir: str = "./outputs"
    learning_rate: float = 2e-5
    batch_size: int = 4
    gradient_accumulation_steps: int = 4
    num_epochs: int = 3
    max_seq_length: int = 4096
    warmup_ratio: float = 0.1
    weight_decay: float = 0.01
    use_lora: bool = False
    lora_r: int = 16
    precision: str = "bf16"
    strategy: str = "ddp"
    gradient_checkpointing: bool = True

    def to_sota_dict(self) -> Dict[str, Any]:
        return {"training_mode": "lora" if self.use_lora else "full", "model": {"name_or_path": self.model_name},
                "lora": {"enabled": self.use_lora, "r": self.lora_r},
                "optimizer": {"learning_rate": self.learning_rate, "weight_decay": self.weight_decay},
                "scheduler": {"warmup_ratio": self.warmup_ratio},
                "distributed": {"strategy": self.strategy, "gradient_checkpointing": self.gradient_checkpointing},
                "hardware": {"precision": self.precision}, "data": {"max_seq_length": self.max_seq_length},
                "training": {"output_dir": self.output_dir, "num_train_epochs": self.num_epochs,
                             "per_device_train_batch_size": self.batch_size,
                             "gradient_accumulation_steps": self.gradient_accumulation_steps}}


def get_quick_test_config() -> TrainingConfig:
    return TrainingConfig(batch_size=2, gradient_accumulation_steps=1, num_epochs=1, max_seq_length=256)


def get_memory_efficient_config() -> TrainingConfig:
    return TrainingConfig(use_lora=True, batch_size=1, gradient_accumulation_steps=16, strategy="fsdp2")


def get_high_throughput_config() -> TrainingConfig:
    return TrainingConfig(batch_size=8, gradient_accumulation_steps=1, strategy="fsdp2", gradient_checkpointing=False)


def get_qlora_config(model_name: str, r: int = 16, max_seq_length: int = 2048) -> TrainingConfig:
    """Adapters of rank r (alpha 2r) on a quantised base, packed sequences
    (data_pipeline/trainer/training_config.py:230)."""
    c = TrainingConfig(model_name=model_name, use_lora=True, lora_r=r, max_seq_length=max_seq_length,
                       learning_rate=2e-4, strategy="ddp")
    c.load_in_4bit, c.lora_alpha, c.pack_sequences = True, 2 * r, True
    return c


def get_full_finetune_config(model_name: str, max_seq_length: int = 2048) -> TrainingConfig:
    c = TrainingConfig(model_name=model_name, use_lora=False, max_seq_length=max_seq_length, learning_rate=1e-5,
                       precision="bf16", strategy="fsdp2", gradient_checkpointing=True)
    c.load_in_4bit, c.pack_sequences = False, False
    return c


def get_pretraining_config(model_name: str, max_seq_length: int = 4096) -> TrainingConfig:
    c = TrainingConfig(model_name=model_name, use_lora=False, max_seq_length=max_seq_length, learning_rate=3e-4,
                       warmup_ratio=0.01, precision="bf16", strategy="fsdp2", gradient_checkpointing=True)
    c.load_in_4bit, c.pack_sequences = False, True
    return c


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
