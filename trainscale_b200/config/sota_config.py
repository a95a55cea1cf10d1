"""SOTAConfig: the training half of the unified YAML file.

Key schema follows data_pipeline/trainer/core/sota_config.py:53-691 (sections model / tokenizer / lora /
quantization / optimizer / scheduler / loss / rl / export / distributed / hardware / kernels / data / training,
enum coercion, unknown keys inside a section raise TypeError, presets).  Additions the reference has no keys for:
`model.architecture` (build the framework's own decoder from a preset name or an inline shape, random-init) and
`distributed.parallel` (dp_replicate, dp_shard, cp, tp, pp, ep, etp, sp - names as in
data_pipeline/trainer/distributed/parallel_dims.py:1049-1057).
"""
from __future__ import annotations

import copy
import dataclasses
from dataclasses import dataclass, field
from enum import Enum
from pathlib import Path
from typing import Any, Dict, List, Optional, Union

import torch
import yaml

from ..utils.refargs import ANY, reference_kwargs


class TrainingMode(str, Enum):
    FULL_FINETUNE = "full"
    LORA = "lora"
    QLORA = "qlora"
    PRETRAIN = "pretrain"
    RL = "rl"
    DISTILL = "distill"


class Precision(str, Enum):
    FP32 = "fp32"
    FP16 = "fp16"
    BF16 = "bf16"
    FP8_E4M3 = "fp8_e4m3"
    FP8_E5M2 = "fp8_e5m2"
    INT8 = "int8"
    INT4 = "int4"


class RLAlgorithm(str, Enum):
    GRPO = "grpo"
    GSPO = "gspo"
    DRGRPO = "drgrpo"
    DAPO = "dapo"
    PPO = "ppo"
    DPO = "dpo"
    ORPO = "orpo"
    SIMPO = "simpo"
    KTO = "kto"


class ExportFormat(str, Enum):
    SAFETENSORS = "safetensors"
    PYTORCH = "pytorch"
    GGUF_Q4 = "gguf_q4_k_m"
    GGUF_Q5 = "gguf_q5_k_m"
    GGUF_Q8 = "gguf_q8_0"
    GGUF_F16 = "gguf_f16"
    VLLM = "vllm"
    SGLANG = "sglang"


class OptimizerType(str, Enum):
    ADAMW = "adamw"
    ADAM_8BIT = "adam8bit"
    LION = "lion"
    CAME = "came"
    SOPHIA = "sophia"
    PRODIGY = "prodigy"
    FUSED_ADAMW = "fused_adamw"
    LAMB = "lamb"
    ADAFACTOR = "adafactor"
    SCHEDULE_FREE = "schedule_free"
    MUON = "muon"
    ADOPT = "adopt"


class SchedulerType(str, Enum):
    COSINE = "cosine"
    WSD = "wsd"
    LINEAR = "linear"
    POLYNOMIAL = "polynomial"
    ONECYCLE = "onecycle"
    INVERSE_SQRT = "inverse_sqrt"
    COSINE_RESTART = "cosine_restart"
    REX = "rex"
    CONSTANT = "constant"


class LossType(str, Enum):
    CROSS_ENTROPY = "cross_entropy"
    CHUNKED_CE = "chunked_ce"
    FOCAL = "focal"
    DPO = "dpo"
    ORPO = "orpo"
    SIMPO = "simpo"
    KTO = "kto"
    CPO = "cpo"
    DISTILLATION = "distillation"
    CONTRASTIVE = "contrastive"


class DeviceType(str, Enum):
    AUTO = "auto"
    CUDA = "cuda"
    CPU = "cpu"


@dataclass
class ModelConfig:
    name_or_path: str = ""
    revision: str = "main"
    trust_remote_code: bool = False
    torch_dtype: str = "auto"
    low_cpu_mem_usage: bool = True
    use_flash_attention_2: bool = True
    attn_implementation: str = "flash_attention_2"
    max_position_embeddings: Optional[int] = None
    architecture: Union[str, Dict[str, Any], None] = None   # preset name or inline LlamaConfig fields


@dataclass
class TokenizerConfig:
    name_or_path: Optional[str] = None
    use_fast: bool = True
    padding_side: str = "right"
    truncation_side: str = "right"
    max_length: int = 4096
    add_bos_token: bool = False
    add_eos_token: bool = True
    add_pad_token: bool = True
    padding: Optional[str] = None
    truncation: Optional[bool] = None
    special_tokens: Optional[Dict[str, Any]] = None
    add_special_tokens: Optional[bool] = None


@dataclass
class LoRAConfig:
    enabled: bool = True
    r: int = 16
    lora_alpha: int = 32
    lora_dropout: float = 0.0
    target_modules: List[str] = field(default_factory=lambda: ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj",
                                                               "up_proj", "down_proj"])
    modules_to_save: List[str] = field(default_factory=lambda: ["embed_tokens", "lm_head"])
    bias: str = "none"
    use_rslora: bool = True
    use_dora: bool = False
    init_lora_weights: Union[bool, str] = True
    rank_pattern: Dict[str, int] = field(default_factory=dict)


@dataclass
class QuantizationConfig:
    enabled: bool = False
    load_in_4bit: bool = False
    load_in_8bit: bool = False
    load_in_fp8: bool = False
    bnb_4bit_quant_type: str = "nf4"
    bnb_4bit_compute_dtype: str = "bfloat16"
    bnb_4bit_use_double_quant: bool = True
    llm_int8_threshold: float = 6.0


@dataclass
class OptimizerConfig:
    type: OptimizerType = OptimizerType.ADAMW
    learning_rate: float = 2e-5
    weight_decay: float = 0.01
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8
    max_grad_norm: float = 1.0
    percentile_clipping: float = 100.0
    block_wise: bool = True
    lion_betas: tuple = (0.9, 0.99)


@dataclass
class SchedulerConfig:
    type: SchedulerType = SchedulerType.COSINE
    warmup_steps: int = 0
    warmup_ratio: float = 0.1
    min_lr_ratio: float = 0.1
    stable_ratio: float = 0.8
    decay_type: str = "cosine"
    power: float = 1.0
    max_lr_ratio: float = 10.0

    def compute_warmup_steps(self, num_training_steps: int) -> int:
        """Explicit `warmup_steps` when set, else `warmup_ratio` of the run (data_pipeline/trainer/core/types.py:517)."""
        if self.warmup_steps > 0:
            return self.warmup_steps
        return int(self.warmup_ratio * max(0, num_training_steps))


@dataclass
class LossConfig:
    type: LossType = LossType.CROSS_ENTROPY
    ignore_index: int = -100
    label_smoothing: float = 0.0
    reduction: str = "mean"
    chunk_size: int = 32768
    focal_gamma: float = 2.0
    focal_alpha: float = 0.25
    dpo_beta: float = 0.1
    dpo_variant: str = "sigmoid"
    simpo_gamma: float = 0.5
    reference_free: bool = False
    temperature: float = 2.0
    alpha: float = 0.5


@dataclass
class RLConfig:
    enabled: bool = False
    algorithm: RLAlgorithm = RLAlgorithm.GRPO
    num_generations: int = 4
    temperature: float = 0.7
    kl_coef: float = 0.01
    gamma: float = 1.0
    clip_range: float = 0.2
    reward_clip: Optional[float] = 10.0
    use_length_penalty: bool = False
    length_penalty_alpha: float = 1.0
    use_ref_model: bool = True
    ref_model_sync_steps: int = 100
    use_vllm: bool = False
    vllm_gpu_memory_utilization: float = 0.9
    group_size: int = 8
    dapo_delta: float = 0.1


@dataclass
class ExportConfig:
    enabled: bool = False
    output_dir: str = "./exported_model"
    format: ExportFormat = ExportFormat.SAFETENSORS
    push_to_hub: bool = False
    hub_model_id: Optional[str] = None
    hub_token: Optional[str] = None
    hub_private: bool = False
    merge_lora: bool = True
    save_merged_16bit: bool = True
    gguf_quantization: str = "q4_k_m"


@dataclass
class ParallelConfig:
    dp_replicate: int = 1
    dp_shard: int = -1          # -1: whatever is left of the world size
    cp: int = 1
    tp: int = 1
    pp: int = 1
    ep: int = 1
    etp: int = 1
    sp: bool = False
    pp_schedule: str = "1f1b"   # gpipe | 1f1b | interleaved | zero_bubble
    pp_microbatches: int = 0    # 0: = num_microbatches
    cp_balancer: str = "head_tail"


@dataclass
class DistributedConfig:
    enabled: bool = False
    backend: str = "nccl"
    strategy: str = "ddp"
    world_size: int = 1
    gradient_checkpointing: bool = True
    gradient_checkpointing_use_reentrant: bool = False
    fsdp_config: Dict[str, Any] = field(default_factory=dict)
    ddp_config: Dict[str, Any] = field(default_factory=dict)
    deepspeed_config: Optional[str] = None
    num_pipeline_stages: int = 4
    num_microbatches: int = 8
    pipeline_memory_limit_gb: float = 4.0
    ddp_gradient_as_bucket_view: bool = True
    ddp_static_graph: bool = True
    ddp_find_unused_parameters: bool = False
    ddp_broadcast_buffers: bool = True
    ddp_bucket_cap_mb: int = 25
    fsdp_limit_all_gathers: bool = True
    fsdp_use_orig_params: bool = False
    fsdp_reduce_dtype: str = "fp32"
    fsdp_sharding_strategy: str = "full"
    fsdp_forward_prefetch: bool = True
    fsdp_backward_prefetch: str = "backward_pre"
    context_parallel_size: int = 2
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    comm: str = "auto"     # auto | fused (peer-memory kernels) | nccl (baseline path)


@dataclass
class HardwareConfig:
    device: DeviceType = DeviceType.AUTO
    device_id: int = 0
    precision: Precision = Precision.BF16
    tf32: bool = True
    compile_model: bool = False
    compile_mode: str = "reduce-overhead"
    num_workers: int = 4
    pin_memory: bool = True
    prefetch_factor: int = 2
    # fp8 precisions: "rowwise" = per-token / per-feature scales, forward + dgrad + wgrad in fp8 (precision fp8_e5m2
    # keeps activations and weights in E4M3 and quantises gradients to E5M2); "block" = 1 x 128 / 128 x 128 scales
    fp8_recipe: str = "rowwise"


@dataclass
class KernelConfig:
    use_triton: bool = True            # accepted for file compatibility; this framework has no Triton path
    use_flash_attention: bool = True
    use_fused_rope: bool = True
    use_fused_rms_norm: bool = True
    use_fused_cross_entropy: bool = True
    use_fused_lora: bool = True
    use_moe_kernels: bool = True
    autotune: bool = True
    activation_checkpointing: bool = True
    memory_efficient_attention: bool = True


@dataclass
class DataConfig:
    dataset_name: str = ""
    dataset_config: Optional[str] = None
    streaming: bool = False
    max_samples: Optional[int] = None
    train_split: str = "train"
    eval_split: Optional[str] = "validation"
    text_column: str = "text"
    max_seq_length: int = 4096
    packing: bool = True
    packing_efficiency: float = 0.95
    shuffle: bool = True
    seed: int = 42


@dataclass
class TrainConfig:
    output_dir: str = "./outputs"
    num_train_epochs: int = 3
    max_steps: int = -1
    per_device_train_batch_size: int = 4
    per_device_eval_batch_size: int = 8
    gradient_accumulation_steps: int = 4
    eval_strategy: str = "steps"
    eval_steps: int = 100
    save_strategy: str = "steps"
    save_steps: int = 100
    save_total_limit: int = 3
    logging_steps: int = 10
    seed: int = 42
    resume_from_checkpoint: Optional[str] = None
    early_stopping_patience: int = 3
    early_stopping_threshold: float = 0.01


def _coerce(cls, value):
    """Build dataclass `cls` from a dict: enums by value, nested dataclasses, tuples; unknown keys -> TypeError."""
    if isinstance(value, cls):
        return value
    if not isinstance(value, dict):
        raise TypeError(f"{cls.__name__} section must be a mapping, got {type(value).__name__}")
    hints = {f.name: f for f in dataclasses.fields(cls)}
    unknown = set(value) - set(hints)
    if unknown:
        raise TypeError(f"{cls.__name__}.__init__() got an unexpected keyword argument {sorted(unknown)[0]!r}")
    kw = {}
    for k, v in value.items():
        default = hints[k].default if hints[k].default is not dataclasses.MISSING else (
            hints[k].default_factory() if hints[k].default_factory is not dataclasses.MISSING else None)
        if isinstance(default, Enum) and not isinstance(v, Enum):
            v = type(default)(v)
        elif dataclasses.is_dataclass(default) and isinstance(v, dict):
            v = _coerce(type(default), v)
        elif isinstance(default, tuple) and isinstance(v, list):
            v = tuple(v)
        kw[k] = v
    return cls(**kw)


def _plain(v):
    if isinstance(v, Enum):
        return v.value
    if dataclasses.is_dataclass(v):
        return {f.name: _plain(getattr(v, f.name)) for f in dataclasses.fields(v)}
    if isinstance(v, (list, tuple)):
        return [_plain(x) for x in v]
    if isinstance(v, dict):
        return {k: _plain(x) for k, x in v.items()}
    return v


_SECTIONS = {"model": ModelConfig, "tokenizer": TokenizerConfig, "lora": LoRAConfig, "quantization": QuantizationConfig,
             "optimizer": OptimizerConfig, "scheduler": SchedulerConfig, "loss": LossConfig, "rl": RLConfig,
             "export": ExportConfig, "distributed": DistributedConfig, "hardware": HardwareConfig,
             "kernels": KernelConfig, "data": DataConfig, "training": TrainConfig}


@dataclass
class SOTAConfig:
    config_version: str = "2.0"
    config_type: str = "sota_training"
    training_mode: TrainingMode = TrainingMode.FULL_FINETUNE
    model: ModelConfig = field(default_factory=ModelConfig)
    tokenizer: TokenizerConfig = field(default_factory=TokenizerConfig)
    lora: LoRAConfig = field(default_factory=lambda: LoRAConfig(enabled=False))
    quantization: QuantizationConfig = field(default_factory=QuantizationConfig)
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    loss: LossConfig = field(default_factory=LossConfig)
    rl: RLConfig = field(default_factory=RLConfig)
    export: ExportConfig = field(default_factory=ExportConfig)
    distributed: DistributedConfig = field(default_factory=DistributedConfig)
    hardware: HardwareConfig = field(default_factory=HardwareConfig)
    kernels: KernelConfig = field(default_factory=KernelConfig)
    data: DataConfig = field(default_factory=DataConfig)
    training: TrainConfig = field(default_factory=TrainConfig)

    def __post_init__(self):
        if not isinstance(self.training_mode, TrainingMode):
            self.training_mode = TrainingMode(self.training_mode)
        self._validate()

    def _validate(self):
        if self.training_mode in (TrainingMode.LORA, TrainingMode.QLORA):
            self.lora.enabled = True
        if self.training_mode == TrainingMode.QLORA and not self.quantization.enabled:
            self.quantization.enabled = True
            self.quantization.load_in_4bit = True
        if self.training_mode == TrainingMode.RL:
            self.rl.enabled = True
        if self.training.gradient_accumulation_steps < 1:
            raise ValueError("training.gradient_accumulation_steps must be >= 1")
        if self.optimizer.learning_rate <= 0:
            raise ValueError("optimizer.learning_rate must be positive")
        p = self.distributed.parallel
        for n in ("dp_replicate", "cp", "tp", "pp", "ep", "etp"):
            if getattr(p, n) < 1:
                raise ValueError(f"distributed.parallel.{n} must be >= 1")

    @classmethod
    @reference_kwargs(d="raw")
    def from_dict(cls, raw: Dict[str, Any]) -> "SOTAConfig":
        """Sections this class does not know (the data half's keys: type, version, dataset, prompt_template, ...)
        are ignored, exactly like the reference loads one YAML file twice."""
        raw = raw or {}
        kw: Dict[str, Any] = {}
        for k in ("config_version", "config_type", "training_mode"):
            if k in raw:
                kw[k] = raw[k]
        for name, sec in _SECTIONS.items():
            if name in raw and raw[name] is not None:
                d = raw[name]
                if name == "tokenizer" and isinstance(d, dict):
                    d = dict(d)
                kw[name] = _coerce(sec, d)
        return cls(**kw)

    @classmethod
    def from_yaml(cls, path: Union[str, Path]) -> "SOTAConfig":
        path = Path(path)
        if not path.exists():
            raise FileNotFoundError(f"Config file not found: {path}")
        with open(path) as f:
            return cls.from_dict(yaml.safe_load(f) or {})

    def to_dict(self) -> Dict[str, Any]:
        return _plain(self)

    def save_yaml(self, path: Union[str, Path]) -> None:
        Path(path).parent.mkdir(parents=True, exist_ok=True)
        with open(path, "w") as f:
            yaml.safe_dump(self.to_dict(), f, sort_keys=False)

    @property
    def effective_batch_size(self) -> int:
        w = self.distributed.world_size if self.distributed.enabled else 1
        return self.training.per_device_train_batch_size * self.training.gradient_accumulation_steps * max(1, w)

    @property
    def compute_dtype(self) -> torch.dtype:
        return {Precision.FP32: torch.float32, Precision.FP16: torch.float16}.get(self.hardware.precision,
                                                                                   torch.bfloat16)

    def copy(self) -> "SOTAConfig":
        return copy.deepcopy(self)


# ---------------------------------------------------------------- presets (data_pipeline/trainer/core/sota_config.py:625-691)
def _preset(fn):
    """Presets also take the reference's `model_name=` for `model` and `max_seq_length=`, which is written to
    `data.max_seq_length` of the returned configuration."""
    import functools
    import inspect

    @functools.wraps(fn)
    def wrapper(model: str = "", *, model_name: str | None = None, max_seq_length: int | None = None):
        cfg = fn(model_name if model_name is not None else model)
        if max_seq_length is not None:
            cfg.data.max_seq_length = int(max_seq_length)
        return cfg
    wrapper.__signature__ = inspect.signature(wrapper, follow_wrapped=False)
    return wrapper


@_preset
def get_qlora_preset(model: str = "") -> SOTAConfig:
    return SOTAConfig(training_mode=TrainingMode.QLORA, model=ModelConfig(name_or_path=model),
                      lora=LoRAConfig(r=16, lora_alpha=32), optimizer=OptimizerConfig(learning_rate=2e-4))


@_preset
def get_lora_preset(model: str = "") -> SOTAConfig:
    return SOTAConfig(training_mode=TrainingMode.LORA, model=ModelConfig(name_or_path=model),
                      lora=LoRAConfig(r=64, lora_alpha=128), optimizer=OptimizerConfig(learning_rate=1e-4))


@_preset
def get_full_finetune_preset(model: str = "") -> SOTAConfig:
    return SOTAConfig(training_mode=TrainingMode.FULL_FINETUNE, model=ModelConfig(name_or_path=model),
                      lora=LoRAConfig(enabled=False), optimizer=OptimizerConfig(learning_rate=2e-5),
                      scheduler=SchedulerConfig(type=SchedulerType.WSD))


@_preset
def get_fp8_preset(model: str = "") -> SOTAConfig:
    c = get_full_finetune_preset(model)
    c.hardware.precision = Precision.FP8_E4M3
    return c


@_preset
def get_rl_grpo_preset(model: str = "") -> SOTAConfig:
    return SOTAConfig(training_mode=TrainingMode.RL, model=ModelConfig(name_or_path=model),
                      rl=RLConfig(enabled=True, algorithm=RLAlgorithm.GRPO),
                      optimizer=OptimizerConfig(learning_rate=1e-6))


@_preset
def get_pretrain_preset(model: str = "") -> SOTAConfig:
    return SOTAConfig(training_mode=TrainingMode.PRETRAIN, model=ModelConfig(name_or_path=model),
                      lora=LoRAConfig(enabled=False), optimizer=OptimizerConfig(learning_rate=3e-4, weight_decay=0.1),
                      scheduler=SchedulerConfig(type=SchedulerType.WSD, warmup_ratio=0.01))


@_preset
def get_dpo_preset(model: str = "") -> SOTAConfig:
    """Preference optimisation with the DPO loss (beta 0.1) against a frozen copy of the starting weights."""
    return SOTAConfig(training_mode=TrainingMode.RL, model=ModelConfig(name_or_path=model),
                      rl=RLConfig(enabled=True, algorithm=RLAlgorithm.DPO),
                      loss=LossConfig(type=LossType.DPO, dpo_beta=0.1), optimizer=OptimizerConfig(learning_rate=5e-7))


_GGUF_FORMATS = {"q4_k_m": ExportFormat.GGUF_Q4, "q5_k_m": ExportFormat.GGUF_Q5, "q8_0": ExportFormat.GGUF_Q8,
                 "f16": ExportFormat.GGUF_F16}


def get_export_gguf_preset(output_dir: str, quant: str = "q4_k_m") -> ExportConfig:
    """Export section for a GGUF file of the given quantisation (adapters merged first)."""
    if quant not in _GGUF_FORMATS:
        raise ValueError(f"unknown GGUF quantisation {quant!r}; choose from {sorted(_GGUF_FORMATS)}")
    return ExportConfig(enabled=True, output_dir=output_dir, format=_GGUF_FORMATS[quant], gguf_quantization=quant,
                        merge_lora=True)
