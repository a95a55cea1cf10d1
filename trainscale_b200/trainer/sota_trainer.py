"""SOTATrainer: YAML-driven training loop over the framework's own decoder and flat sharded engine.

Public surface follows data_pipeline/trainer/trainers/sota_trainer.py:640-3701:
`SOTATrainer(config)`, `.setup_model(model=None, model_init_fn=None)`, `.setup_optimizer()`, `.setup_scheduler(n)`,
`.train(train_dl, eval_dl, compute_metrics) -> dict`, `.evaluate(dl)`, `.save_checkpoint(path)`,
`.load_checkpoint(path)`, `.export(tokenizer)`, `.cleanup()`, `create_trainer(path_or_config)`; strategy aliases
(:264-277); checkpoint layout `{output_dir}/checkpoint-{step}` with an atomic `trainer_state.pt` (:2920-2958);
log line `Epoch | Step | Loss | PPL | LR | Grad | Tok/s | MFU` (:2412-2422); step arithmetic
`num_training_steps = len(dl) // grad_accum * epochs`, boundary when `(step+1) % grad_accum == 0` (:1938-1942,2199).

What is different by design: the hot loop never synchronises the host (loss, token counts, grad-norm and the
non-finite check stay on the device and are read only at logging steps), throughput comes from CUDA events, the
causal shift + loss run in the fused lm_head/cross-entropy head, and DDP/FSDP are the flat engine of
`parallel/flat_engine.py` rather than torch wrappers.
"""
from __future__ import annotations

import contextlib

import logging
import math
import os
import random
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, Iterable, Optional

import numpy as np
import torch
import torch.distributed as dist
import torch.nn as nn

from ..callbacks import (CallbackContext, CallbackHandler, CheckpointCallback, EarlyStoppingCallback, LoggingCallback)
from ..config.sota_config import OptimizerType, Precision, SOTAConfig, TrainingMode
from ..core.errors import CheckpointLoadError, TrainingConfigurationError
from ..metrics.throughput import ThroughputTracker, device_peak_tflops
from ..models.llama import LlamaConfig, LlamaForCausalLM, build_model, preset_config
from ..parallel.flat_engine import EngineConfig, FlatShardedEngine
from ..schedulers import create_scheduler

from ..utils.tracing import nvtx_range

logger = logging.getLogger("trainscale_b200")

STRATEGY_ALIASES = {
    "ddp": "ddp", "sota_ddp": "ddp", "dp": "ddp", "none": "single", "single": "single",
    "fsdp": "fsdp", "fsdp2": "fsdp", "fsdp_v2": "fsdp", "sota_fsdp": "fsdp", "sota_fsdp2": "fsdp",
    "full_shard": "fsdp", "zero3": "fsdp", "zero2": "fsdp", "hsdp": "fsdp",
    "zbpp": "pipeline", "pipeline_zbpp": "pipeline", "pipeline": "pipeline", "pp": "pipeline",
    "context_parallel": "context_parallel", "cp": "context_parallel", "tp": "tensor_parallel",
    "tensor_parallel": "tensor_parallel", "nd": "nd", "3d": "nd",
}

PREFERENCE_LOSSES = ("dpo", "simpo", "orpo", "kto", "cpo")

_SHARDING = {"full": "FULL_SHARD", "full_shard": "FULL_SHARD", "shard_grad_op": "SHARD_GRAD_OP",
             "zero2": "SHARD_GRAD_OP", "no_shard": "NO_SHARD", "hybrid_shard": "FULL_SHARD", "auto": "SHARD_GRAD_OP"}


@dataclass
class TrainingState:
    epoch: int = 0
    global_step: int = 0
    best_metric: float = float("inf")
    total_loss: float = 0.0
    samples_seen: int = 0
    patience_counter: int = 0
    max_steps: int = 0
    tokens_seen: int = 0

    def with_update(self, **kwargs) -> "TrainingState":
        """A copy with the given fields replaced (the state object of a running trainer is not touched)."""
        import dataclasses
        return dataclasses.replace(self, **kwargs)


def set_seed(seed: int, rank: int = 0, deterministic: bool = False) -> None:
    """seed + rank for python / numpy / torch (data_pipeline/trainer/distributed/sota_utils.py:1731-1768)."""
    s = seed + rank
    random.seed(s)
    np.random.seed(s % (2 ** 32))
    torch.manual_seed(s)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(s)
    if deterministic:
        torch.use_deterministic_algorithms(True, warn_only=True)


class SOTATrainer:
    def __init__(self, config: SOTAConfig, callbacks: list | None = None):
        self.config = config
        self.state = TrainingState()
        self.model: nn.Module | None = None
        self.engine: FlatShardedEngine | None = None
        self.optimizer = None
        self.scheduler = None
        self.loss_fn = None
        self.tokenizer = None
        self._own_pg = False
        self._setup_distributed()
        self._setup_device()
        set_seed(config.training.seed, self.rank)
        self.callbacks = CallbackHandler()
        t = config.training
        self.callbacks.add(LoggingCallback(t.logging_steps, ("console",), t.output_dir, self.rank))
        self.callbacks.add(CheckpointCallback(t.output_dir, t.save_strategy, t.save_steps, t.save_total_limit))
        if t.early_stopping_patience and t.early_stopping_patience > 0:
            self.callbacks.add(EarlyStoppingCallback(t.early_stopping_patience, t.early_stopping_threshold))
        for cb in callbacks or []:
            self.callbacks.add(cb)
        self.throughput = ThroughputTracker(world_size=self.world_size)
        self.ema_loss: float | None = None
        self._ctx = CallbackContext(trainer=self, state=self.state, config=config)
        self.callbacks.fire("on_init_end", self._ctx)

    # ------------------------------------------------------------------ environment
    def _setup_distributed(self):
        self.world_size = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        d = self.config.distributed
        want = self.world_size > 1 and (d.enabled or self.world_size > 1)
        if want and not dist.is_initialized():
            backend = d.backend
            if backend == "nccl" and not torch.cuda.is_available():
                backend = "gloo"
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            if backend == "nccl":
                torch.cuda.set_device(self.local_rank)
            dist.init_process_group(backend=backend, rank=self.rank, world_size=self.world_size,
                                    **({"device_id": torch.device("cuda", self.local_rank)} if backend == "nccl" else {}))
            self._own_pg = True
        self.is_distributed = dist.is_initialized() and dist.get_world_size() > 1
        if self.is_distributed:
            self.world_size, self.rank = dist.get_world_size(), dist.get_rank()
        else:
            self.world_size, self.rank = 1, 0
        self.is_main = self.rank == 0

    def _setup_device(self):
        hw = self.config.hardware
        dev = getattr(hw.device, "value", hw.device)
        if dev in ("auto", "cuda") and torch.cuda.is_available():
            idx = self.local_rank if self.is_distributed else hw.device_id
            self.device = torch.device("cuda", idx)
            torch.cuda.set_device(self.device)
            torch.backends.cuda.matmul.allow_tf32 = bool(hw.tf32)
        else:
            self.device = torch.device("cpu")
        self.dtype = self.config.compute_dtype if self.device.type == "cuda" else (
            torch.float32 if hw.precision in (Precision.FP32,) or self.device.type == "cpu" else self.config.compute_dtype)

    @property
    def strategy(self) -> str:
        d = self.config.distributed
        s = STRATEGY_ALIASES.get(str(d.strategy).lower())
        if s is None:
            raise TrainingConfigurationError(f"unknown distributed.strategy {d.strategy!r}",
                                             choices=sorted(STRATEGY_ALIASES))
        if not self.is_distributed and s in ("ddp",):
            return "single"
        return s

    @property
    def preference_kind(self) -> str | None:
        """The preference objective this run trains with, or None for language-model training: `loss.type` in
        dpo / simpo / orpo / kto / cpo, or `training_mode: rl` with such an `rl.algorithm`
        (data_pipeline/trainer/core/sota_config.py:53-60,261; losses data_pipeline/trainer/loss/sota_losses.py:1151,1448)."""
        lt = str(getattr(self.config.loss.type, "value", self.config.loss.type)).lower()
        if lt in PREFERENCE_LOSSES:
            return lt
        mode = str(getattr(self.config.training_mode, "value", self.config.training_mode)).lower()
        alg = str(getattr(self.config.rl.algorithm, "value", self.config.rl.algorithm)).lower()
        if mode == "rl" and alg in PREFERENCE_LOSSES:
            return alg
        return None

    # ------------------------------------------------------------------ model
    def _build_own_model(self) -> nn.Module:
        arch = self.config.model.architecture
        if arch is None:
            name = (self.config.model.name_or_path or "").lower()
            for k in ("llama3-8b", "llama3-70b", "llama3-1b", "mistral-7b", "qwen2-7b", "tiny"):
                if k in name.replace("_", "-"):
                    arch = k
                    break
        if arch is None:
            p = Path(self.config.model.name_or_path or "")
            if p.is_dir() and (p / "config.json").exists():
                from ..hub import load_pretrained
                return load_pretrained(p, dtype=self.dtype)
            raise TrainingConfigurationError(
                "no model given: pass setup_model(model=...), set model.architecture to a preset name / inline "
                "shape, or point model.name_or_path at a local HF-format directory")
        cfg = preset_config(arch) if isinstance(arch, str) else LlamaConfig.from_dict(arch)
        if self.config.model.max_position_embeddings:
            cfg.max_position_embeddings = self.config.model.max_position_embeddings
        seed = self.config.training.seed
        big = (cfg.num_parameters() > 2_000_000_000 and self.device.type == "cuda") or \
            os.environ.get("TS_BUILD_LOCAL_SLICE", "0") == "1"
        par = self.config.distributed.parallel
        tp, pp = int(getattr(par, "tp", 1) or 1), int(getattr(par, "pp", 1) or 1)
        if big and self.is_distributed and self.strategy in ("pipeline", "tensor_parallel", "nd") and (tp > 1 or pp > 1):
            # A random-init model too large to be built whole on every rank: build only what this rank will hold (its
            # tensor-parallel slice of every projection, its pipeline stage's layers), with weights drawn on the GPU.
            from ..parallel.mesh import create_parallel_dims_from_config
            from ..parallel.pp import split_layers
            dims = create_parallel_dims_from_config(self.config.distributed)
            local = cfg.tensor_parallel_local(tp) if tp > 1 else cfg
            layers = split_layers(cfg.num_hidden_layers, pp)[dims.local_rank("pp")] if pp > 1 else None
            model = build_model(local, dtype=self.dtype, device=self.device, layer_range=layers, init_on_device=True,
                                seed=seed + 7919 * dims.local_rank("tp"))
            model.config = cfg                       # the whole model's shape (FLOP accounting, checkpoint export)
            model.tp_presharded = tp
            return model
        return build_model(cfg, dtype=self.dtype, device=self.device, seed=seed, init_on_device=big)

    def setup_model(self, model: nn.Module | None = None, model_init_fn: Callable[[], nn.Module] | None = None):
        if model is None and model_init_fn is not None:
            model = model_init_fn()
        if model is None:
            model = self._build_own_model()
        model = model.to(self.device)
        if self.dtype != torch.float32 and not any(p.dtype == self.dtype for p in model.parameters()):
            model = model.to(self.dtype)
        self.model = model
        if self.config.lora.enabled:
            from ..lora import apply_lora
            self.model = apply_lora(self.model, self.config.lora)
        prec = getattr(self.config.hardware.precision, "value", self.config.hardware.precision)
        if prec in ("fp8_e4m3", "fp8_e5m2", "fp8") and hasattr(self.model, "enable_fp8") and self.device.type == "cuda":
            # bf16 parameters, fp8 tensor-core GEMMs for the layer projections
            self.model.enable_fp8(True, recipe=self.config.hardware.fp8_recipe,
                                  grad_format="e5m2" if prec == "fp8_e5m2" else "e4m3")
        d = self.config.distributed
        fc = dict(d.fsdp_config or {})
        use_ckpt = bool(fc.get("activation_checkpointing", d.gradient_checkpointing))
        if str(fc.get("ac_mode", "")).lower() == "op_selective" and hasattr(self.model, "op_selective_recompute"):
            self.model.op_selective_recompute(True)   # operator-level: nothing is re-run but norm / GLU outputs
            use_ckpt = False
        if use_ckpt and hasattr(self.model, "gradient_checkpointing_enable"):
            every = int(fc.get("ac_frequency", 1)) or 1
            self.model.gradient_checkpointing_enable(every)
        self.throughput.flops_per_token = self._flops_per_token()
        strat = self.strategy
        kind = self.preference_kind
        ref_model = None
        lc = self.config.loss
        if kind in ("dpo", "kto") and not lc.reference_free and self.config.rl.use_ref_model:
            # the frozen reference is the policy as it is now, copied before the engine re-points the policy's
            # parameters at its flat buffers
            import copy
            ref_model = copy.deepcopy(self.model).eval()
        ep = int(getattr(d.parallel, "ep", 1) or 1)
        if ep > 1 and self.is_distributed and strat in ("ddp", "fsdp") and self._flat_engine_ok():
            # expert parallelism inside data parallelism: experts sharded over groups of `ep` ranks
            from ..parallel.ep import ExpertParallelEngine
            proto = self._build_flat_engine_config(strat)
            self.engine = ExpertParallelEngine(self.model, proto, ep, self.device, proto.sharding_strategy)
        elif strat in ("single", "ddp", "fsdp") and all(p.requires_grad for p in self.model.parameters()) \
                and self._flat_engine_ok():
            self.engine = self._build_flat_engine(strat)
            if ref_model is not None:
                # parameter-only shards under the same sharding as the policy: no gradients, no optimizer state
                self.ref_engine = self._build_flat_engine(strat, model=ref_model, frozen=True)
        elif strat in ("pipeline", "context_parallel", "tensor_parallel", "nd"):
            from ..parallel.nd import build_nd_engine
            self.engine = build_nd_engine(self, strat)
        else:
            self.engine = None   # generic nn.Module path: torch optimizer (+ DDP all-reduce of .grad)
        if kind is not None:
            from ..rl import PreferenceTrainer
            kw = {"dpo": dict(loss_type=lc.dpo_variant, label_smoothing=lc.label_smoothing,
                              reference_free=lc.reference_free or ref_model is None),
                  "simpo": dict(gamma=lc.simpo_gamma, label_smoothing=lc.label_smoothing),
                  "orpo": dict(alpha=lc.alpha), "cpo": dict(alpha=lc.alpha, label_smoothing=lc.label_smoothing),
                  "kto": {}}[kind]
            if kind == "orpo":
                self.preference = PreferenceTrainer(self.model, None, None, "orpo", **kw)
            else:
                self.preference = PreferenceTrainer(self.model, None, ref_model, kind, lc.dpo_beta, **kw)
        self._ctx.model = self.model
        return self.model

    def _flat_engine_ok(self) -> bool:
        t = getattr(self.config.optimizer.type, "value", self.config.optimizer.type)
        return t in ("adamw", "fused_adamw", "lion")

    def _build_flat_engine_config(self, strat: str) -> EngineConfig:
        c, d = self.config, self.config.distributed
        fc = dict(d.fsdp_config or {})
        if strat == "ddp":
            sharding = "NO_SHARD"
        elif strat == "single":
            sharding = "SHARD_GRAD_OP"
        else:
            sharding = _SHARDING.get(str(fc.get("sharding_strategy", d.fsdp_sharding_strategy)).lower(), "SHARD_GRAD_OP")
        opt_type = getattr(c.optimizer.type, "value", c.optimizer.type)
        betas = tuple(c.optimizer.lion_betas if opt_type == "lion" else c.optimizer.betas)
        ec = EngineConfig(
            sharding_strategy=sharding, param_dtype=self.dtype,
            gradient_accumulation_steps=int(fc.get("gradient_accumulation_steps",
                                                   c.training.gradient_accumulation_steps)),
            max_grad_norm=float(fc.get("gradient_clipping_norm", c.optimizer.max_grad_norm) or 0.0),
            lr=c.optimizer.learning_rate, betas=betas, eps=c.optimizer.eps, weight_decay=c.optimizer.weight_decay,
            optimizer="lion" if opt_type == "lion" else "adamw", comm=d.comm,
            reshard_after_forward=bool(fc.get("reshard_after_forward", True)),
            gather_engine=str(fc.get("gather_engine", "ce")))
        c.training.gradient_accumulation_steps = ec.gradient_accumulation_steps
        return ec

    def _build_flat_engine(self, strat: str, model: nn.Module | None = None, frozen: bool = False) -> FlatShardedEngine:
        d = self.config.distributed
        model = self.model if model is None else model
        ec = self._build_flat_engine_config(strat)
        par = d.parallel
        if self.is_distributed and strat == "fsdp" and int(getattr(par, "dp_replicate", 1) or 1) > 1:
            # hybrid sharding: shard inside groups of world / dp_replicate ranks, replicate across them
            from ..parallel.mesh import create_parallel_dims_from_config
            dims = create_parallel_dims_from_config(d)
            self._hsdp_dims = dims
            return FlatShardedEngine(model, ec, process_group=dims.group("fsdp"), device=self.device,
                                     replicate_group=dims.group("dp_replicate"), frozen=frozen)
        return FlatShardedEngine(model, ec, device=self.device, frozen=frozen)

    @staticmethod
    def _batch_tokens(batch: Dict[str, Any]) -> int:
        if "input_ids" in batch:
            return int(batch["input_ids"].numel())
        return sum(int(v.numel()) for k, v in batch.items() if k in ("chosen_input_ids", "rejected_input_ids"))

    def _data_parallel_size(self) -> int:
        """Ranks that consume different samples (tensor / pipeline / context ranks of one replica share theirs)."""
        dims = getattr(self.engine, "dims", None)
        if dims is not None:
            return max(1, dims.size("dp"))
        return self.world_size

    def data_rank(self) -> int:
        """Index of the data shard this rank reads: ranks of one model replica (tensor / pipeline / context parallel
        peers) must see the same samples, so it is the data-parallel coordinate, not the global rank."""
        dims = getattr(self.engine, "dims", None)
        return dims.local_rank("dp") if dims is not None else self.rank

    def _token_multiplier(self) -> int:
        """Whole-job tokens per token of this rank's (sharded) batch: data-parallel replicas, times the context-parallel
        size (a context-parallel rank holds only its slice of every sequence)."""
        dims = getattr(self.engine, "dims", None)
        if dims is not None:
            return max(1, dims.size("dp")) * (dims.size("cp") if dims.enabled("cp") else 1)
        return self.world_size

    def _flops_per_token(self) -> float:
        cfg = getattr(self.model, "config", None)
        seq = self.config.data.max_seq_length
        if isinstance(cfg, LlamaConfig):
            return cfg.flops_per_token(seq)
        n = sum(p.numel() for p in self.model.parameters())
        return 6.0 * n

    # ------------------------------------------------------------------ optimizer / scheduler / loss
    def setup_optimizer(self):
        if self.engine is not None and hasattr(self.engine, "param_groups"):
            self.optimizer = self.engine
        else:
            from ..optim import create_optimizer
            self.optimizer = create_optimizer(self.model.parameters(), self.config.optimizer)
        self._ctx.optimizer = self.optimizer
        return self.optimizer

    def setup_scheduler(self, num_training_steps: int):
        s = self.config.scheduler
        self.scheduler = create_scheduler(
            self.optimizer, getattr(s.type, "value", s.type), num_training_steps, warmup_steps=s.warmup_steps,
            warmup_ratio=s.warmup_ratio, min_lr_ratio=s.min_lr_ratio, stable_ratio=s.stable_ratio,
            decay_type=s.decay_type, power=s.power, max_lr_ratio=s.max_lr_ratio)
        self._ctx.scheduler = self.scheduler
        return self.scheduler

    def setup_loss(self):
        from ..losses import create_loss_from_config
        self.loss_fn = create_loss_from_config(self.config.loss)
        return self.loss_fn

    # ------------------------------------------------------------------ one micro-step
    def _to_device(self, batch: Dict[str, Any]) -> Dict[str, Any]:
        batch = {k: (v.to(self.device, non_blocking=True) if torch.is_tensor(v) else v) for k, v in batch.items()}
        if self.engine is not None and hasattr(self.engine, "shard_batch"):
            batch = self.engine.shard_batch(batch)     # context parallelism: this rank's sequence chunks
        return batch

    def _loss_and_backward(self, batch: Dict[str, Any], loss_scale: float):
        """Forward + backward of one micro-batch.  A pipeline engine runs its own schedule over the batch."""
        if self.engine is not None and hasattr(self.engine, "forward_backward") and self.engine.pipelined:
            return self.engine.forward_backward(batch, loss_scale)
        cp_group = getattr(self.engine, "cp_group", None) if self.engine is not None else None
        denom = None
        if cp_group is not None and batch.get("labels_shifted", False):
            # context parallelism: every rank averages over ITS valid tokens and the engine averages the ranks, which
            # equals the mean over the whole sequence only if the shards hold the same number of valid labels.  They do
            # not in general (the last position has no label; packed documents mask more), so each rank divides its
            # summed loss by n_global / cp.  The count stays on the device: the loss head takes it as a tensor.
            n_global = (batch["labels"] != self.config.loss.ignore_index).sum().float().reshape(1)
            dist.all_reduce(n_global, group=cp_group)
            denom = n_global.clamp(min=1.0) / dist.get_world_size(cp_group)
        loss, ntok = self._forward_loss(batch, loss_scale, denom)
        if self.engine is not None:
            self.engine.backward(loss)
        return loss, ntok

    def _forward_loss(self, batch: Dict[str, Any], loss_scale: float, loss_denominator: torch.Tensor | None = None):
        """Returns (scaled loss, valid-token count tensor)."""
        lc = self.config.loss
        m = self.model
        if "chosen_input_ids" in batch:
            if getattr(self, "preference", None) is None:
                raise TrainingConfigurationError("a preference batch (chosen_/rejected_ keys) needs loss.type or "
                                                 "rl.algorithm in " + "/".join(PREFERENCE_LOSSES))
            loss, metrics = self.preference.compute_loss(batch)
            self.last_preference_metrics = metrics
            ntok = (batch["chosen_labels"] != lc.ignore_index).sum() + (batch["rejected_labels"] != lc.ignore_index).sum()
            return loss * loss_scale, ntok
        if isinstance(m, LlamaForCausalLM) or hasattr(m, "loss_chunk_tokens"):
            out = m(input_ids=batch["input_ids"], attention_mask=batch.get("attention_mask"),
                    labels=batch.get("labels", batch["input_ids"]), position_ids=batch.get("position_ids"),
                    doc_ids=batch.get("document_ids"), cu_seqlens=batch.get("cu_seqlens"), loss_scale=loss_scale,
                    label_smoothing=lc.label_smoothing, ignore_index=lc.ignore_index,
                    shift_labels=not batch.get("labels_shifted", False), loss_denominator=loss_denominator)
            return out.loss, out.num_tokens
        out = m(**{k: v for k, v in batch.items() if k in ("input_ids", "attention_mask", "labels")})
        loss = out.loss if hasattr(out, "loss") and out.loss is not None else None
        if loss is None:
            logits = out.logits if hasattr(out, "logits") else out
            labels = batch["labels"]
            loss = torch.nn.functional.cross_entropy(logits[..., :-1, :].reshape(-1, logits.shape[-1]).float(),
                                                     labels[..., 1:].reshape(-1), ignore_index=lc.ignore_index,
                                                     label_smoothing=lc.label_smoothing)
        ntok = (batch.get("labels", batch["input_ids"])[..., 1:] != lc.ignore_index).sum()
        return loss * loss_scale, ntok

    def _generic_backward_step(self, loss, sync: bool):
        loss.backward()
        if not sync:
            return None
        params = [p for p in self.model.parameters() if p.grad is not None]
        if self.is_distributed:
            for p in params:
                dist.all_reduce(p.grad)
                p.grad.div_(self.world_size)
        mg = self.config.optimizer.max_grad_norm
        gn = torch.nn.utils.clip_grad_norm_(params, mg if mg and mg > 0 else float("inf"))
        self.optimizer.step()
        self.optimizer.zero_grad(set_to_none=True)
        return gn

    # ------------------------------------------------------------------ single public step
    def train_step(self, batch: Dict[str, Any]) -> float:
        """One optimizer step on one host batch (no accumulation): host->device copy of the batch, forward,
        backward, reduction, update, and the loss read back to the host as a float."""
        if self.optimizer is None:
            self.setup_optimizer()
        if self.scheduler is None:
            self.setup_scheduler(max(1, self.config.training.max_steps))
        self.model.train()
        batch = self._to_device(batch)
        if self.engine is not None:
            self.engine.micro_step = max(1, self.config.training.gradient_accumulation_steps) - 1
            loss, _ = self._loss_and_backward(batch, 1.0)
            self.engine.step(self.optimizer.param_groups[0]["lr"])
        else:
            loss, _ = self._forward_loss(batch, 1.0)
            self._generic_backward_step(loss, True)
        self.scheduler.step()
        self.state.global_step += 1
        out = float(loss.detach().float().item())
        self._check_comm()
        return out

    def _check_comm(self) -> None:
        """After a host read of the loss (the stream has drained): did a fused collective give up on a peer, did any
        kernel record an error?  Raises CommunicationError / KernelError instead of training on skipped updates."""
        eng = self.engine
        if eng is not None and hasattr(eng, "check_comm_status"):
            eng.check_comm_status()

    # ------------------------------------------------------------------ train
    def train(self, train_dataloader: Iterable, eval_dataloader: Iterable | None = None,
              compute_metrics: Callable | None = None) -> Dict[str, Any]:
        if self.model is None:
            self.setup_model()
        cfg, t = self.config, self.config.training
        gas = max(1, t.gradient_accumulation_steps)
        if self.optimizer is None:
            self.setup_optimizer()
        try:
            steps_per_epoch = max(1, len(train_dataloader) // gas)
        except TypeError:
            steps_per_epoch = max(1, t.max_steps)
        total_steps = steps_per_epoch * max(1, t.num_train_epochs)
        if t.max_steps and t.max_steps > 0:
            total_steps = min(total_steps, t.max_steps) if t.num_train_epochs > 0 else t.max_steps
        self.state.max_steps = total_steps
        if self.scheduler is None:
            self.setup_scheduler(total_steps)
        if t.resume_from_checkpoint:
            target = t.resume_from_checkpoint
            if str(target).lower() in ("latest", "auto", "true"):
                # elastic restart: newest checkpoint of this run that is complete and undamaged, whatever world size
                # wrote it (optimizer shards are re-sliced on load); nothing to resume from on the first launch
                from ..ckpt import find_latest_valid_checkpoint
                target = find_latest_valid_checkpoint(Path(t.output_dir), log=logger.warning)
            if target:
                self.load_checkpoint(target)
        self.model.train()
        ctx = self._ctx
        self.callbacks.fire("on_train_begin", ctx)
        dev = self.device
        loss_acc = torch.zeros((), dtype=torch.float32, device=dev)
        tok_acc = torch.zeros((), dtype=torch.float32, device=dev)
        window_loss = torch.zeros((), dtype=torch.float32, device=dev)
        window_steps = 0
        last_gn = torch.zeros((), dtype=torch.float32, device=dev)
        t_start = time.time()
        history: list[dict] = []
        done = False
        start_epoch = self.state.epoch
        for epoch in range(start_epoch, max(1, t.num_train_epochs)):
            self.state.epoch = epoch
            self.callbacks.fire("on_epoch_begin", ctx)
            sampler = getattr(train_dataloader, "sampler", None)
            if hasattr(sampler, "set_epoch"):
                sampler.set_epoch(epoch)
            for step, batch in enumerate(train_dataloader):
                micro = step % gas
                if micro == 0:
                    self.callbacks.fire("on_step_begin", ctx)
                    self.throughput.start_step()
                    step_tokens = 0
                with nvtx_range("h2d_batch"):
                    batch = self._to_device(batch)
                step_tokens += self._batch_tokens(batch)
                sync = (step + 1) % gas == 0
                if self.engine is not None:
                    if not getattr(self.engine, "pipelined", False):
                        # this loop decides where an accumulation window ends; the engine's own counter (which picks
                        # the micro-batch whose backward starts the overlapped reduction) follows it
                        self.engine.micro_step = micro
                    with nvtx_range("forward_backward"):
                        loss, ntok = self._loss_and_backward(batch, 1.0 / gas)
                    if sync:
                        with nvtx_range("reduce_clip_update"):
                            last_gn = self.engine.step(self.optimizer.param_groups[0]["lr"])
                else:
                    loss, ntok = self._forward_loss(batch, 1.0 / gas)
                    gn = self._generic_backward_step(loss, sync)
                    if gn is not None:
                        last_gn = gn.detach()
                loss_acc += loss.detach().float()
                tok_acc += ntok.float() if torch.is_tensor(ntok) else float(ntok)
                self.state.samples_seen += int(next(v for v in batch.values() if torch.is_tensor(v)).shape[0]) * \
                    self._data_parallel_size()
                if not sync:
                    continue
                self.scheduler.step()
                self.state.global_step += 1
                self.state.tokens_seen += step_tokens * self._data_parallel_size()
                self.throughput.end_step(step_tokens)
                window_loss += loss_acc
                window_steps += 1
                loss_acc.zero_()
                ctx.should_log = ctx.should_save = ctx.should_evaluate = False
                self.callbacks.fire("on_step_end", ctx)
                if ctx.should_log or self.state.global_step == total_steps:
                    rec = self._log(window_loss, window_steps, last_gn, t_start, total_steps)
                    history.append(rec)
                    window_loss.zero_()
                    window_steps = 0
                if eval_dataloader is not None and t.eval_strategy == "steps" and t.eval_steps > 0 \
                        and self.state.global_step % t.eval_steps == 0:
                    self._run_eval(eval_dataloader, compute_metrics)
                if ctx.should_save:
                    self.save_checkpoint()
                if ctx.should_stop or self.state.global_step >= total_steps:
                    done = True
                    break
            if not done and (step + 1) % gas != 0:
                # the loader ended inside an accumulation window: those micro-batches make no step (the step count is
                # len(loader) // gas per epoch) and must not leak into the first update of the next epoch
                if self.engine is not None and hasattr(self.engine, "zero_grad"):
                    self.engine.zero_grad()
                elif self.optimizer is not None and self.engine is None:
                    self.optimizer.zero_grad(set_to_none=True)
                loss_acc.zero_()
            self.callbacks.fire("on_epoch_end", ctx)
            if eval_dataloader is not None and t.eval_strategy == "epoch" and not done:
                self._run_eval(eval_dataloader, compute_metrics)
            if ctx.should_save and not done:
                self.save_checkpoint()
            if done:
                break
        self.callbacks.fire("on_train_end", ctx)
        final = history[-1] if history else {}
        return {"global_step": self.state.global_step, "train_loss": final.get("loss"), "history": history,
                "tokens_per_second": self.throughput.tokens_per_second(), "mfu": self.throughput.compute_mfu(),
                "train_runtime": time.time() - t_start, "best_metric": self.state.best_metric}

    def _log(self, window_loss, window_steps, grad_norm, t_start, total_steps) -> dict:
        vals = torch.stack([window_loss / max(1, window_steps), grad_norm.reshape(()).float()])
        if self.is_distributed:
            dist.all_reduce(vals)
            vals /= self.world_size
        loss, gn = (float(x) for x in vals.tolist())     # the only host sync of the loop
        self._check_comm()
        self._check_numerical_stability(loss, gn, self.state.global_step)
        self.ema_loss = loss if self.ema_loss is None else 0.99 * self.ema_loss + 0.01 * loss
        self.state.total_loss += loss * max(1, window_steps)
        lr = self.optimizer.param_groups[0]["lr"]
        tps, mfu = self.throughput.tokens_per_second(), self.throughput.compute_mfu()
        step = self.state.global_step
        elapsed = time.time() - t_start
        eta = elapsed / max(1, step) * max(0, total_steps - step)
        ppl = math.exp(min(loss, 20.0)) if math.isfinite(loss) else float("nan")
        line = (f"Epoch {self.state.epoch + 1}/{max(1, self.config.training.num_train_epochs)} | Step {step}/{total_steps}"
                f" | Loss {loss:.4f} | PPL {ppl:.2f} | LR {lr:.3e} | Grad {gn:.3f} | Tok/s {tps:,.0f} | MFU {mfu:.3f}"
                f" | ETA {eta:.0f}s")
        if self.engine is not None and self.is_main and hasattr(self.engine, "memory_summary"):
            line += " | " + self.engine.memory_summary()
        rec = {"step": step, "loss": loss, "ppl": ppl, "lr": lr, "grad_norm": gn, "tokens_per_second": tps, "mfu": mfu}
        for k, v in (getattr(self, "last_preference_metrics", None) or {}).items():
            rec[k] = float(v)          # reward accuracy / margin of the last micro-batch (already a log-time sync)
            line += f" | {k} {rec[k]:.3f}"
        self._ctx.logs = {**rec, "line": line}
        self.callbacks.fire("on_log", self._ctx)
        return rec

    def _check_numerical_stability(self, loss: float | torch.Tensor, grad_norm: float | None = None,
                                   step: int | None = None) -> bool:
        """NaN / Inf loss or gradient norm -> False (and a warning); a finite norm above 1e6 only warns.  Called with
        values that are on the host already (log time).  The update of a step whose gradients are non-finite has been
        skipped on the device by the engine (`EngineConfig.skip_nonfinite`), with no host round trip; this check is
        the visible trace of that, and after `max_nonfinite_windows` consecutive bad log windows training stops with
        GradientOverflowError instead of running on with a diverged model."""
        from ..core.errors import GradientOverflowError
        lv = float(loss) if not isinstance(loss, float) else loss
        where = f" at step {step}" if step is not None else ""
        ok = True
        if not math.isfinite(lv):
            logger.warning("non-finite loss%s: %s", where, lv)
            ok = False
        if grad_norm is not None:
            if not math.isfinite(grad_norm):
                logger.warning("non-finite gradient norm%s", where)
                ok = False
            elif grad_norm > 1e6:
                logger.warning("exploding gradient norm%s: %.2e", where, grad_norm)
        self._bad_windows = 0 if ok else getattr(self, "_bad_windows", 0) + 1
        limit = getattr(self, "max_nonfinite_windows", 5)
        if self._bad_windows >= limit:
            raise GradientOverflowError(f"{self._bad_windows} consecutive log windows with non-finite loss or gradients")
        return ok

    # ------------------------------------------------------------------ evaluation
    def _run_eval(self, dl, compute_metrics=None):
        m = self.evaluate(dl, compute_metrics)
        self._ctx.metrics = m
        self.callbacks.fire("on_evaluate", self._ctx)
        if m["eval_loss"] < self.state.best_metric - self.config.training.early_stopping_threshold:
            self.state.best_metric = m["eval_loss"]
            self.state.patience_counter = 0
            self.save_checkpoint(Path(self.config.training.output_dir) / "checkpoint-best")
        else:
            self.state.patience_counter += 1
        return m

    @torch.no_grad()
    def evaluate(self, eval_dataloader: Iterable, compute_metrics: Callable | None = None) -> Dict[str, float]:
        was_training = self.model.training
        self.model.eval()
        tot = torch.zeros(2, dtype=torch.float64, device=self.device)
        limit = 5 if 0 < self.config.training.max_steps < 100 else None
        for i, batch in enumerate(eval_dataloader):
            if limit is not None and i >= limit:
                break
            batch = self._to_device(batch)
            loss, ntok = self._forward_loss(batch, 1.0)
            n = ntok.double() if torch.is_tensor(ntok) else torch.tensor(float(ntok), device=self.device)
            tot[0] += loss.double() * n
            tot[1] += n
            self.callbacks.fire("on_prediction_step", self._ctx)
        if self.is_distributed:
            t32 = tot.float()
            dist.all_reduce(t32)
            tot = t32.double()
        loss = float(tot[0] / tot[1].clamp(min=1))
        out = {"eval_loss": loss, "eval_perplexity": math.exp(min(loss, 20.0)), "eval_tokens": float(tot[1])}
        if compute_metrics is not None:
            out.update(compute_metrics(out) or {})
        if was_training:
            self.model.train()
        return out

    # ------------------------------------------------------------------ checkpoints
    def _collect_rng_states(self) -> dict:
        return {"python": random.getstate(), "numpy": np.random.get_state(), "torch": torch.get_rng_state(),
                "cuda": [s.cpu() for s in torch.cuda.get_rng_state_all()] if torch.cuda.is_available() else []}

    def _restore_rng_states(self, r: dict) -> None:
        try:
            random.setstate(r["python"])
            np.random.set_state(r["numpy"])
            torch.set_rng_state(r["torch"])
            if torch.cuda.is_available() and r.get("cuda"):
                torch.cuda.set_rng_state_all(r["cuda"])
        except Exception as e:   # a different host / device count: keep going with fresh streams
            logger.warning("could not restore RNG state: %s", e)

    def save_checkpoint(self, path: str | os.PathLike | None = None) -> Path:
        from ..ckpt import save_training_checkpoint
        path = Path(path) if path is not None else Path(self.config.training.output_dir) / \
            f"checkpoint-{self.state.global_step}"
        save_training_checkpoint(self, path)
        self._ctx.logs = {"checkpoint": str(path)}
        self.callbacks.fire("on_save", self._ctx)
        return path

    def load_checkpoint(self, path: str | os.PathLike) -> None:
        from ..ckpt import load_training_checkpoint
        load_training_checkpoint(self, Path(path))

    # ------------------------------------------------------------------ export / cleanup
    def export(self, tokenizer=None, output_dir: str | None = None, fmt: str | None = None) -> Path | None:
        from ..export import export_model
        e = self.config.export
        out = Path(output_dir or e.output_dir)
        fmt = fmt or getattr(e.format, "value", e.format)
        eng = self.engine
        if self.is_distributed:
            dist.barrier()
        if eng is not None and hasattr(eng, "dims") and (eng.tp is not None or eng.pipelined):
            # tensor / pipeline parallel: the weights live on several ranks; all of them take part
            if str(fmt).lower() not in ("safetensors", "hf", "huggingface"):
                raise ValueError(f"export format {fmt!r} of a model-parallel run: export safetensors, then convert "
                                 "the checkpoint on one process")
            from ..ckpt import save_model_parallel_weights
            if self.is_main:
                out.mkdir(parents=True, exist_ok=True)
            dist.barrier()
            save_model_parallel_weights(self, out)
            dist.barrier()
            if self.is_main and tokenizer is not None and hasattr(tokenizer, "save_pretrained"):
                tokenizer.save_pretrained(str(out))
            return out if self.is_main else None
        summon = eng.summon_full_params() if eng is not None and hasattr(eng, "summon_full_params") \
            else contextlib.nullcontext()
        with summon:       # FULL_SHARD keeps only shards between steps; every rank materialises, rank 0 writes
            model = self.model
            if eng is not None and hasattr(eng, "ep_group"):
                # expert parallelism: gathering the experts is a collective of every rank; rank 0 writes the result
                model = _GatheredWeights(self.model, self.model.to_hf_state_dict())
            if not self.is_main:
                return None
            return export_model(model, out, fmt, tokenizer=tokenizer, merge_lora=e.merge_lora)

    def cleanup(self) -> None:
        self.engine = None
        self.optimizer = None
        self.scheduler = None
        self.model = None
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
        if self._own_pg and dist.is_initialized():
            dist.destroy_process_group()
            self._own_pg = False


class _GatheredWeights:
    """Stands in for a model whose full state dict has already been assembled (by a collective of all ranks)."""

    def __init__(self, model, state_dict):
        self._model, self._sd = model, state_dict

    def to_hf_state_dict(self):
        return self._sd

    def hf_config_dict(self):
        return self._model.hf_config_dict()

    def named_parameters(self):
        return self._model.named_parameters()


def create_trainer(config: str | os.PathLike | dict | SOTAConfig, **kw) -> SOTATrainer:
    if isinstance(config, SOTAConfig):
        cfg = config
    elif isinstance(config, dict):
        cfg = SOTAConfig.from_dict(config)
    else:
        cfg = SOTAConfig.from_yaml(config)
    return SOTATrainer(cfg, **kw)


def create_trainer_from_config(config) -> "SOTATrainer":
    """Trainer from an already built `SOTAConfig` (a dict or a YAML path is accepted too)."""
    from ..config.sota_config import SOTAConfig
    if isinstance(config, dict):
        config = SOTAConfig.from_dict(config)
    elif isinstance(config, (str, os.PathLike)):
        config = SOTAConfig.from_yaml(config)
    return SOTATrainer(config)


from ..metrics import is_distributed as metrics_is_distributed  # noqa: E402,F401  (alias of the reference's trainer module)
