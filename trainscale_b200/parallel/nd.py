"""Glue between SOTATrainer and the tensor / pipeline / context parallel engines."""
from __future__ import annotations

import torch
import torch.distributed as dist

from .mesh import create_parallel_dims_from_config


class NDEngine:
    """Wraps the flat engine of the data-parallel sub-group plus the model-parallel contexts; exposes the same
    backward / step / param_groups surface so that SOTATrainer's loop is unchanged."""

    def __init__(self, trainer, strategy: str):
        from .flat_engine import EngineConfig, FlatShardedEngine
        cfg = trainer.config
        self.dims = create_parallel_dims_from_config(cfg.distributed)
        self.strategy = strategy
        model = trainer.model
        p = cfg.distributed.parallel
        if self.dims.enabled("tp"):
            from . import tp as TP
            heap = None
            ctx = TP.TPContext.from_group(self.dims.group("tp"), p.sp, "nccl", heap)
            if p.sp:
                raise NotImplementedError("sequence-parallel training through SOTATrainer: use parallel/tp.py directly")
            TP.shard_model_for_tensor_parallel(model, ctx)
            self.tp = ctx
        if self.dims.enabled("cp"):
            g = self.dims.group("cp")
            for layer in model.model.layers:
                attn = getattr(layer.self_attn, "inner", layer.self_attn)
                attn.cp_group = g
            self.cp_group = g
        if self.dims.enabled("pp"):
            raise NotImplementedError("pipeline training through SOTATrainer: use parallel/pp.PipelineRuntime directly")
        ec = EngineConfig(sharding_strategy="SHARD_GRAD_OP", param_dtype=trainer.dtype,
                          gradient_accumulation_steps=cfg.training.gradient_accumulation_steps,
                          max_grad_norm=cfg.optimizer.max_grad_norm, lr=cfg.optimizer.learning_rate,
                          betas=tuple(cfg.optimizer.betas), eps=cfg.optimizer.eps, weight_decay=cfg.optimizer.weight_decay,
                          comm="nccl")
        # gradients are averaged over every rank that saw different tokens of the same weights: dp x cp
        self.flat = FlatShardedEngine(model, ec, process_group=self.dims.group("dp_cp"), device=trainer.device)
        self.param_groups = self.flat.param_groups
        self.cfg = ec

    def shard_batch(self, batch: dict) -> dict:
        if self.dims.enabled("cp"):
            from .cp import shard_inputs
            return shard_inputs(batch, self.dims.size("cp"), self.dims.local_rank("cp"))
        return batch

    def backward(self, loss):
        return self.flat.backward(loss)

    def step(self, lr=None):
        return self.flat.step(lr)

    @property
    def micro_step(self):
        return self.flat.micro_step

    @micro_step.setter
    def micro_step(self, v):
        self.flat.micro_step = v

    def state_dict(self):
        return self.flat.state_dict()

    def load_state_dict(self, sd):
        self.flat.load_state_dict(sd)

    def memory_summary(self):
        return self.dims.describe() + " | " + self.flat.memory_summary()

    @property
    def units(self):
        return self.flat.units


def build_nd_engine(trainer, strategy: str) -> NDEngine:
    return NDEngine(trainer, strategy)
