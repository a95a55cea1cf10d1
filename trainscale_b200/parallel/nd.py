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
        self.trainer = trainer
        model = trainer.model
        p = cfg.distributed.parallel
        self.tp = None
        self.pipelined = False
        gas = max(1, cfg.training.gradient_accumulation_steps)
        overlap = True
        if self.dims.enabled("tp"):
            from . import tp as TP
            heap = None
            if cfg.distributed.comm in ("auto", "fused") and torch.device(trainer.device).type == "cuda":
                # all-gather->GEMM and GEMM->reduce-scatter inside one kernel over the tp group's peer memory
                from .symm import SymmetricHeap
                heap = SymmetricHeap.try_create(self.dims.group("tp"), trainer.device)
            ctx = TP.TPContext.from_group(self.dims.group("tp"), p.sp, "fused" if heap is not None else "nccl", heap)
            TP.shard_model_for_tensor_parallel(model, ctx)
            self.tp = ctx
            if p.sp:
                # token-sharded residual stream between blocks (see LlamaModel.forward); the norm-weight gradients
                # are summed over the tp group after backward, before the data-parallel reduction
                model.model.sp_ctx = ctx
                overlap = False
        self.cp_balancer = "head_tail"
        if self.dims.enabled("cp"):
            g = self.dims.group("cp")
            # cp_balancer: head_tail (default) = exact ring attention on causally balanced shards;
            # ulysses / contiguous = all-to-all between token shards and head shards (heads must divide by cp)
            self.cp_balancer = (getattr(p, "cp_balancer", None) or "head_tail").lower()
            if self.cp_balancer not in ("head_tail", "ulysses", "contiguous"):
                raise ValueError(f"cp_balancer {self.cp_balancer!r}: the trainer supports head_tail (ring) and ulysses")
            mode = "ring" if self.cp_balancer == "head_tail" else "ulysses"
            for layer in model.model.layers:
                attn = getattr(layer.self_attn, "inner", layer.self_attn)
                attn.cp_group, attn.cp_mode = g, mode
            self.cp_group = g
        opt_model = model
        if self.dims.enabled("pp"):
            from . import pp as PP
            P, stage = self.dims.size("pp"), self.dims.local_rank("pp")
            self.pp_ranks = self.dims.group_ranks("pp")
            self.stage_module = PP.split_model_into_stages(model, P, stage)
            mine = {id(l) for l in self.stage_module.layers}
            for i, layer in enumerate(model.model.layers):     # other stages' layers are dropped on this rank
                if id(layer) not in mine:
                    model.model.layers[i] = torch.nn.Identity()
            # one communicator per direction (activations down the pipeline, gradients up): see PipelineRuntime
            world = list(range(dist.get_world_size()))
            self._pp_act_group, self._pp_grad_group = dist.new_group(world), dist.new_group(world)
            self.runtime = PP.PipelineRuntime(self.stage_module, stage, P, group=self._pp_act_group,
                                              schedule=p.pp_schedule, grad_group=self._pp_grad_group,
                                              prev_rank=self.pp_ranks[stage - 1] if stage > 0 else None,
                                              next_rank=self.pp_ranks[stage + 1] if stage < P - 1 else None)
            self.pp_microbatches = int(p.pp_microbatches or 0)
            self.pipelined = True
            if self.tp is not None and p.sp:
                self.stage_module.sp_ctx = self.tp     # token-sharded activations inside and between the stages
            opt_model = self.stage_module
            overlap = False            # the schedule interleaves micro-batches: reduce once, in step()
            gas = gas * max(1, self.pp_microbatches or 1)
        ec = EngineConfig(sharding_strategy="SHARD_GRAD_OP", param_dtype=trainer.dtype,
                          gradient_accumulation_steps=gas, overlap_grad_reduce=overlap,
                          max_grad_norm=cfg.optimizer.max_grad_norm, lr=cfg.optimizer.learning_rate,
                          betas=tuple(cfg.optimizer.betas), eps=cfg.optimizer.eps, weight_decay=cfg.optimizer.weight_decay,
                          comm="nccl")
        fc = dict(cfg.distributed.fsdp_config or {})
        gd = str(fc.get("grad_dtype", "")).lower()
        if gd in ("bf16", "bfloat16"):
            ec.grad_dtype = torch.bfloat16    # halves the gradient buffers; every micro-batch's addition rounds to bf16
        elif gd in ("fp32", "float32"):
            ec.grad_dtype = torch.float32
        if self.pipelined and ec.grad_dtype is None:
            ec.grad_dtype = torch.float32     # gradients of several micro-batches accumulate in the buffers
        # gradients are averaged over every rank that saw different tokens of the same weights: dp x cp
        self.flat = FlatShardedEngine(opt_model, ec, process_group=self.dims.group("dp_cp"), device=trainer.device,
                                      solo=self.dims.size("dp_cp") == 1)
        if self.pipelined:
            self.flat.norm_groups.append(self.dims.group("pp"))
        if self.tp is not None:
            # sharded weights contribute once per shard, replicated ones (norms, embeddings, head) once in total
            self.flat.norm_groups.append(self.dims.group("tp"))
            self.flat.replicated_params = [q for n, q in opt_model.named_parameters()
                                           if q.dim() == 1 or "embed_tokens" in n or "lm_head" in n]
            self.flat.replica_factor = self.dims.size("tp")
        self.param_groups = self.flat.param_groups
        self.cfg = ec

    # ------------------------------------------------------------------ pipeline step
    def forward_backward(self, batch: dict, loss_scale: float):
        """Runs the pipeline schedule over the micro-batches of `batch`; returns (loss, token count) on every stage
        (the last stage's values are broadcast over the pipeline group for logging)."""
        from . import pp as PP
        B, S = batch["input_ids"].shape
        M = self.pp_microbatches or B
        if B % M != 0:
            raise ValueError(f"batch of {B} sequences does not split into {M} pipeline micro-batches")
        mbs = PP.split_into_microbatches({k: v for k, v in batch.items() if torch.is_tensor(v)}, M)
        H = self.stage_module.config.hidden_size
        sp = self.tp.size if (self.tp is not None and self.tp.sequence_parallel) else 1
        act_shape = (B // M, S // sp, 2 * H)      # with sequence parallelism a rank exchanges only its token shard
        dev = batch["input_ids"].device
        loss = self.runtime.train_step(mbs, act_shape, self.trainer.dtype, dev, extra_scale=loss_scale)
        lc = self.trainer.config.loss
        labels = batch.get("labels", batch["input_ids"])
        ntok = (labels[..., 1:] != lc.ignore_index).sum()
        out = torch.zeros(1, dtype=torch.float32, device=dev)
        if loss is not None:
            out[0] = loss.float()
        dist.broadcast(out, src=self.pp_ranks[-1], group=self.dims.group("pp"))
        if getattr(self.stage_module, "_tied", False) or (self.stage_module.first and
                                                          self.stage_module.config.tie_word_embeddings):
            PP.allreduce_tied_embedding_grads(self.stage_module, self.dims.group("pp"), self.pp_ranks[0],
                                              self.pp_ranks[-1])
        if self.tp is not None and self.tp.sequence_parallel:
            from . import tp as TP
            TP.allreduce_sequence_parallel_grads(self.stage_module, self.tp)
        self.flat.micro_step += 1
        return out[0], ntok

    def shard_batch(self, batch: dict) -> dict:
        if self.dims.enabled("cp"):
            from .cp import shard_inputs
            return shard_inputs(batch, self.dims.size("cp"), self.dims.local_rank("cp"), self.cp_balancer)
        return batch

    def backward(self, loss):
        sync = self.flat.backward(loss)
        if self.tp is not None and self.tp.sequence_parallel:
            from . import tp as TP
            TP.allreduce_sequence_parallel_grads(self.trainer.model, self.tp)
        return sync

    def step(self, lr=None):
        return self.flat.step(lr)

    def zero_grad(self):
        self.flat.zero_grad()

    def check_comm_status(self) -> None:
        """Status words of every symmetric heap this engine's kernels wait on (tensor-parallel GEMMs, context-parallel
        K/V exchange, data-parallel reduction); raises CommunicationError when a peer wait ran out."""
        heaps = []
        if self.tp is not None and getattr(self.tp, "heap", None) is not None:
            heaps.append(self.tp.heap)
        if self.dims.enabled("cp"):
            from .cp import _PeerKV
            heaps.extend(h for h in _PeerKV._heaps.values() if h is not None)
        for h in heaps:
            h.check_status()
        self.flat.check_comm_status()

    @property
    def micro_step(self):
        return self.flat.micro_step

    @micro_step.setter
    def micro_step(self, v):
        self.flat.micro_step = v

    def mesh_coordinates(self) -> dict:
        """{axis: [rank on that axis, size of that axis]} for the axes that decide WHICH parameters this rank's
        optimizer shard holds (tp: a slice of every projection, pp: a stage's layers) and for the data axis the shard
        is cut along."""
        return {a: [self.dims.local_rank(a), self.dims.size(a)] for a in ("tp", "pp", "dp_cp")}

    def state_dict(self):
        sd = self.flat.state_dict()
        sd["mesh"] = self.mesh_coordinates()
        return sd

    def load_state_dict(self, sd):
        self.flat.load_state_dict(sd)

    def memory_summary(self):
        return self.dims.describe() + " | " + self.flat.memory_summary()

    @property
    def units(self):
        return self.flat.units


def build_nd_engine(trainer, strategy: str) -> NDEngine:
    return NDEngine(trainer, strategy)
