"""Pipeline parallelism for arbitrary `nn.Module` stages, under the reference's class names.

`parallel/pp.py` holds the schedule generators and the fast runtime for the framework decoder (packed activations,
deferred weight-gradient GEMMs).  This module is the general API of
data_pipeline/trainer/distributed/pipeline_parallel.py:144-2619: `PipelineConfig`, `PipelineStage`,
`VirtualPipelineStage`, the schedule classes (`GPipeSchedule`, `OneFOneBSchedule`, `InterleavedOneFOneBSchedule`,
`ZeroBubbleSchedule`, `ChimeraSchedule`), `PipelineParallel`, `P2PCommunicator`, `ActivationMemoryManager`,
`TensorPool`, `GradientBucket`, `CheckpointFunction`, stage balancing and a profiler.

One executor serves every schedule: a schedule is a per-worker list of (op, micro-batch, chunk) actions, a worker runs
its list in order, and an action runs when its inputs exist.  With all stages in one process (`stages` holds every
virtual stage) the workers are stepped round-robin; with one worker per rank the same lists drive point-to-point
transfers whose receive order on each link is derived from the sender's list, so no tags are needed.
"""
from __future__ import annotations

import contextlib
import time
from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, NamedTuple, Sequence

import torch
import torch.distributed as dist

from ..utils.refargs import ANY, reference_kwargs
import torch.nn as nn

from ..core.types import Err, Ok, Result
from . import pp as PP
from .pp import Action, B_OP, F_OP, W_OP


class PipelineError(Enum):
    INVALID_CONFIG = "invalid_config"
    COMMUNICATION = "communication"
    DEADLOCK = "deadlock"
    SHAPE_MISMATCH = "shape_mismatch"


def unwrap_or_raise(result, context: str = ""):
    if result.is_ok():
        return result.unwrap()
    raise RuntimeError(f"{context}: {result}")


class ScheduleType(Enum):
    GPIPE = "gpipe"
    ONE_F_ONE_B = "1f1b"
    INTERLEAVED_ONE_F_ONE_B = "interleaved"
    ZERO_BUBBLE = "zero_bubble"
    CHIMERA = "chimera"


class PrecisionMode(Enum):
    FP32 = "fp32"
    BF16 = "bf16"
    FP16 = "fp16"


@dataclass
class MemoryConfig:
    enable_activation_checkpointing: bool = False
    enable_tensor_pool: bool = True
    pool_max_bytes: int = 4 * 2 ** 30
    offload_activations: bool = False


@dataclass
class CommunicationConfig:
    async_p2p: bool = True
    static_shapes: bool = True            # shape / dtype of a link's tensors is sent once, then assumed
    timeout_seconds: float = 1800.0


@dataclass
class PrecisionConfig:
    mode: PrecisionMode = PrecisionMode.BF16
    enable_dynamic_loss_scaling: bool = False
    initial_loss_scale: float = 65536.0
    growth_factor: float = 2.0
    backoff_factor: float = 0.5
    growth_interval: int = 2000


@dataclass
class ProfilingConfig:
    enabled: bool = False
    record_stage_times: bool = True


@dataclass
class PipelineConfig:
    num_stages: int = 4
    num_virtual_stages: int = 1
    num_microbatches: int = 8
    gradient_accumulation_steps: int = 1
    schedule: ScheduleType = ScheduleType.ONE_F_ONE_B
    memory: MemoryConfig = field(default_factory=MemoryConfig)
    communication: CommunicationConfig = field(default_factory=CommunicationConfig)
    precision: PrecisionConfig = field(default_factory=PrecisionConfig)
    profiling: ProfilingConfig = field(default_factory=ProfilingConfig)
    enable_cuda_graphs: bool = False
    enable_sequence_parallelism: bool = False
    enable_expert_parallelism: bool = False
    debug_mode: bool = False

    def __post_init__(self) -> None:
        if isinstance(self.schedule, str):
            self.schedule = ScheduleType(self.schedule.lower())
        if self.num_stages < 1 or self.num_virtual_stages < 1 or self.gradient_accumulation_steps < 1:
            raise ValueError("num_stages, num_virtual_stages and gradient_accumulation_steps must be positive")
        if self.num_microbatches < 1:
            raise ValueError("num_microbatches must be positive")
        if self.schedule is ScheduleType.INTERLEAVED_ONE_F_ONE_B and self.num_microbatches % self.num_stages:
            raise ValueError("the interleaved schedule needs num_microbatches divisible by num_stages")
        if self.schedule is ScheduleType.CHIMERA and (self.num_microbatches % 2 or self.num_stages % 2):
            raise ValueError("Chimera needs an even number of stages and of micro-batches")

    @property
    def total_virtual_stages(self) -> int:
        return self.num_stages * self.num_virtual_stages


# ------------------------------------------------------------------------------------------------ process context
class DistributedContext:
    """Where this process sits in the pipeline group (a sub-group of the job, or the whole world)."""

    def __init__(self, group=None, ranks: Sequence[int] | None = None):
        self.group = group
        self._ranks = list(ranks) if ranks is not None else None

    @property
    def is_distributed(self) -> bool:
        return dist.is_available() and dist.is_initialized() and self.pipeline_parallel_size > 1

    @property
    def world_size(self) -> int:
        return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1

    @property
    def rank(self) -> int:
        return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0

    @property
    def local_rank(self) -> int:
        import os
        return int(os.environ.get("LOCAL_RANK", "0"))

    @property
    def pipeline_parallel_size(self) -> int:
        if not (dist.is_available() and dist.is_initialized()):
            return 1
        return len(self._ranks) if self._ranks is not None else dist.get_world_size(self.group)

    @property
    def pipeline_parallel_rank(self) -> int:
        if not (dist.is_available() and dist.is_initialized()):
            return 0
        return self._ranks.index(self.rank) if self._ranks is not None else dist.get_rank(self.group)

    def initialize_pipeline_group(self, ranks: Sequence[int], backend: str | None = None) -> "DistributedContext":
        """Collective over the whole job: creates the group of `ranks` (every rank must call it with the same list);
        `backend`: of the new group (that of the default group when None)."""
        self._ranks = list(ranks)
        self.group = dist.new_group(self._ranks, backend=backend) if dist.is_initialized() else None
        return self

    def global_rank_of(self, pipeline_rank: int) -> int:
        if self._ranks is not None:
            return self._ranks[pipeline_rank]
        return dist.get_global_rank(self.group, pipeline_rank) if self.group is not None else pipeline_rank

    def get_prev_rank(self, pipeline_rank: int | None = None) -> int | None:
        r = self.pipeline_parallel_rank if pipeline_rank is None else pipeline_rank
        return self.global_rank_of(r - 1) if r > 0 else None

    def get_next_rank(self, pipeline_rank: int | None = None) -> int | None:
        r = self.pipeline_parallel_rank if pipeline_rank is None else pipeline_rank
        return self.global_rank_of(r + 1) if r < self.pipeline_parallel_size - 1 else None


_DEFAULT_CTX = DistributedContext()


def get_pipeline_parallel_rank() -> int:
    return _DEFAULT_CTX.pipeline_parallel_rank


def get_pipeline_parallel_world_size() -> int:
    return _DEFAULT_CTX.pipeline_parallel_size


# ------------------------------------------------------------------------------------------------ memory helpers
class TensorPool:
    """Exact-shape recycling of communication / activation buffers."""

    def __init__(self, device: torch.device | str = "cpu", max_bytes: int = 4 * 2 ** 30):
        self.device, self.max_bytes = torch.device(device), max_bytes
        self._free: dict[tuple, list[torch.Tensor]] = {}
        self._bytes = 0
        self._stats = {"allocations": 0, "reuses": 0, "returns": 0}

    def allocate(self, shape: Sequence[int], dtype: torch.dtype = torch.float32, zero: bool = False) -> torch.Tensor:
        key = (tuple(shape), dtype)
        lst = self._free.get(key)
        if lst:
            t = lst.pop()
            self._bytes -= t.numel() * t.element_size()
            self._stats["reuses"] += 1
        else:
            t = torch.empty(key[0], dtype=dtype, device=self.device)
            self._stats["allocations"] += 1
        return t.zero_() if zero else t

    def deallocate(self, tensor: torch.Tensor) -> None:
        nb = tensor.numel() * tensor.element_size()
        if self._bytes + nb > self.max_bytes or tensor.requires_grad:
            return
        self._free.setdefault((tuple(tensor.shape), tensor.dtype), []).append(tensor.detach())
        self._bytes += nb
        self._stats["returns"] += 1

    def clear(self) -> None:
        self._free.clear()
        self._bytes = 0

    def stats(self) -> dict[str, int]:
        return dict(self._stats, cached_bytes=self._bytes)


class ActivationMemoryManager:
    """Holds what a stage must keep between the forward and the backward of a micro-batch, and accounts for it."""

    def __init__(self, config: MemoryConfig | None = None, device: torch.device | str = "cpu"):
        self.config = config or MemoryConfig()
        self.device = torch.device(device)
        self._stash: dict[tuple, Any] = {}
        self._cur = 0
        self._peak = 0

    @staticmethod
    def _nbytes(obj) -> int:
        if torch.is_tensor(obj):
            return obj.numel() * obj.element_size()
        if isinstance(obj, (tuple, list)):
            return sum(ActivationMemoryManager._nbytes(o) for o in obj)
        return 0

    @staticmethod
    def _key(key, microbatch_id, stage_id):
        if stage_id is not None or microbatch_id is not None:
            return (key if stage_id is None else stage_id, microbatch_id)
        return key

    def stash_activation(self, key: "tuple | int | None" = None, value: Any = None, activation: Any = None, *,
                         stage_id: int | None = None, microbatch_id: int | None = None) -> None:
        """`stash_activation(key, value)`, or `(stage_id, microbatch_id, activation)`: the key is then the pair."""
        if activation is not None or stage_id is not None or microbatch_id is not None:
            if activation is None:                       # (stage_id, microbatch_id, activation) positionally
                raise TypeError("stash_activation(stage_id, microbatch_id, activation) needs the activation")
            if stage_id is None and microbatch_id is None:
                key, value = (key, value), activation
            else:
                key, value = self._key(key, microbatch_id if microbatch_id is not None else value, stage_id), activation
        self._stash[key] = value
        self._cur += self._nbytes(value)
        self._peak = max(self._peak, self._cur)

    def pop_activation(self, key: "tuple | int | None" = None, microbatch_id: int | None = None, *,
                       stage_id: int | None = None) -> Any:
        """`pop_activation(key)` or `pop_activation(stage_id, microbatch_id)`."""
        key = self._key(key, microbatch_id, stage_id)
        v = self._stash.pop(key)
        self._cur -= self._nbytes(v)
        return v

    def has(self, key: tuple) -> bool:
        return key in self._stash

    # ---- per-micro-batch, named storage (data_pipeline/trainer/distributed/zbpp.py:458-495)
    def store_activation(self, microbatch_id: int, name: str, tensor: torch.Tensor, limit_bytes: int | None = None) -> None:
        """Keep `tensor` under (microbatch_id, name).  When the stash would exceed `limit_bytes` the tensor is kept on
        the host instead (pinned when it comes from a GPU) and comes back in `retrieve_activation`."""
        nb = self._nbytes(tensor)
        if limit_bytes is not None and self._cur + nb > limit_bytes and tensor.is_cuda:
            host = torch.empty(tensor.shape, dtype=tensor.dtype, pin_memory=True)
            host.copy_(tensor, non_blocking=True)
            tensor = (host, tensor.device, torch.cuda.current_stream().record_event())
            nb = 0                                         # host copies do not count against the device stash
        self._stash[("mb", microbatch_id, name)] = tensor
        self._cur += nb
        self._peak = max(self._peak, self._cur)

    def retrieve_activation(self, microbatch_id: int, name: str):
        v = self._stash.get(("mb", microbatch_id, name))
        if isinstance(v, tuple) and len(v) == 3 and torch.is_tensor(v[0]):
            host, dev, ev = v
            ev.synchronize()
            return host.to(dev, non_blocking=True)
        return v

    def release_activation(self, microbatch_id: int) -> int:
        """Drop everything stored for the micro-batch (after its weight-gradient pass); returns how many entries."""
        keys = [k for k in self._stash if len(k) == 3 and k[0] == "mb" and k[1] == microbatch_id]
        for k in keys:
            v = self._stash.pop(k)
            self._cur -= self._nbytes(v) if torch.is_tensor(v) else 0
        return len(keys)

    def clear(self) -> None:
        self._stash.clear()
        self._cur = 0

    @property
    def peak_memory_mb(self) -> float:
        return self._peak / 2 ** 20

    @property
    def current_memory_mb(self) -> float:
        return self._cur / 2 ** 20


class TensorMetadata(NamedTuple):
    shape: tuple
    dtype: torch.dtype
    requires_grad: bool = True


_DTYPES = [torch.float32, torch.bfloat16, torch.float16, torch.float64, torch.int64, torch.int32, torch.uint8, torch.bool]


# ------------------------------------------------------------------------------------------------ point to point
class P2PCommunicator:
    """Sends / receives of activations and their gradients between pipeline ranks.  With `static_shapes` the shape and
    dtype of a link's tensor travel once (a small int64 header) and are assumed afterwards."""

    def __init__(self, ctx: "DistributedContext | CommunicationConfig | PipelineConfig | None" = None,
                 device: torch.device | str = "cpu", config: CommunicationConfig | None = None,
                 pool: TensorPool | None = None, *, group=None):
        """`P2PCommunicator(ctx, device, config, pool)`, or the reference's `(config, device, group)` with the
        communication (or whole pipeline) configuration first and the process group of the pipeline
        (data_pipeline/trainer/distributed/pipeline_parallel.py:629)."""
        if isinstance(ctx, (CommunicationConfig, PipelineConfig)):
            if config is not None and not isinstance(config, CommunicationConfig):
                group, config = config, None                             # positional (config, device, group)
            config, ctx = ctx, None
        if isinstance(config, PipelineConfig):
            config = config.communication
        if group is not None:
            ctx = DistributedContext(group)
        self.ctx = ctx or _DEFAULT_CTX
        self.group = self.ctx.group
        self.device = torch.device(device)
        self.config = config or CommunicationConfig()
        self.pool = pool
        self._pending: list = []
        self._meta: dict[tuple, TensorMetadata] = {}
        self.bytes_sent = self.bytes_received = 0

    def _send_meta(self, t: torch.Tensor, dst: int, tag_key: tuple) -> None:
        if self.config.static_shapes and tag_key in self._meta:
            return
        hdr = torch.zeros(10, dtype=torch.int64)
        hdr[0], hdr[1] = t.dim(), _DTYPES.index(t.dtype)
        hdr[2:2 + t.dim()] = torch.tensor(list(t.shape), dtype=torch.int64)
        hdr = hdr.to(self.device)
        # never block in a send: two ranks that open a link towards each other at the same moment would deadlock
        self._pending.append((dist.isend(hdr, dst, group=self.ctx.group), hdr))
        self._meta[tag_key] = TensorMetadata(tuple(t.shape), t.dtype)

    def _recv_meta(self, src: int, tag_key: tuple) -> TensorMetadata:
        if self.config.static_shapes and tag_key in self._meta:
            return self._meta[tag_key]
        hdr = torch.zeros(10, dtype=torch.int64, device=self.device)
        dist.recv(hdr, src, group=self.ctx.group)
        hdr = hdr.cpu()
        nd = int(hdr[0])
        md = TensorMetadata(tuple(int(x) for x in hdr[2:2 + nd]), _DTYPES[int(hdr[1])])
        self._meta[tag_key] = md
        return md

    def _as_result(self, fn, *args):
        """The reference's spelling (`dst_rank=` / `src_rank=`, integer `tag=`) returns Ok(...) / Err(...) instead of raising."""
        from ..core.types import Err, Ok
        if not (dist.is_available() and dist.is_initialized()):
            return Err(RuntimeError(f"{PipelineError.COMMUNICATION.value}: torch.distributed is not initialised"))
        try:
            return Ok(fn(*args))
        except (RuntimeError, ValueError) as e:
            return Err(RuntimeError(f"{PipelineError.COMMUNICATION.value}: {e}"))

    @staticmethod
    def _kind(kind, tag):
        return kind if tag is None else f"tag{int(tag)}"

    def send_async(self, tensor: torch.Tensor, dst: int | None = None, kind: str = "act", *, dst_rank: int | None = None,
                   tag: int | None = None):
        if dst_rank is not None or tag is not None:
            return self._as_result(self.send_async, tensor, dst_rank if dst_rank is not None else dst, self._kind(kind, tag))
        t = tensor.detach().contiguous()
        self._send_meta(t, dst, ("s", dst, kind))
        w = dist.isend(t, dst, group=self.ctx.group)
        self._pending.append((w, t))          # keep the buffer alive until the send completes
        self.bytes_sent += t.numel() * t.element_size()
        return w

    def recv_async(self, src: int | None = None, kind: str = "act", meta: TensorMetadata | None = None, *,
                   src_rank: int | None = None, tag: int | None = None):
        if src_rank is not None or tag is not None:
            return self._as_result(self.recv_async, src_rank if src_rank is not None else src, self._kind(kind, tag), meta)
        md = meta or self._recv_meta(src, ("r", src, kind))
        buf = self.pool.allocate(md.shape, md.dtype) if self.pool is not None else \
            torch.empty(md.shape, dtype=md.dtype, device=self.device)
        w = dist.irecv(buf, src, group=self.ctx.group)
        self.bytes_received += buf.numel() * buf.element_size()
        return buf, w

    def send_sync(self, tensor: torch.Tensor, dst: int | None = None, kind: str = "act", *, dst_rank: int | None = None):
        if dst_rank is not None:
            return self._as_result(self.send_sync, tensor, dst_rank, kind)
        self.send_async(tensor, dst, kind).wait()

    def recv_sync(self, src: int | None = None, kind: str = "act", meta: TensorMetadata | None = None, *,
                  src_rank: int | None = None):
        if src_rank is not None:
            return self._as_result(self.recv_sync, src_rank, kind, meta)
        buf, w = self.recv_async(src, kind, meta)
        w.wait()
        return buf

    def wait_all(self) -> None:
        for w, _ in self._pending:
            w.wait()
        self._pending.clear()

    # ---- neighbour-addressed form (data_pipeline/trainer/distributed/zbpp.py:691-830): the peer is implied by the
    # direction, a missing neighbour (first / last stage) makes the call a no-op that returns None
    @property
    def stage_id(self) -> int:
        return self.ctx.pipeline_parallel_rank

    @property
    def prev_rank(self) -> int | None:
        return self.ctx.get_prev_rank()

    @property
    def next_rank(self) -> int | None:
        return self.ctx.get_next_rank()

    def send_activation_async(self, tensor: torch.Tensor, microbatch_id: int = 0):
        return None if self.next_rank is None else self.send_async(tensor, self.next_rank, "act")

    def recv_activation_async(self, shape=None, dtype: torch.dtype | None = None, microbatch_id: int = 0):
        """(work, buffer).  The shape travels in the link's header (once with `static_shapes`); `shape` / `dtype`, when
        given, are checked against it."""
        return (None, torch.empty(0)) if self.prev_rank is None else self._recv_checked(self.prev_rank, "act", shape, dtype)

    def _recv_checked(self, src: int, kind: str, shape, dtype):
        buf, w = self.recv_async(src, kind)
        if (shape is not None and tuple(shape) != tuple(buf.shape)) or (dtype is not None and dtype != buf.dtype):
            raise ValueError(f"expected {tuple(shape) if shape is not None else '?'} {dtype} from rank {src}, "
                             f"the sender announced {tuple(buf.shape)} {buf.dtype}")
        self._pending.append((w, buf))
        return w, buf

    def send_grad_async(self, grad: torch.Tensor, microbatch_id: int = 0):
        return None if self.prev_rank is None else self.send_async(grad, self.prev_rank, "grad")

    def recv_grad_async(self, shape=None, dtype: torch.dtype | None = None, microbatch_id: int = 0):
        return (None, torch.empty(0)) if self.next_rank is None else self._recv_checked(self.next_rank, "grad", shape, dtype)

    synchronize_pending = wait_all


class GradientBucket:
    """Flat gradient bucket of a stage, all-reduced over its data-parallel group in one call."""

    @reference_kwargs(max_size_bytes="capacity_bytes")
    def __init__(self, capacity_bytes: int = 25 * 2 ** 20, dtype: torch.dtype = torch.float32, device=None):
        if not isinstance(dtype, torch.dtype):                  # (max_size_bytes, device, dtype)
            dtype, device = (device if isinstance(device, torch.dtype) else torch.float32), dtype
        self.capacity, self.dtype, self.device = capacity_bytes, dtype, device
        self._items: list[tuple[torch.Tensor, torch.Tensor]] = []
        self._bytes = 0

    def add_gradient(self, param: torch.Tensor, grad: torch.Tensor) -> bool:
        """True when the bucket is full after this addition (reduce it now)."""
        self._items.append((param, grad))
        self._bytes += grad.numel() * grad.element_size()
        return self._bytes >= self.capacity

    def reduce(self, group=None, average: bool = True) -> None:
        if not self._items:
            return
        flat = torch.cat([g.reshape(-1).to(self.dtype) for _, g in self._items])
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(flat, group=group)
            if average:
                flat /= dist.get_world_size(group)
        off = 0
        for _, g in self._items:
            g.copy_(flat[off:off + g.numel()].view_as(g))
            off += g.numel()
        self._items.clear()
        self._bytes = 0


class CheckpointFunction(torch.autograd.Function):
    """Recompute-in-backward for one stage call: keeps the inputs and the RNG state, drops everything else."""

    @staticmethod
    def forward(ctx, run_function, preserve_rng_state, *args):
        """`apply(run_function, preserve_rng_state, *inputs)`; an int in the second place is the number of leading
        `args` that are inputs (the rest are ignored), with the RNG state kept."""
        run_fn = run_function
        n_inputs = len(args) if isinstance(preserve_rng_state, bool) else int(preserve_rng_state)
        ctx.run_fn = run_fn
        ctx.preserve_rng = preserve_rng_state is not False
        ctx.cpu_rng = torch.get_rng_state() if ctx.preserve_rng else None
        ctx.cuda_rng = torch.cuda.get_rng_state() if ctx.preserve_rng and torch.cuda.is_available() and any(
            torch.is_tensor(a) and a.is_cuda for a in args) else None
        ctx.save_for_backward(*[a for a in args[:n_inputs] if torch.is_tensor(a)])
        ctx.layout = [torch.is_tensor(a) for a in args[:n_inputs]]
        ctx.consts = [a for a in args[:n_inputs] if not torch.is_tensor(a)]
        with torch.no_grad():
            return run_fn(*args[:n_inputs])

    @staticmethod
    def backward(ctx, *grad_outputs):
        saved, consts = list(ctx.saved_tensors), list(ctx.consts)
        inputs = [(saved.pop(0).detach().requires_grad_(True) if is_t else consts.pop(0)) for is_t in ctx.layout]
        for x in inputs:
            if torch.is_tensor(x) and not x.is_floating_point():
                x.requires_grad_(False)
        devs = [torch.cuda.current_device()] if ctx.cuda_rng is not None else []
        with torch.random.fork_rng(devices=devs, enabled=ctx.preserve_rng):
            if ctx.preserve_rng:
                torch.set_rng_state(ctx.cpu_rng)
            if ctx.cuda_rng is not None:
                torch.cuda.set_rng_state(ctx.cuda_rng)
            with torch.enable_grad():
                out = ctx.run_fn(*inputs)
        outs = out if isinstance(out, (tuple, list)) else (out,)
        pairs = [(o, g) for o, g in zip(outs, grad_outputs) if torch.is_tensor(o) and o.requires_grad and g is not None]
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        grads = tuple(x.grad if torch.is_tensor(x) and x.requires_grad else None for x in inputs)
        return (None, None) + grads


@reference_kwargs({"preserve_rng_state": ANY}, function="module")
def selective_checkpoint(module, *args, enabled: bool = True):
    """Run `module(*args)` under recompute-in-backward when `enabled` (parameters get their gradients in backward).
    `module` may be any callable (`function=` in the reference's spelling)."""
    if not enabled or not torch.is_grad_enabled():
        return module(*args)
    # a dummy that requires grad makes autograd call backward even when no input does (first stage: token ids)
    dev = next(module.parameters()).device if isinstance(module, nn.Module) and any(True for _ in module.parameters()) \
        else next((a.device for a in args if torch.is_tensor(a)), torch.device("cpu"))
    anchor = torch.zeros((), requires_grad=True, device=dev)
    return CheckpointFunction.apply(lambda *a: module(*a[:-1]), len(args) + 1, *args, anchor)


# ------------------------------------------------------------------------------------------------ stages
class PipelineStage(nn.Module):
    """One stage: a module plus its place in the pipeline, optional recompute, and forward timing."""

    def __init__(self, module: nn.Module, stage_id: int, num_stages: int, device: torch.device | str | None = None,
                 checkpoint_activations: "bool | PipelineConfig" = False, *, config: "PipelineConfig | None" = None):
        """`config`: the pipeline configuration; activations are recomputed when its memory section asks for it."""
        super().__init__()
        if isinstance(checkpoint_activations, PipelineConfig):           # (module, stage_id, num_stages, device, config)
            config, checkpoint_activations = checkpoint_activations, False
        if config is not None:
            checkpoint_activations = checkpoint_activations or bool(config.memory.enable_activation_checkpointing)
        self.config = config
        self.module = module
        self.stage_id, self.num_stages = stage_id, num_stages
        self.checkpoint_activations = checkpoint_activations
        if device is not None:
            self.module.to(device)
        self._times: list[float] = []

    @property
    def device(self) -> torch.device:
        p = next(self.module.parameters(), None)
        return p.device if p is not None else torch.device("cpu")

    @property
    def is_first(self) -> bool:
        return self.stage_id == 0

    @property
    def is_last(self) -> bool:
        return self.stage_id == self.num_stages - 1

    def forward(self, *inputs, input_=None, checkpoint: bool | None = None):
        """`stage(*inputs)`; `stage(input_=x, checkpoint=True)` recomputes this call whatever the stage's setting."""
        if input_ is not None:
            inputs = (input_,) + inputs
        on = self.checkpoint_activations and self.training if checkpoint is None else bool(checkpoint)
        t0 = time.perf_counter()
        out = selective_checkpoint(self.module, *inputs, enabled=on)
        self._times.append((time.perf_counter() - t0) * 1e3)
        return out

    def forward_time_stats(self) -> dict[str, float]:
        if not self._times:
            return {"count": 0, "mean_ms": 0.0, "max_ms": 0.0}
        return {"count": len(self._times), "mean_ms": sum(self._times) / len(self._times), "max_ms": max(self._times)}


class VirtualPipelineStage:
    """The V model chunks one rank holds under the interleaved schedule (virtual stage = chunk * P + rank)."""

    class _StageId(int):
        """This rank's first virtual stage as an int; called with a chunk id it gives that chunk's virtual stage."""

        def __new__(cls, value, step):
            self = int.__new__(cls, value)
            self.step = step
            return self

        def __call__(self, chunk_id: int) -> int:
            return int(chunk_id) * self.step + int(self) % self.step if self.step else int(self)

    def __init__(self, stages: Sequence[PipelineStage], physical_rank: int | None = None, num_physical: int | None = None, *,
                 virtual_stage_id: int | None = None, physical_stage_id: int | None = None):
        """`VirtualPipelineStage(stages, physical_rank, num_physical)`; with the reference's keywords
        (`virtual_stage_id`, `physical_stage_id`) the number of physical stages is taken from the stages themselves
        (data_pipeline/trainer/distributed/pipeline_parallel.py:1101)."""
        self.stages = list(stages)
        if virtual_stage_id is not None or physical_stage_id is not None:
            physical_rank = physical_stage_id if physical_stage_id is not None else 0
            total = getattr(self.stages[0], "num_stages", len(self.stages)) if self.stages else 1
            num_physical = max(1, total // max(1, len(self.stages)))
        self.physical_rank, self.num_physical = int(physical_rank or 0), int(num_physical or 1)
        self.physical_stage_id = self.physical_rank
        first = virtual_stage_id if virtual_stage_id is not None else self.physical_rank
        self.virtual_stage_id = self._StageId(first, self.num_physical)
        self.num_stages = len(self.stages)

    @property
    def num_chunks(self) -> int:
        return len(self.stages)

    def get_stage(self, chunk_id: int) -> PipelineStage:
        return self.stages[chunk_id % len(self.stages)]

    def forward(self, chunk_id=None, *inputs, input_=None, checkpoint: bool | None = None):
        """`forward(chunk_id, *inputs)`, or the reference's `forward(input_, chunk_id, checkpoint=False)`."""
        if torch.is_tensor(chunk_id):                                   # (input_, chunk_id, checkpoint)
            input_, chunk_id, inputs = chunk_id, inputs[0], inputs[1:]
            if inputs and isinstance(inputs[0], bool):
                checkpoint, inputs = inputs[0], inputs[1:]
        if input_ is not None:
            return self.get_stage(chunk_id)(input_, *inputs, checkpoint=checkpoint)
        return self.stages[chunk_id](*inputs)

    __call__ = forward


@dataclass
class ScheduleMetrics:
    total_time_ms: float = 0.0
    compute_time_ms: float = 0.0
    num_microbatches: int = 0
    num_forward: int = 0
    num_backward: int = 0
    num_weight_grad: int = 0
    simulated_bubble: float = 0.0
    peak_activation_mb: float = 0.0

    @property
    def bubble_ratio(self) -> float:
        """Measured idle share of the step when timings exist, else the simulated bubble of the schedule."""
        if self.total_time_ms > 0 and self.compute_time_ms > 0:
            return max(0.0, 1.0 - self.compute_time_ms / self.total_time_ms)
        return self.simulated_bubble

    @property
    def throughput(self) -> float:
        return self.num_microbatches / (self.total_time_ms / 1e3) if self.total_time_ms > 0 else 0.0


# ------------------------------------------------------------------------------------------------ Chimera order
def chimera_schedule(P: int, M: int, cost: dict[str, float] | None = None) -> list[list[Action]]:
    """Bidirectional pipelines (Li & Hoefler 2021): worker w runs stage w of the "down" pipeline (chunk 0, micro-batches
    0 .. M/2-1) and stage P-1-w of the "up" pipeline (chunk 1, micro-batches M/2 .. M-1).  The per-worker order comes
    out of a greedy list scheduling of both pipelines' 1F1B queues: a worker runs whichever head action becomes ready
    first, backward before forward on ties.  Returns one action list per worker."""
    if P % 2 or M % 2:
        raise ValueError("Chimera needs an even number of stages and of micro-batches")
    cost = cost or {F_OP: 1.0, B_OP: 2.0}
    half = M // 2
    queues = []
    for w in range(P):
        down = [Action(a.op, a.mb, 0) for a in PP.one_f_one_b_schedule(w, P, half)]
        up = [Action(a.op, a.mb + half, 1) for a in PP.one_f_one_b_schedule(P - 1 - w, P, half)]
        queues.append([down, up])

    def vstage(w, chunk):
        return w if chunk == 0 else P - 1 - w

    def owner(stage, chunk):
        return stage if chunk == 0 else P - 1 - stage

    done: dict[tuple, float] = {}
    t = [0.0] * P
    heads = [[0, 0] for _ in range(P)]
    out: list[list[Action]] = [[] for _ in range(P)]
    remaining = sum(len(q) for qs in queues for q in qs)
    while remaining:
        best = None
        for w in range(P):
            for c in (0, 1):
                i = heads[w][c]
                if i >= len(queues[w][c]):
                    continue
                a = queues[w][c][i]
                s = vstage(w, c)
                deps = []
                if a.op == F_OP and s > 0:
                    deps.append((F_OP, s - 1, a.mb))
                if a.op == B_OP:
                    deps.append((F_OP, s, a.mb))
                    if s < P - 1:
                        deps.append((B_OP, s + 1, a.mb))
                if any(d not in done for d in deps):
                    continue
                ready = max([t[w]] + [done[d] for d in deps])
                key = (ready, 0 if a.op == B_OP else 1, w, c)
                if best is None or key < best[0]:
                    best = (key, w, c, a, s)
        if best is None:
            raise RuntimeError("Chimera order deadlocks")
        (ready, _, _, _), w, c, a, s = best
        done[(a.op, s, a.mb)] = ready + cost[a.op]
        t[w] = ready + cost[a.op]
        heads[w][c] += 1
        out[w].append(a)
        remaining -= 1
    return out


# ------------------------------------------------------------------------------------------------ schedules
class PipelineSchedule(ABC):
    """A schedule = per-worker action lists + the executor below.

    `stages`: with all stages in this process, every virtual stage in order (P * V modules; P for Chimera, whose two
    directions share the modules).  With one worker per rank (`ctx.is_distributed`), this rank's chunks: V modules for
    the interleaved schedule (chunk c is virtual stage c * P + rank), [stage rank, stage P-1-rank] for Chimera, else one.
    The distributed mode has been exercised on the gloo backend; on NCCL the framework decoder's `pp.PipelineRuntime`
    (batched exchanges) is the tested path."""

    schedule_name = "1f1b"

    def __init__(self, stages: Sequence[PipelineStage], config: PipelineConfig,
                 loss_fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
                 communicator: P2PCommunicator | None = None, memory_manager: ActivationMemoryManager | None = None,
                 ctx: DistributedContext | None = None):
        self.stages, self.config, self.loss_fn = list(stages), config, loss_fn
        self.ctx = ctx or (communicator.ctx if communicator is not None else _DEFAULT_CTX)
        self.communicator = communicator
        self.num_stages = config.num_stages
        self.num_microbatches = config.num_microbatches
        dev = self.stages[0].device if self.stages else torch.device("cpu")
        self.memory_manager = memory_manager or ActivationMemoryManager(config.memory, dev)
        self.metrics = ScheduleMetrics()
        self.distributed = self.ctx.is_distributed and communicator is not None
        self.grad_scaler = None

    # -- layout of the schedule: which (pipe, stage) a worker's chunk is, and who owns a (pipe, stage)
    @property
    def stages_per_pipe(self) -> int:
        return self.config.total_virtual_stages

    def node_of(self, worker: int, chunk: int) -> tuple[int, int]:
        return 0, chunk * self.num_stages + worker

    def worker_of(self, pipe: int, s: int) -> int:
        return s % self.num_stages

    def local_module(self, pipe: int, s: int) -> PipelineStage:
        if self.distributed:
            return self.stages[s // self.num_stages]
        return self.stages[s]

    def actions(self) -> list[list[Action]]:
        P, M, V = self.num_stages, self.num_microbatches, self.config.num_virtual_stages
        return [PP.create_schedule(self.schedule_name, w, P, M, V) for w in range(P)]

    def simulated_bubble(self) -> float:
        try:
            return PP.simulate(self.actions())["bubble_fraction"] if self.config.num_virtual_stages == 1 else 0.0
        except (RuntimeError, KeyError):
            return 0.0

    def reset_metrics(self) -> None:
        self.metrics = ScheduleMetrics()

    # -- executor
    def run(self, input_batches: Sequence[torch.Tensor], target_batches: Sequence[torch.Tensor]) -> torch.Tensor:
        """Forward + backward of every micro-batch in this schedule's order.  Parameter gradients are accumulated in
        `.grad`; returns the mean loss (on every rank that holds a last stage; zeros elsewhere)."""
        M = self.num_microbatches
        if len(input_batches) != M or len(target_batches) != M:
            raise ValueError(f"expected {M} micro-batches, got {len(input_batches)} / {len(target_batches)}")
        acts = self.actions()
        split = any(a.op == W_OP for lst in acts for a in lst)
        S = self.stages_per_pipe
        me = self.ctx.pipeline_parallel_rank if self.distributed else None
        workers = [me] if self.distributed else list(range(self.num_stages))
        mem = self.memory_manager
        avail_act: dict[tuple, torch.Tensor] = {}
        avail_grad: dict[tuple, torch.Tensor] = {}
        pending_w: dict[tuple, tuple] = {}
        total = None
        t_start = time.perf_counter()
        compute_ms = 0.0

        expected: dict[int, list] = {}
        if self.distributed:
            for w, lst in enumerate(acts):
                if w == me:
                    continue
                q = []
                for a in lst:
                    pipe, s = self.node_of(w, a.chunk)
                    if a.op == F_OP and s < S - 1 and self.worker_of(pipe, s + 1) == me:
                        q.append(("act", (pipe, s + 1, a.mb)))
                    if a.op == B_OP and s > 0 and self.worker_of(pipe, s - 1) == me:
                        q.append(("grad", (pipe, s - 1, a.mb)))
                expected[w] = q

        def fetch(kind: str, key: tuple, src_worker: int) -> torch.Tensor:
            store = avail_act if kind == "act" else avail_grad
            while key not in store:
                k2, key2 = expected[src_worker].pop(0)
                t = self.communicator.recv_sync(self.ctx.global_rank_of(src_worker), f"{k2}:{key2[0]}:{key2[1]}")
                (avail_act if k2 == "act" else avail_grad)[key2] = t
            return store.pop(key)

        def deliver(kind: str, key: tuple, t: torch.Tensor) -> None:
            dst = self.worker_of(key[0], key[1])
            if self.distributed and dst != me:
                self.communicator.send_async(t, self.ctx.global_rank_of(dst), f"{kind}:{key[0]}:{key[1]}")
            else:
                (avail_act if kind == "act" else avail_grad)[key] = t.detach()

        def ready(w: int, a: Action) -> bool:
            pipe, s = self.node_of(w, a.chunk)
            key = (pipe, s, a.mb)
            if a.op == F_OP:
                return s == 0 or self.distributed or key in avail_act
            if a.op == B_OP:
                return s == S - 1 or self.distributed or key in avail_grad
            return True

        def execute(w: int, a: Action) -> None:
            nonlocal total, compute_ms
            pipe, s = self.node_of(w, a.chunk)
            key = (pipe, s, a.mb)
            mod = self.local_module(pipe, s)
            last = s == S - 1
            t0 = time.perf_counter()
            if a.op == F_OP:
                if s == 0:
                    x = input_batches[a.mb]
                else:
                    x = (fetch("act", key, self.worker_of(pipe, s - 1)) if self.distributed and key not in avail_act
                         else avail_act.pop(key)).to(mod.device).detach().requires_grad_(True)
                y = mod(x if s > 0 else x.to(mod.device))
                if last:
                    out = self.loss_fn(y, target_batches[a.mb].to(y.device)) / M
                    total = out.detach() if total is None else total + out.detach()
                else:
                    out = y
                    deliver("act", (pipe, s + 1, a.mb), y)
                mem.stash_activation(key, (x, out))
                self.metrics.num_forward += 1
            elif a.op == B_OP:
                x, out = mem.pop_activation(key)
                g = None
                if not last:
                    g = (fetch("grad", key, self.worker_of(pipe, s + 1)) if self.distributed and key not in avail_grad
                         else avail_grad.pop(key)).to(out.device)
                if split:
                    if s > 0:
                        gx = torch.autograd.grad(out, [x], g, retain_graph=True)[0]
                        deliver("grad", (pipe, s - 1, a.mb), gx)
                    pending_w[key] = (out, g)
                else:
                    torch.autograd.backward(out, g)
                    if s > 0:
                        deliver("grad", (pipe, s - 1, a.mb), x.grad)
                self.metrics.num_backward += 1
            else:
                out, g = pending_w.pop(key)
                params = [p for p in mod.parameters() if p.requires_grad]
                grads = torch.autograd.grad(out, params, g, allow_unused=True)
                with torch.no_grad():
                    for p, gr in zip(params, grads):
                        if gr is not None:
                            p.grad = gr if p.grad is None else p.grad + gr
                self.metrics.num_weight_grad += 1
            compute_ms += (time.perf_counter() - t0) * 1e3

        heads = {w: 0 for w in workers}
        left = sum(len(acts[w]) for w in workers)
        while left:
            progressed = False
            for w in workers:
                while heads[w] < len(acts[w]) and ready(w, acts[w][heads[w]]):
                    execute(w, acts[w][heads[w]])
                    heads[w] += 1
                    left -= 1
                    progressed = True
            if not progressed:
                raise RuntimeError(f"{type(self).__name__}: no action can run (unmet dependencies)")
        if self.distributed:
            self.communicator.wait_all()
        mem.clear()
        self.metrics.total_time_ms += (time.perf_counter() - t_start) * 1e3
        self.metrics.compute_time_ms += compute_ms / max(1, len(workers))
        self.metrics.num_microbatches += M
        self.metrics.peak_activation_mb = max(self.metrics.peak_activation_mb, mem.peak_memory_mb)
        if total is None:
            total = torch.zeros((), device=self.stages[0].device if self.stages else "cpu")
        return total


class GPipeSchedule(PipelineSchedule):
    """All forwards, then all backwards (fill / drain)."""
    schedule_name = "gpipe"


class OneFOneBSchedule(PipelineSchedule):
    """Warm-up of P-1-stage forwards, then one forward / one backward alternating, then the drain."""
    schedule_name = "1f1b"


class InterleavedOneFOneBSchedule(PipelineSchedule):
    """1F1B over V model chunks per rank (virtual stage = chunk * P + rank): the bubble shrinks by 1/V."""
    schedule_name = "interleaved"

    def __init__(self, stages, config, loss_fn, communicator=None, memory_manager=None, ctx=None, *,
                 num_chunks: int | None = None):
        """`num_chunks`: model chunks per rank; must agree with `config.num_virtual_stages` (which it sets when that is
        still 1)."""
        if isinstance(ctx, int) and num_chunks is None:                 # (..., memory_manager, num_chunks) positionally
            num_chunks, ctx = ctx, None
        if num_chunks is not None and int(num_chunks) != config.num_virtual_stages:
            if config.num_virtual_stages != 1:
                raise ValueError(f"num_chunks={num_chunks} but config.num_virtual_stages={config.num_virtual_stages}")
            import dataclasses
            config = dataclasses.replace(config, num_virtual_stages=int(num_chunks))
        super().__init__(stages, config, loss_fn, communicator, memory_manager, ctx)
        self.num_chunks = config.num_virtual_stages


class ZeroBubbleSchedule(PipelineSchedule):
    """1F1B order with the backward split in two: B (input gradients, on the critical path) and W (weight gradients,
    deferred into the idle slots).  For arbitrary modules the split is two `autograd.grad` calls over the retained
    graph; the framework decoder uses parked weight-gradient GEMMs instead (`pp.PipelineRuntime`)."""
    schedule_name = "zero_bubble"


class ChimeraSchedule(PipelineSchedule):
    """Two pipelines over the same workers in opposite directions; each takes half of the micro-batches.  In one
    process both directions run through the same stage modules; across ranks each rank holds [stage r, stage P-1-r] and
    the gradients of the two replicas of a stage must be summed afterwards (`sync_replica_grads`)."""
    schedule_name = "chimera"

    @property
    def stages_per_pipe(self) -> int:
        return self.num_stages

    def node_of(self, worker: int, chunk: int) -> tuple[int, int]:
        return chunk, (worker if chunk == 0 else self.num_stages - 1 - worker)

    def worker_of(self, pipe: int, s: int) -> int:
        return s if pipe == 0 else self.num_stages - 1 - s

    def local_module(self, pipe: int, s: int) -> PipelineStage:
        return self.stages[pipe] if self.distributed else self.stages[s]

    def actions(self) -> list[list[Action]]:
        return chimera_schedule(self.num_stages, self.num_microbatches)

    def simulated_bubble(self) -> float:
        return 0.0

    def sync_replica_grads(self) -> None:
        """Distributed mode: stage s has one replica on rank s (down direction) and one on rank P-1-s (up direction).
        This rank's peer for BOTH of its modules is rank P-1-me: the peer's down module is my up module's stage and the
        other way round.  One exchange of [grad(down) | grad(up)], then each side adds the crossed halves."""
        if not self.distributed:
            return
        me, P = self.ctx.pipeline_parallel_rank, self.num_stages
        peer = self.ctx.global_rank_of(P - 1 - me)
        down, up = list(self.stages[0].parameters()), list(self.stages[1].parameters())

        def flat(ps):
            return [(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1).float() for p in ps]

        send = torch.cat(flat(down) + flat(up))
        recv = torch.empty_like(send)
        ops = [dist.P2POp(dist.isend, send, peer, self.ctx.group), dist.P2POp(dist.irecv, recv, peer, self.ctx.group)]
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        n_up = sum(p.numel() for p in up)          # the peer's down module is my up module's stage
        off = 0
        with torch.no_grad():
            for p in up + down:                     # peer layout: [its down = my up | its up = my down]
                g = recv[off:off + p.numel()].view_as(p).to(p.dtype)
                p.grad = g.clone() if p.grad is None else p.grad + g
                off += p.numel()
        assert off == recv.numel() and n_up <= off


_SCHEDULES = {ScheduleType.GPIPE: GPipeSchedule, ScheduleType.ONE_F_ONE_B: OneFOneBSchedule,
              ScheduleType.INTERLEAVED_ONE_F_ONE_B: InterleavedOneFOneBSchedule,
              ScheduleType.ZERO_BUBBLE: ZeroBubbleSchedule, ScheduleType.CHIMERA: ChimeraSchedule}


def create_schedule(stages, config=None, loss_fn=None, communicator: P2PCommunicator | None = None,
                    memory_manager: ActivationMemoryManager | None = None, ctx: DistributedContext | None = None, *,
                    schedule_type=None) -> PipelineSchedule:
    """Schedule object for `config.schedule`.  The reference passes the kind first, `create_schedule(schedule_type,
    stages, config, loss_fn, ...)` (data_pipeline/trainer/distributed/pipeline_parallel.py:2029): a `ScheduleType` or
    its name in the first position, or `schedule_type=`, overrides `config.schedule`."""
    if isinstance(stages, (ScheduleType, str)):
        schedule_type, stages, config, loss_fn, communicator, memory_manager = (stages, config, loss_fn, communicator,
                                                                                memory_manager, ctx)
        ctx = None
    kind = config.schedule if schedule_type is None else schedule_type
    kind = kind if isinstance(kind, ScheduleType) else ScheduleType(str(kind).lower())
    return _SCHEDULES[kind](stages, config, loss_fn, communicator, memory_manager, ctx)


# ------------------------------------------------------------------------------------------------ wrapper
class PipelineParallel(nn.Module):
    """`PipelineParallel(stages, config, loss_fn)(input_batches, target_batches)` runs one pipelined forward+backward
    and returns the mean loss; parameter gradients are left in `.grad` for any optimizer."""

    def __init__(self, stages: Sequence[nn.Module], config: PipelineConfig,
                 loss_fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor], ctx: DistributedContext | None = None,
                 device: torch.device | str | None = None):
        super().__init__()
        self.config = config
        self.ctx = ctx or _DEFAULT_CTX
        wrapped = []
        for i, m in enumerate(stages):
            if not isinstance(m, PipelineStage):
                m = PipelineStage(m, i, len(stages), device,
                                  checkpoint_activations=config.memory.enable_activation_checkpointing)
            wrapped.append(m)
        self.stages = nn.ModuleList(wrapped)
        dev = wrapped[0].device if wrapped else torch.device("cpu")
        self.pool = TensorPool(dev, config.memory.pool_max_bytes) if config.memory.enable_tensor_pool else None
        self.communicator = P2PCommunicator(self.ctx, dev, config.communication, None) if self.ctx.is_distributed \
            else None
        self.schedule = create_schedule(list(self.stages), config, loss_fn, self.communicator, None, self.ctx)

    def forward(self, input_batches: Sequence[torch.Tensor], target_batches: Sequence[torch.Tensor]) -> torch.Tensor:
        loss = self.schedule.run(input_batches, target_batches)
        if isinstance(self.schedule, ChimeraSchedule):
            self.schedule.sync_replica_grads()
        return loss

    def get_metrics(self) -> ScheduleMetrics:
        m = self.schedule.metrics
        m.simulated_bubble = self.schedule.simulated_bubble()
        return m

    def reset_metrics(self) -> None:
        self.schedule.reset_metrics()

    def get_stage_timing_stats(self) -> dict[int, dict[str, float]]:
        return {st.stage_id: st.forward_time_stats() for st in self.stages}


# ------------------------------------------------------------------------------------------------ partitioning
def split_model_into_stages(model: nn.Module | Sequence[nn.Module], num_stages: int,
                            costs: Sequence[float] | None = None, device: torch.device | str | None = None,
                            checkpoint_activations: bool = False, *, split_points: Sequence[str] | None = None,
                            balance: Sequence[int] | None = None) -> list[PipelineStage]:
    """Cut a sequence of layers (an `nn.Sequential`, a list of modules, or a module whose children form the chain)
    into `num_stages` contiguous stages: equal layer counts, or minimal maximum cost when `costs` are given.
    `balance` fixes the number of layers per stage; `split_points` names the child modules at which a new stage
    begins (data_pipeline/trainer/distributed/pipeline_parallel.py:2318)."""
    if isinstance(model, (nn.Sequential, list, tuple, nn.ModuleList)):
        named = [(str(i), m) for i, m in enumerate(model)]
    else:
        named = list(model.named_children())
    layers = [m for _, m in named]
    if len(layers) < num_stages:
        raise ValueError(f"{len(layers)} layers cannot fill {num_stages} stages")
    if balance is not None:
        if len(balance) != num_stages or sum(balance) != len(layers) or min(balance) < 1:
            raise ValueError(f"balance {list(balance)} must give {num_stages} positive counts summing to {len(layers)}")
        cuts = [0]
        for n in balance:
            cuts.append(cuts[-1] + n)
        ranges = [range(a, b) for a, b in zip(cuts, cuts[1:])]
    elif split_points is not None:
        names = [n for n, _ in named]
        cuts = [0] + sorted(names.index(p) for p in split_points) + [len(layers)]
        if len(cuts) - 1 != num_stages or any(b <= a for a, b in zip(cuts, cuts[1:])):
            raise ValueError(f"split_points {list(split_points)} do not give {num_stages} non-empty stages")
        ranges = [range(a, b) for a, b in zip(cuts, cuts[1:])]
    else:
        ranges = PP.split_layers(len(layers), num_stages, costs)
    return [PipelineStage(nn.Sequential(*[layers[i] for i in r]), s, num_stages, device, checkpoint_activations)
            for s, r in enumerate(ranges)]


def estimate_stage_memory(stage: nn.Module = None, batch_size: int = 1, seq_len: int = 1, hidden: int | None = None,
                          dtype_bytes: int = 2, optimizer_bytes_per_param: int = 12, in_flight: int = 1, *,
                          stages: Sequence[nn.Module] | None = None, input_shape: Sequence[int] | None = None,
                          dtype: torch.dtype | None = None):
    """Bytes a stage needs: parameters + gradients + optimizer state + `in_flight` micro-batches of activations
    (counted as outputs of its linear layers, or batch*seq*hidden per child when `hidden` is given).
    The reference's form `estimate_stage_memory(stages, input_shape, dtype)` returns one total in MiB per stage."""
    if stages is not None or isinstance(stage, (list, tuple)):
        stages = stages if stages is not None else stage
        shape = tuple(input_shape if input_shape is not None else (batch_size if isinstance(batch_size, (list, tuple))
                                                                   else (1, 1)))
        b, sq = (shape + (1, 1))[:2]
        eb = torch.empty((), dtype=dtype).element_size() if dtype is not None else dtype_bytes
        return [estimate_stage_memory(st, b, sq, None, eb, optimizer_bytes_per_param, in_flight)["total"] / 2 ** 20
                for st in stages]
    n = sum(p.numel() for p in stage.parameters())
    if hidden is not None:
        act = batch_size * seq_len * hidden * dtype_bytes * max(1, len(list(stage.modules())) - 1)
    else:
        act = sum(batch_size * seq_len * m.out_features * dtype_bytes for m in stage.modules()
                  if isinstance(m, nn.Linear))
    return {"params": n * dtype_bytes, "grads": n * dtype_bytes, "optimizer": n * optimizer_bytes_per_param,
            "activations": act * in_flight,
            "total": n * (2 * dtype_bytes + optimizer_bytes_per_param) + act * in_flight}


@reference_kwargs({"target_memory_mb": ANY}, model="layers")
def balance_stages_by_memory(layers: Sequence[nn.Module], num_stages: int, batch_size: int = 1, seq_len: int = 1,
                             schedule: str = "1f1b", *, input_shape: Sequence[int] | None = None) -> list[range]:
    """Contiguous split minimising the largest stage footprint.  Under 1F1B stage s keeps P - s micro-batches of
    activations alive, so early stages are charged more per layer; two passes refine the split with those weights.
    `layers` may be a module (its children are the layers); `input_shape` = (batch, seq, ...) sets both sizes."""
    if isinstance(layers, nn.Module) and not isinstance(layers, (nn.Sequential, nn.ModuleList)):
        layers = list(layers.children())
    layers = list(layers)
    if isinstance(batch_size, (tuple, list, torch.Size)):        # (model, num_stages, input_shape), the reference's order
        input_shape, batch_size = batch_size, 1
    if input_shape is not None:
        batch_size, seq_len = (tuple(input_shape) + (1, 1))[:2]
    base = [estimate_stage_memory(l, batch_size, seq_len) for l in layers]
    costs = [b["total"] for b in base]
    ranges = PP.split_layers(len(layers), num_stages, costs)
    if schedule in ("1f1b", "interleaved", "zero_bubble"):
        for _ in range(2):
            stage_of = {}
            for s, r in enumerate(ranges):
                for i in r:
                    stage_of[i] = s
            costs = [b["total"] - b["activations"] + b["activations"] * (num_stages - stage_of.get(i, 0))
                     for i, b in enumerate(base)]
            ranges = PP.split_layers(len(layers), num_stages, costs)
    return ranges


@reference_kwargs(tensor="batch")
def split_into_microbatches(batch, num_microbatches: int):
    """Tensor -> list of chunks along dim 0; dict of tensors -> list of dicts."""
    if isinstance(batch, dict):
        return PP.split_into_microbatches(batch, num_microbatches)
    return list(batch.chunk(num_microbatches, dim=0))


@reference_kwargs(microbatches="outputs")
def merge_microbatches(outputs: Sequence) -> Any:
    if not outputs:
        return outputs
    if isinstance(outputs[0], dict):
        return {k: merge_microbatches([o[k] for o in outputs]) for k in outputs[0]}
    if torch.is_tensor(outputs[0]):
        return torch.stack(list(outputs)).mean() if outputs[0].dim() == 0 else torch.cat(list(outputs), dim=0)
    return list(outputs)


@contextlib.contextmanager
def pipeline_profiler(pipeline=None, name: str = "pipeline", log: Callable[[str], None] | None = None, *,
                      config: "ProfilingConfig | None" = None, output_dir: str | None = None):
    """Times the block (CUDA-synchronised when the stages are on a GPU) and reports the schedule's counters.
    The reference's form `pipeline_profiler(config, output_dir)` (a ProfilingConfig first) wraps the block in
    `torch.profiler` and writes a Chrome trace under `output_dir` when `config.enabled`; it yields the profiler."""
    if isinstance(pipeline, ProfilingConfig) or config is not None:
        config = config if config is not None else pipeline
        out = output_dir if output_dir is not None else (name if name != "pipeline" else "./profiles")
        if not config.enabled:
            yield None
            return
        import os
        from torch.profiler import ProfilerActivity, profile
        os.makedirs(out, exist_ok=True)
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
        with profile(activities=acts) as prof:
            yield prof
        prof.export_chrome_trace(os.path.join(out, "pipeline_trace.json"))
        return
    dev = pipeline.stages[0].device if len(pipeline.stages) else torch.device("cpu")
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)
    pipeline.reset_metrics()
    t0 = time.perf_counter()
    report: dict[str, Any] = {}
    try:
        yield report
    finally:
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)
        m = pipeline.get_metrics()
        report.update(name=name, wall_ms=(time.perf_counter() - t0) * 1e3, microbatches=m.num_microbatches,
                      forwards=m.num_forward, backwards=m.num_backward, weight_grads=m.num_weight_grad,
                      bubble_ratio=m.bubble_ratio, simulated_bubble=m.simulated_bubble,
                      peak_activation_mb=m.peak_activation_mb, stage_times=pipeline.get_stage_timing_stats())
        if log is not None:
            log(f"[{name}] {report['wall_ms']:.1f} ms, {m.num_microbatches} micro-batches, "
                f"bubble {m.bubble_ratio:.2%} (schedule {m.simulated_bubble:.2%})")
