"""Process-group bring-up and small distributed utilities.

After data_pipeline/trainer/distributed/sota_utils.py:92-2022 and __init__.py:66-1203: `DistributedBackend.auto_detect`,
`DistributedState.from_environment / initialize / shutdown`, NCCL environment defaults, `NanoTimer` / `CUDATimer`
(event timers read later, never a host sync in the hot path), `fused_clip_grad_norm_`, `dist_reduce`,
`dist_all_gather`, `set_deterministic_seed`, `GradScaler`, `log_rank_0`, `main_process_first`, `get_world_info`.
"""
from __future__ import annotations

import contextlib
import datetime
import logging
import math
import os
import random
import time
from dataclasses import dataclass
from enum import Enum
from typing import NamedTuple

import numpy as np
import torch
import torch.distributed as dist

from ..utils.refargs import ANY, reference_kwargs

logger = logging.getLogger("trainscale_b200")


class DistributedBackend(str, Enum):
    NCCL = "nccl"
    GLOO = "gloo"

    @classmethod
    def auto_detect(cls) -> "DistributedBackend":
        return cls.NCCL if torch.cuda.is_available() else cls.GLOO


def configure_nccl_environment(nvls: bool = True) -> dict[str, str]:
    """Defaults for a single NVSwitch node; existing values win. NVLS (in-switch reduction) stays on unless asked
    otherwise (failure-injection tests turn it off)."""
    want = {"NCCL_NVLS_ENABLE": "1" if nvls else "0", "TORCH_NCCL_ASYNC_ERROR_HANDLING": "1", "NCCL_P2P_LEVEL": "NVL"}
    for k, v in want.items():
        os.environ.setdefault(k, v)
    return {k: os.environ[k] for k in want}


@dataclass
class DistributedState:
    rank: int = 0
    local_rank: int = 0
    world_size: int = 1
    local_world_size: int = 1
    backend: str = "gloo"
    initialized_here: bool = False

    @classmethod
    def from_environment(cls) -> "DistributedState":
        e = os.environ
        return cls(int(e.get("RANK", 0)), int(e.get("LOCAL_RANK", 0)), int(e.get("WORLD_SIZE", 1)),
                   int(e.get("LOCAL_WORLD_SIZE", e.get("WORLD_SIZE", 1))), DistributedBackend.auto_detect().value)

    @classmethod
    def initialize(cls, backend: str | None = None, timeout_s: int = 1800, init_method: str | None = None
                   ) -> "DistributedState":
        """`init_method`: torch's rendezvous URL (default: env://, i.e. MASTER_ADDR / MASTER_PORT)."""
        st = cls.from_environment()
        if backend:
            st.backend = backend
        if st.world_size > 1 and not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            kw = {}
            if st.backend == "nccl":
                configure_nccl_environment()
                torch.cuda.set_device(st.local_rank)
                kw["device_id"] = torch.device("cuda", st.local_rank)
            if init_method:
                kw["init_method"] = init_method
            dist.init_process_group(st.backend, rank=st.rank, world_size=st.world_size,
                                    timeout=datetime.timedelta(seconds=timeout_s), **kw)
            st.initialized_here = True
        return st

    @property
    def is_main(self) -> bool:
        return self.rank == 0

    @property
    def device(self) -> torch.device:
        return torch.device("cuda", self.local_rank) if torch.cuda.is_available() else torch.device("cpu")

    def barrier(self, group=None):
        if dist.is_initialized():
            dist.barrier(group=group)

    # ---- the reference's accessors (data_pipeline/trainer/distributed/__init__.py:176-262, sota_utils.py:666-1060)
    is_main_process = property(lambda self: self.rank == 0)
    is_local_main = property(lambda self: self.local_rank == 0)
    is_local_main_process = property(lambda self: self.local_rank == 0)
    is_distributed = property(lambda self: self.world_size > 1)
    is_initialized = property(lambda self: self.world_size == 1 or (dist.is_available() and dist.is_initialized()))
    initialized = property(lambda self: self.is_initialized)
    num_nodes = property(lambda self: max(1, self.world_size // max(1, self.local_world_size)))
    node_rank = property(lambda self: self.rank // max(1, self.local_world_size))

    @property
    def tensor_pool(self) -> "TensorPool":
        if "_pool" not in self.__dict__:
            self.__dict__["_pool"] = TensorPool(self.device)
        return self.__dict__["_pool"]

    def broadcast(self, tensor: torch.Tensor, src: int = 0, group=None, async_op: bool = False):
        if not (self.is_distributed and dist.is_initialized()):
            return tensor
        work = dist.broadcast(tensor, src=src, group=group, async_op=async_op)
        return work if async_op else tensor

    def all_reduce(self, tensor: torch.Tensor, op: str = "sum", group=None, async_op: bool = False):
        """In-place all-reduce; `op` sum | mean | max | min | prod (a `dist.ReduceOp` works too).  With `async_op` the
        work handle is returned and a mean still has to be divided by the caller after `wait()`."""
        if not (self.is_distributed and dist.is_initialized()):
            return tensor
        name = op if isinstance(op, str) else str(getattr(op, "name", op))
        name = name.lower().split(".")[-1]
        table = {"sum": dist.ReduceOp.SUM, "mean": dist.ReduceOp.SUM, "avg": dist.ReduceOp.SUM,
                 "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN, "prod": dist.ReduceOp.PRODUCT,
                 "product": dist.ReduceOp.PRODUCT}
        work = dist.all_reduce(tensor, op=table[name], group=group, async_op=async_op)
        if async_op:
            return work
        if name in ("mean", "avg"):
            tensor.div_(dist.get_world_size(group))
        return tensor

    def get_process_group(self, name: str, ranks: list | None = None):
        """Named process group, created once (collectively: every rank must ask for the same groups in the same
        order); None without an initialised job."""
        groups = self.__dict__.setdefault("_groups", {})
        if name not in groups:
            if not (dist.is_available() and dist.is_initialized()):
                return None
            groups[name] = dist.new_group(ranks=ranks if ranks is not None else list(range(self.world_size)))
        return groups[name]

    def get_data_parallel_group(self):
        return self.get_process_group("data_parallel")

    def get_tensor_parallel_group(self, tp_size: int):
        """Group of this rank among groups of `tp_size` consecutive ranks (all groups are created, in rank order)."""
        if self.world_size % tp_size:
            raise ValueError(f"world size {self.world_size} is not divisible by tp_size {tp_size}")
        mine = None
        for g in range(self.world_size // tp_size):
            ranks = list(range(g * tp_size, (g + 1) * tp_size))
            grp = self.get_process_group(f"tensor_parallel_{tp_size}_{g}", ranks)
            if self.rank in ranks:
                mine = grp
        return mine

    def shutdown(self):
        if self.initialized_here and dist.is_initialized():
            dist.destroy_process_group()
            self.initialized_here = False


class NanoTimer:
    """Device timer: `with timer("fwd"):` records two CUDA events; durations are read by `flush()` for events that
    have completed (no synchronisation)."""

    def __init__(self, name: str = "", use_cuda: bool | None = None, stream=None):
        """`name`: default label of `start()` / `stop()` spans; `use_cuda=False` forces the host clock; `stream`: the
        CUDA stream whose work is timed (the current stream when None)."""
        if use_cuda is not None and not isinstance(use_cuda, bool):      # CUDATimer(name, stream)
            use_cuda, stream = None, use_cuda
        self.name, self.stream = name, stream
        self.cuda = torch.cuda.is_available() if use_cuda is None else (bool(use_cuda) and torch.cuda.is_available())
        self.pending: list[tuple[str, object, object]] = []
        self.totals: dict[str, float] = {}
        self.counts: dict[str, int] = {}

    @contextlib.contextmanager
    def __call__(self, name: str):
        if self.cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(self.stream)
            yield
            b.record(self.stream)
            self.pending.append((name, a, b))
        else:
            t0 = time.perf_counter()
            yield
            self._add(name, (time.perf_counter() - t0) * 1e3)

    def _add(self, name, ms):
        self.totals[name] = self.totals.get(name, 0.0) + ms
        self.counts[name] = self.counts.get(name, 0) + 1

    def flush(self):
        keep = []
        for name, a, b in self.pending:
            if b.query():
                self._add(name, a.elapsed_time(b))
            else:
                keep.append((name, a, b))
        self.pending = keep

    def summary(self) -> dict[str, float]:
        self.flush()
        return {k: self.totals[k] / self.counts[k] for k in self.totals}

    # ---- single-interval interface (data_pipeline/trainer/distributed/sota_utils.py NanoTimer, context_parallel.py
    # CUDATimer): start() ... stop(), then elapsed_*; on CUDA the interval is measured with two events on the current
    # stream and reading it waits for the second event only.
    def start(self) -> "NanoTimer":
        if self.cuda:
            self._a, self._b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self._a.record(self.stream)
        else:
            self._a, self._b = time.perf_counter_ns(), None
        return self

    def stop(self) -> "NanoTimer":
        if self.cuda:
            self._b.record(self.stream)
        else:
            self._b = time.perf_counter_ns()
        return self

    def elapsed_ns(self) -> int:
        if getattr(self, "_b", None) is None:
            return 0
        if self.cuda:
            self._b.synchronize()
            return int(self._a.elapsed_time(self._b) * 1e6)
        return int(self._b - self._a)

    def elapsed_us(self) -> float:
        return self.elapsed_ns() / 1e3

    def elapsed_ms(self) -> float:
        return self.elapsed_ns() / 1e6

    sync_and_elapsed_ms = elapsed_ms

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.stop()
        return False


CUDATimer = NanoTimer
Timer = NanoTimer


class TensorPool:
    """Recycles scratch tensors by size class (powers of two of the byte count), per dtype, so that collectives and
    staging copies do not hit the allocator every step (data_pipeline/trainer/distributed/sota_utils.py:511-640).
    `acquire(shape, dtype)` returns a view of a pooled buffer, `release(t)` gives it back."""

    def __init__(self, device=None, max_bytes: int = 4 * 2 ** 30, *, pin_memory: bool = False):
        """`pin_memory`: host-side pools allocate page-locked buffers (when a CUDA device is present), for staging
        copies that overlap with compute (data_pipeline/trainer/distributed/activation_offload.py TensorPool)."""
        if isinstance(max_bytes, bool):                          # TensorPool(device, pin_memory)
            pin_memory, max_bytes = max_bytes, 4 * 2 ** 30
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.pin_memory = bool(pin_memory) and self.device.type == "cpu" and torch.cuda.is_available()
        self.max_bytes = max_bytes
        self._free: dict[tuple, list[torch.Tensor]] = {}
        self._owner: dict[int, torch.Tensor] = {}
        self._held = 0
        self._stats = {"acquires": 0, "hits": 0, "releases": 0, "dropped": 0}

    @staticmethod
    def _size_class(nbytes: int) -> int:
        return 1 << max(9, (max(nbytes, 1) - 1).bit_length())          # 512 B granularity at the bottom

    def acquire(self, shape, dtype: torch.dtype = torch.float32, zero: bool = False) -> torch.Tensor:
        shape = (shape,) if isinstance(shape, int) else tuple(shape)
        n = math.prod(shape)
        esz = torch.empty(0, dtype=dtype).element_size()
        cls_bytes = self._size_class(n * esz)
        self._stats["acquires"] += 1
        lst = self._free.get((cls_bytes, dtype))
        if lst:
            buf = lst.pop()
            self._held -= cls_bytes
            self._stats["hits"] += 1
        else:
            buf = torch.empty(cls_bytes // esz, dtype=dtype, device=self.device, pin_memory=self.pin_memory)
        out = buf[:n].view(shape)
        self._owner[out.data_ptr()] = buf
        return out.zero_() if zero else out

    def release(self, tensor: torch.Tensor) -> None:
        buf = self._owner.pop(tensor.data_ptr(), None)
        if buf is None:
            return                                   # not from this pool
        nbytes = buf.numel() * buf.element_size()
        self._stats["releases"] += 1
        if self._held + nbytes > self.max_bytes:
            self._stats["dropped"] += 1
            return
        self._free.setdefault((nbytes, buf.dtype), []).append(buf)
        self._held += nbytes

    def free(self, tensor: torch.Tensor | None = None) -> None:
        """`free()` drops every pooled buffer (outstanding tensors stay valid); `free(tensor)` gives one tensor back to
        the pool, like `release`."""
        if tensor is not None:
            return self.release(tensor)
        self._free.clear()
        self._held = 0

    def reset(self) -> None:
        self.free()

    def get_stats(self) -> dict:
        a = self._stats["acquires"]
        return dict(self._stats, pooled_bytes=self._held, hit_rate=self._stats["hits"] / a if a else 0.0)


@torch.no_grad()
@reference_kwargs({"foreach": ANY}, model_or_params="parameters", process_group="group")
def fused_clip_grad_norm_(parameters, max_norm: float, group=None, norm_type: float = 2.0,
                          error_if_nonfinite: bool = False) -> torch.Tensor:
    """Global norm over `.grad` (all-reduced over `group` for sharded grads), coefficient max_norm / (norm + 1e-6)
    clamped to 1, applied in place. The coefficient stays on the device.  `parameters` may be a module."""
    if isinstance(parameters, torch.nn.Module):
        parameters = parameters.parameters()
    grads = [p.grad for p in parameters if p.grad is not None]
    if not grads:
        return torch.zeros(())
    sharded = group is not None and dist.is_initialized() and dist.get_world_size(group) > 1
    if norm_type == float("inf"):
        norm = torch.stack([g.float().abs().max() for g in grads]).max()
        if sharded:
            dist.all_reduce(norm, op=dist.ReduceOp.MAX, group=group)
    else:
        sq = torch.stack([g.float().abs().pow(norm_type).sum() for g in grads]).sum()
        if sharded:
            dist.all_reduce(sq, group=group)
        norm = sq.pow(1.0 / norm_type)
    if error_if_nonfinite and not bool(torch.isfinite(norm)):
        raise RuntimeError(f"the total gradient norm is {float(norm)}")
    coef = (max_norm / (norm + 1e-6)).clamp(max=1.0)
    for g in grads:
        g.mul_(coef.to(g.dtype))
    return norm


@reference_kwargs({"async_op": (False, None)}, tensor="t", process_group="group")
def dist_reduce(t: torch.Tensor, op="mean", group=None) -> torch.Tensor:
    """`op`: "mean" | "sum" | "max" | "min", or a `torch.distributed.ReduceOp`."""
    if not (dist.is_initialized() and dist.get_world_size(group) > 1):
        return t
    t = t.clone()
    if not isinstance(op, str):
        dist.all_reduce(t, op=op, group=group)
        return t
    red = {"max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}.get(op, dist.ReduceOp.SUM)
    dist.all_reduce(t, op=red, group=group)
    return t / dist.get_world_size(group) if op == "mean" else t


@reference_kwargs({"contiguous": ANY}, tensor="t", process_group="group")
def dist_all_gather(t: torch.Tensor, group=None) -> list[torch.Tensor]:
    if not (dist.is_initialized() and dist.get_world_size(group) > 1):
        return [t]
    out = [torch.empty_like(t) for _ in range(dist.get_world_size(group))]
    dist.all_gather(out, t.contiguous(), group=group)
    return out


def set_deterministic_seed(seed: int, rank: "int | DistributedState" = 0, fully_deterministic: bool = False, *more,
                           state=None, per_rank_offset: bool = True) -> int:
    """Seeds python / numpy / torch with seed + rank and returns that number.  `state` (a DistributedState) supplies
    the rank; `per_rank_offset=False` gives every rank the same seed.  The positional form `(seed, state,
    per_rank_offset, fully_deterministic)` of data_pipeline/trainer/distributed/sota_utils.py is taken as well."""
    if isinstance(rank, DistributedState):                    # (seed, state, per_rank_offset, fully_deterministic)
        state, per_rank_offset, rank = rank, bool(fully_deterministic), 0
        fully_deterministic = bool(more[0]) if more else False
    elif more:
        raise TypeError("set_deterministic_seed() got too many positional arguments")
    if state is not None:
        rank = int(getattr(state, "rank", rank))
    s = seed + (rank if per_rank_offset else 0)
    random.seed(s)
    np.random.seed(s % 2 ** 32)
    torch.manual_seed(s)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(s)
    if fully_deterministic:
        torch.backends.cudnn.deterministic = True
        torch.backends.cudnn.benchmark = False
        torch.use_deterministic_algorithms(True, warn_only=True)
    return s


class GradScaler:
    """Dynamic loss scaling for fp16 (bf16 training does not need it)."""

    def __init__(self, init_scale: float = 2.0 ** 16, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 2000, enabled: bool = True):
        self.scale_value, self.growth, self.backoff, self.interval, self.enabled = init_scale, growth_factor, backoff_factor, growth_interval, enabled
        self._good = 0

    def scale(self, loss):
        return loss * self.scale_value if self.enabled else loss

    def step(self, optimizer, parameters) -> bool:
        if not self.enabled:
            optimizer.step()
            return True
        params = [p for p in parameters if p.grad is not None]
        finite = all(bool(torch.isfinite(p.grad).all()) for p in params)
        if finite:
            for p in params:
                p.grad.div_(self.scale_value)
            optimizer.step()
            self._good += 1
            if self._good % self.interval == 0:
                self.scale_value *= self.growth
        else:
            self.scale_value *= self.backoff
            self._good = 0
        return finite

    def unscale_(self, optimizer=None, parameters=None) -> bool:
        """Divide the gradients by the scale in place; returns whether they are all finite (the verdict `update` uses)."""
        if not self.enabled:
            return True
        params = list(parameters) if parameters is not None else [p for g in optimizer.param_groups for p in g["params"]]
        params = [p for p in params if p.grad is not None]
        self._finite = all(bool(torch.isfinite(p.grad).all()) for p in params)
        if self._finite:
            for p in params:
                p.grad.div_(self.scale_value)
        return self._finite

    def update(self, new_scale: float | None = None) -> None:
        """Grow the scale after `growth_interval` finite steps in a row, back off after a non-finite one
        (the verdict of the last `unscale_`); or set it."""
        if new_scale is not None:
            self.scale_value = float(new_scale)
            return
        if getattr(self, "_finite", True):
            self._good += 1
            if self._good % self.interval == 0:
                self.scale_value *= self.growth
        else:
            self.scale_value *= self.backoff
            self._good = 0

    def get_scale(self) -> float:
        return self.scale_value

    def state_dict(self):
        return {"scale": self.scale_value, "good": self._good}

    def load_state_dict(self, sd):
        self.scale_value, self._good = sd["scale"], sd["good"]


@reference_kwargs(message="msg")
def log_rank_0(msg: str, level: int | str = logging.INFO, include_timestamp: bool = False):
    if not dist.is_initialized() or dist.get_rank() == 0:
        if isinstance(level, str):
            level = getattr(logging, level.upper(), logging.INFO)
        if include_timestamp:
            msg = f"[{datetime.datetime.now().isoformat(timespec='seconds')}] {msg}"
        logger.log(level, msg)


@contextlib.contextmanager
def main_process_first(dist_manager=None):
    """Rank 0 runs the block first (e.g. dataset preprocessing with a cache), the others after it.  `dist_manager` is
    accepted for the reference's call form; rank and world come from torch.distributed either way."""
    multi = dist.is_initialized() and dist.get_world_size() > 1
    if multi and dist.get_rank() != 0:
        dist.barrier()
    yield
    if multi and dist.get_rank() == 0:
        dist.barrier()


def get_world_info() -> dict:
    st = DistributedState.from_environment()
    return {"rank": st.rank, "local_rank": st.local_rank, "world_size": st.world_size, "backend": st.backend,
            "initialized": dist.is_initialized(), "cuda_devices": torch.cuda.device_count()}


class HeartbeatMonitor:
    """Rank liveness over the process group's store: every rank bumps a counter key; `stale_ranks` lists ranks whose
    counter has not moved for `timeout_s`. Host-side only (no collective, no GPU work)."""

    def __init__(self, store, rank: int, world_size: int, prefix: str = "hb"):
        self.store, self.rank, self.world, self.prefix = store, rank, world_size, prefix
        self.last_seen: dict[int, tuple[int, float]] = {}

    def beat(self):
        self.store.add(f"{self.prefix}/{self.rank}", 1)

    def stale_ranks(self, timeout_s: float, now: float | None = None) -> list[int]:
        now = time.monotonic() if now is None else now
        stale = []
        for r in range(self.world):
            v = int(self.store.add(f"{self.prefix}/{r}", 0))
            prev = self.last_seen.get(r)
            if prev is None or v != prev[0]:
                self.last_seen[r] = (v, now)
            elif now - prev[1] > timeout_s:
                stale.append(r)
        return stale


# ------------------------------------------------------------------------------------------------ gradient plumbing
@reference_kwargs({"async_op": (False, None), "op": (None, dist.ReduceOp.SUM)}, output_tensor="output",
                  input_tensor="input")
def reduce_scatter_with_fp32_accumulation(output: torch.Tensor, input: torch.Tensor, group=None) -> torch.Tensor:
    """Reduce-scatter of a low-precision tensor whose sum is taken in fp32: every rank receives the W slices meant
    for it (all-to-all) and adds them in fp32 (data_pipeline/trainer/distributed/reduce_scatter_fp32.py:90).
    `input` is [W * n], `output` [n] in any float dtype.  On the flat engine's CUDA path the same arithmetic runs
    inside `ts_symm_reduce_scatter`; this is the library-collective form."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        output.copy_(input.view(-1)[:output.numel()])
        return output
    n = output.numel()
    recv = torch.empty_like(input.view(-1))
    if input.is_cuda:
        dist.all_to_all_single(recv, input.contiguous().view(-1), group=group)
    else:   # gloo has no all_to_all_single on every build: gather slices with all_gather
        parts = [torch.empty_like(input.view(-1)) for _ in range(world)]
        dist.all_gather(parts, input.contiguous().view(-1), group=group)
        r = dist.get_rank(group)
        recv = torch.cat([p[r * n:(r + 1) * n] for p in parts])
    output.copy_(recv.view(world, n).float().sum(0))
    return output


def _chunks(model) -> list:
    """A model, or the reference's list of model chunks (virtual pipeline stages), as a list."""
    return list(model) if isinstance(model, (list, tuple)) else [model]


def _grad_of(p):
    return p.grad if p.grad is not None else getattr(p, "main_grad", None)


def allreduce_layernorm_grads(model, group=None, *, tp_group=None, sequence_parallel: bool = True,
                              qk_layernorm: bool = False) -> None:
    """Sequence parallelism: norm weights saw only this rank's tokens; sum their gradients over the TP group.  With
    `qk_layernorm` the per-head q / k norm weights are summed too (they see only this rank's heads' tokens).
    `model` may be a list of chunks; `tp_group` is the reference's name for `group`; nothing happens unless
    `sequence_parallel` or `qk_layernorm` (data_pipeline/trainer/distributed/finalize_grads.py:148-208)."""
    group = group if group is not None else tp_group
    if group is None or not dist.is_initialized() or dist.get_world_size(group) <= 1:
        return
    from .tp import TPContext, allreduce_sequence_parallel_grads
    ctx = TPContext(group, dist.get_world_size(group), dist.get_rank(group), True)
    for chunk in _chunks(model):
        if sequence_parallel:
            allreduce_sequence_parallel_grads(chunk, ctx)
        if qk_layernorm:
            for name, p in chunk.named_parameters():
                if ("q_layernorm" in name or "k_layernorm" in name or "q_norm" in name or "k_norm" in name) \
                        and _grad_of(p) is not None:
                    dist.all_reduce(_grad_of(p), group=group)


@reference_kwargs(model="stage_module")
def allreduce_word_embedding_grads(stage_module, group=None, first_rank: int | None = None, last_rank: int | None = None,
                                   *, embedding_group=None, pp_group=None,
                                   share_embeddings_and_output_weights: bool = True) -> None:
    """Tied embeddings on the first and last pipeline stage: sum their gradients.  Two calling forms: this framework's
    (stage module, pipeline group, first rank, last rank), and the reference's (model or list of chunks,
    embedding_group= the group of the two end stages), where the shared weight is looked up on the chunks
    (`embed_tokens`, `tied_embedding`, `lm_head`)."""
    if not share_embeddings_and_output_weights:
        return
    if first_rank is not None and last_rank is not None and not isinstance(stage_module, (list, tuple)):
        from .pp import allreduce_tied_embedding_grads
        allreduce_tied_embedding_grads(stage_module, group if group is not None else pp_group, first_rank, last_rank)
        return
    g = embedding_group if embedding_group is not None else group
    if g is None or not dist.is_initialized() or dist.get_world_size(g) <= 1:
        return
    for chunk in _chunks(stage_module):
        for attr in ("embed_tokens", "tied_embedding", "lm_head", "word_embeddings"):
            mod = getattr(chunk, attr, None) or getattr(getattr(chunk, "model", None), attr, None)
            w = getattr(mod, "weight", None)
            if w is not None and _grad_of(w) is not None:
                dist.all_reduce(_grad_of(w), group=g)
                return


def finalize_model_grads(model, num_tokens: torch.Tensor | None = None, *, tp_group=None, sequence_parallel: bool = False,
                         pp_group=None, stage_module=None, first_rank: int = 0, last_rank: int = 0, dp_group=None,
                         embedding_group=None, pos_embedding_group=None, qk_layernorm: bool = False,
                         share_embeddings_and_output_weights: bool = True, force_all_reduce: bool = False) -> None:
    """Everything that must happen to gradients between backward and the optimizer step besides the data-parallel
    reduction (data_pipeline/trainer/distributed/finalize_grads.py:314): SP / qk norm-weight all-reduce, tied-embedding
    all-reduce across pipeline ends, position-embedding all-reduce, optional scaling by the global number of tokens.
    `model` may be a list of chunks.  `force_all_reduce` also sums every gradient over `dp_group` (for engines that do
    not reduce by themselves)."""
    chunks = _chunks(model)
    if force_all_reduce and dp_group is not None and dist.is_initialized() and dist.get_world_size(dp_group) > 1:
        for c in chunks:
            for p in c.parameters():
                if _grad_of(p) is not None:
                    dist.all_reduce(_grad_of(p), group=dp_group)
                    _grad_of(p).div_(dist.get_world_size(dp_group))
    if (sequence_parallel or qk_layernorm) and tp_group is not None:
        allreduce_layernorm_grads(chunks, tp_group, sequence_parallel=sequence_parallel, qk_layernorm=qk_layernorm)
    if pp_group is not None and stage_module is not None:
        allreduce_word_embedding_grads(stage_module, pp_group, first_rank, last_rank)
    elif embedding_group is not None:
        allreduce_word_embedding_grads(chunks, embedding_group=embedding_group, pp_group=pp_group,
                                       share_embeddings_and_output_weights=share_embeddings_and_output_weights)
    if pos_embedding_group is not None:
        allreduce_position_embedding_grads(chunks, pos_embedding_group)
    if num_tokens is not None:
        total = num_tokens.detach().float().clone()
        if dist.is_initialized() and dp_group is not False:
            dist.all_reduce(total, group=dp_group)
        scale = 1.0 / total.clamp(min=1.0)
        for c in chunks:
            for p in c.parameters():
                g = _grad_of(p)
                if g is not None:
                    g.mul_(scale.to(g.dtype))


class GradientSynchronizer:
    """`with sync.accumulate(step):` suppresses the engine's gradient reduction except on the last micro-batch of an
    accumulation window (data_pipeline/trainer/distributed/__init__.py GradientSynchronizer)."""

    @reference_kwargs({"async_sync": ANY}, model="engine")
    def __init__(self, engine, accumulation_steps: int = 1, bucket_size_mb: float = 25.0):
        """`engine`: a sharded / DDP engine, or a plain module (`model=`), whose gradients `sync_gradients()` then
        reduces in buckets of `bucket_size_mb`."""
        self.engine, self.steps, self.bucket_size_mb = engine, max(1, accumulation_steps), bucket_size_mb

    def should_sync(self, micro_step: int) -> bool:
        return (micro_step + 1) % self.steps == 0

    def accumulate(self, micro_step: int):
        import contextlib
        if self.should_sync(micro_step) or not hasattr(self.engine, "no_sync"):
            return contextlib.nullcontext()
        return self.engine.no_sync()

    def sync_gradients(self, group=None, average: bool = True) -> None:
        """Reduce the gradients now.  An engine with its own reduction (`reduce_gradients` / `sync_gradients`) does it;
        for a plain module the gradients are flattened per dtype, all-reduced in one call each and averaged."""
        for name in ("reduce_gradients", "sync_gradients", "finish_gradient_synchronization"):
            fn = getattr(self.engine, name, None)
            if callable(fn):
                fn()
                return
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
            return
        by_dtype: dict = {}
        for p in self.engine.parameters():
            if p.grad is not None:
                by_dtype.setdefault(p.grad.dtype, []).append(p.grad)
        for grads in by_dtype.values():
            flat = torch.cat([g.reshape(-1) for g in grads])
            dist.all_reduce(flat, group=group)
            if average:
                flat /= dist.get_world_size(group)
            off = 0
            for g in grads:
                g.copy_(flat[off:off + g.numel()].view_as(g))
                off += g.numel()


class DistributedManager:
    """Process-wide entry point: process-group initialisation, model wrapping into the flat engine, thin collective
    helpers (data_pipeline/trainer/distributed/__init__.py:265)."""

    _instance: "DistributedManager | None" = None

    def __new__(cls, config=None):
        if cls._instance is None:
            cls._instance = super().__new__(cls)
            cls._instance.state = None
            cls._instance.config = None
        if config is not None:
            cls._instance.config = config          # a distributed configuration (backend, timeout_seconds, ...)
        return cls._instance

    def __init__(self, config=None):
        pass

    @classmethod
    def get_instance(cls) -> "DistributedManager":
        return cls()

    def barrier(self, group=None) -> None:
        if dist.is_available() and dist.is_initialized():
            dist.barrier(group=group)

    def destroy_process_group(self) -> None:
        if dist.is_available() and dist.is_initialized():
            dist.destroy_process_group()
        self.state = None

    def init_process_group(self, backend: str | None = None, init_method: str | None = None) -> "DistributedState":
        cfg = getattr(self, "config", None)
        get = (cfg.get if isinstance(cfg, dict) else (lambda k, d=None: getattr(cfg, k, d))) if cfg is not None else \
            (lambda k, d=None: d)
        backend = backend or getattr(get("backend"), "value", get("backend"))
        self.state = DistributedState.initialize(backend, int(get("timeout_seconds", 1800) or 1800), init_method)
        return self.state

    @property
    def world_size(self) -> int:
        return dist.get_world_size() if dist.is_initialized() else 1

    @property
    def rank(self) -> int:
        return dist.get_rank() if dist.is_initialized() else 0

    def wrap_model(self, model, strategy: str = "fsdp", **engine_kwargs):
        """strategy: ddp | fsdp / zero2 | full_shard / zero3. Returns the FlatShardedEngine that owns the model's
        parameters, gradients and sharded optimizer state."""
        from .flat_engine import EngineConfig, FlatShardedEngine
        sharding = {"ddp": "NO_SHARD", "fsdp": "SHARD_GRAD_OP", "zero2": "SHARD_GRAD_OP", "full_shard": "FULL_SHARD",
                    "zero3": "FULL_SHARD"}[strategy.lower()]
        p = next(model.parameters())
        return FlatShardedEngine(model, EngineConfig(sharding_strategy=sharding, param_dtype=p.dtype, **engine_kwargs),
                                 device=p.device)

    @reference_kwargs({"async_op": (False, None)}, tensor="t")
    def all_reduce(self, t: torch.Tensor, op="sum", group=None) -> torch.Tensor:
        return dist_reduce(t, op, group)

    @reference_kwargs({"async_op": (False, None)}, tensor="t")
    def all_gather(self, t: torch.Tensor, group=None) -> list[torch.Tensor]:
        return dist_all_gather(t, group)

    @reference_kwargs(tensor="t")
    def broadcast(self, t: torch.Tensor, src: int = 0, group=None) -> torch.Tensor:
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.broadcast(t, src, group=group)
        return t

    @reference_kwargs(values="d")
    def reduce_dict(self, d: dict, average: bool = True, group=None, op: str | None = None) -> dict:
        """`op`: "mean" / "sum" (the reference's argument) instead of `average`."""
        if op is not None:
            average = str(getattr(op, "value", op)).lower() in ("mean", "avg", "average")
        if not dist.is_initialized() or dist.get_world_size(group) == 1:
            return dict(d)
        keys = sorted(d)
        flat = torch.stack([torch.as_tensor(d[k], dtype=torch.float32).reshape(()) for k in keys])
        if torch.cuda.is_available() and dist.get_backend(group) == "nccl":
            flat = flat.cuda()
        dist.all_reduce(flat, group=group)
        if average:
            flat /= dist.get_world_size(group)
        return {k: flat[i].item() for i, k in enumerate(keys)}


# ------------------------------------------------------------------------------------------------ more of the utility surface
def allreduce_position_embedding_grads(model, group=None, attr: str = "position_embeddings", *,
                                       pos_embedding_group=None) -> None:
    """Learned position embeddings replicated over a group (e.g. on several pipeline stages): sum their gradients.
    `model` may be a list of chunks; `pos_embedding_group` is the reference's name for `group`."""
    group = group if group is not None else pos_embedding_group
    if group is None or not dist.is_initialized():
        return
    for chunk in _chunks(model):
        for name, p in chunk.named_parameters():
            if attr in name:
                g = getattr(p, "main_grad", None) if p.grad is None else p.grad
                if g is not None:
                    dist.all_reduce(g, group=group)


def scale_grads_by_token_count(model, num_tokens: torch.Tensor, group=None) -> torch.Tensor:
    """Divide every gradient by the number of (non-ignored) tokens of the global batch; returns that number."""
    total = num_tokens.detach().float().clone()
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(total, group=group)
    scale = 1.0 / total.clamp(min=1.0)
    for p in model.parameters():
        g = getattr(p, "main_grad", None) if p.grad is None else p.grad
        if g is not None:
            g.mul_(scale.to(g.dtype))
    return total


_scale_grads_by_token_count = scale_grads_by_token_count


class DeviceManager:
    """Which device this process uses and what it can do (read-only queries)."""

    @reference_kwargs(device_id="local_rank")
    def __init__(self, local_rank: int | None = None, device_type: str | None = None):
        """`device_type`: "cuda" | "cpu" | None (auto); asking for "cuda" without one raises DeviceNotAvailableError."""
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0")) if local_rank is None else local_rank
        dt = getattr(device_type, "value", device_type)
        if dt in ("cuda", "gpu") and not torch.cuda.is_available():
            from ..core.errors import DeviceNotAvailableError
            raise DeviceNotAvailableError("no CUDA device is visible", device_type="cuda", available_devices=("cpu",))
        self.cuda = torch.cuda.is_available() and dt not in ("cpu",)

    @property
    def device(self) -> torch.device:
        return torch.device("cuda", self.local_rank % max(1, torch.cuda.device_count())) if self.cuda \
            else torch.device("cpu")

    def set_device(self) -> torch.device:
        if self.cuda:
            torch.cuda.set_device(self.device)
        return self.device

    def device_count(self) -> int:
        return torch.cuda.device_count() if self.cuda else 0

    def supports_bf16(self) -> bool:
        return (not self.cuda) or torch.cuda.get_device_capability(self.device)[0] >= 8

    @classmethod
    def auto_detect(cls) -> "DeviceManager":
        return cls()

    @property
    def compute_capability(self) -> tuple:
        return torch.cuda.get_device_capability(self.device) if self.cuda else (0, 0)

    def supports_fp8(self) -> bool:
        return self.cuda and self.compute_capability >= (8, 9)

    def memory_stats(self) -> dict[str, float]:
        if not self.cuda:
            return {"allocated_gb": 0.0, "reserved_gb": 0.0, "total_gb": 0.0}
        d = self.device
        return {"allocated_gb": torch.cuda.memory_allocated(d) / 2 ** 30,
                "reserved_gb": torch.cuda.memory_reserved(d) / 2 ** 30,
                "total_gb": torch.cuda.get_device_properties(d).total_memory / 2 ** 30}

    def synchronize(self) -> None:
        if self.cuda:
            torch.cuda.synchronize(self.device)

    def empty_cache(self) -> None:
        if self.cuda:
            torch.cuda.empty_cache()


@dataclass
class HardwareTopology:
    """GPUs of this node as seen by the runtime: count, name, memory, who can read whose memory directly."""
    num_gpus: int = 0
    gpu_name: str | None = None
    memory_gb: float = 0.0
    sm_count: int = 0
    peer_access: tuple = ()
    nvswitch: bool = False
    numa: dict | None = None

    @classmethod
    def detect(cls) -> "HardwareTopology":
        from .mesh import HardwareDetector
        i = HardwareDetector.detect()
        return cls(i["num_gpus"], i["name"], i["memory_gb"], i["sm_count"],
                   tuple(tuple(r) for r in i["peer_access"]), i["nvswitch"], i["numa"])

    @property
    def fully_connected(self) -> bool:
        return self.num_gpus > 1 and all(all(r) for r in self.peer_access)

    @property
    def total_gpus(self) -> int:
        return self.num_gpus

    @property
    def has_nvlink(self) -> bool:
        """Some pair of GPUs reads each other's memory directly (peer access), which on these machines is NVLink."""
        return any(ok for i, row in enumerate(self.peer_access) for j, ok in enumerate(row) if i != j)

    def recommended_bucket_mb(self) -> int:
        from .ddp import BUCKET_MB, detect_gpu_topology
        return BUCKET_MB[detect_gpu_topology()][0]


class DistributedLogger:
    """Rank-aware logging: by default only rank 0 emits; `all_ranks=True` prefixes every line with the rank."""

    @reference_kwargs(verbose_all_ranks="all_ranks")
    def __init__(self, name: str = "trainscale_b200", all_ranks: bool = False, level: int = logging.INFO):
        self._log = logging.getLogger(name)
        self._log.setLevel(level)
        self.all_ranks = all_ranks

    @staticmethod
    def _rank() -> int:
        return dist.get_rank() if dist.is_available() and dist.is_initialized() else int(os.environ.get("RANK", "0"))

    def _emit(self, level: int, msg: str, *a) -> None:
        r = self._rank()
        if self.all_ranks:
            self._log.log(level, f"[rank {r}] {msg}", *a)
        elif r == 0:
            self._log.log(level, msg, *a)


    @reference_kwargs(message="msg")
    def info(self, msg: str, *a) -> None:
        self._emit(logging.INFO, msg, *a)


    @reference_kwargs(message="msg")
    def warning(self, msg: str, *a) -> None:
        self._emit(logging.WARNING, msg, *a)

    def metric(self, name: str, value: float, unit: str = "") -> None:
        """One machine-readable line: METRIC|<ns timestamp>|<name>|<value>|<unit>|rank=<r>."""
        import time
        self._emit(logging.INFO, "METRIC|%d|%s|%s|%s|rank=%d", time.time_ns(), name, value, unit, self._rank())


    @reference_kwargs(message="msg")
    def error(self, msg: str, *a) -> None:          # errors are never silenced
        self._log.error(f"[rank {self._rank()}] {msg}", *a)


    @reference_kwargs(message="msg")
    def debug(self, msg: str, *a) -> None:
        self._emit(logging.DEBUG, msg, *a)


_GROUPS: dict[str, object] = {}


def setup_distributed(backend: str | None = None, timeout_s: int = 1800, *, config=None) -> DistributedState:
    """Rendezvous from the launcher's environment (no-op for a single process); selects this rank's GPU.  `config`
    (a mapping or object with `backend` / `timeout_seconds`) fills what the arguments leave unset."""
    if backend is not None and not isinstance(backend, str):        # setup_distributed(config, backend=None)
        config, backend = backend, None
    if config is not None:
        get = config.get if isinstance(config, dict) else (lambda k, d=None: getattr(config, k, d))
        backend = backend or get("backend")
        backend = getattr(backend, "value", backend)
        timeout_s = int(get("timeout_seconds", None) or get("timeout_s", None) or timeout_s)
    return DistributedState.initialize(backend, timeout_s)


def register_process_group(name: str, group) -> None:
    _GROUPS[name] = group


def get_process_group(name: str = "world"):
    """Named groups registered by the mesh / parallel engines ("world" is the default group)."""
    if name == "world":
        return dist.group.WORLD if dist.is_available() and dist.is_initialized() else None
    return _GROUPS.get(name)


@reference_kwargs({"async_op": (False, None), "compression": (None, "none", False)}, process_group="group")
def sync_gradients(model, group=None, average: bool = True, bucket_mb: float = 25.0) -> None:
    """One-shot bucketed all-reduce of a plain model's `.grad`s (for code that does not use an engine)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return
    from .dist_kernels import DistributedConfig, DistributedKernels
    grads = [p.grad for p in model.parameters() if p.grad is not None]
    DistributedKernels(DistributedConfig(bucket_size_mb=bucket_mb)).all_reduce_fused(grads, group=group, average=average)


def prepare_model_for_distributed(model, strategy: str = "ddp", device=None, **engine_kwargs):
    """Moves the model to this rank's device and builds the engine for `strategy` (ddp | fsdp | zero2 | zero3 |
    single).  Returns (model, engine); the engine is None for `single`.  `prepare_model_for_distributed(model, state,
    strategy)` with a `DistributedState` second (data_pipeline/trainer/distributed/sota_utils.py) is taken as well: the
    state supplies the device."""
    if isinstance(strategy, DistributedState):
        state, strategy = strategy, (device if isinstance(device, str) else "ddp")
        device = getattr(state, "device", None)
    dev = torch.device(device) if device is not None else DeviceManager().set_device()
    model.to(dev)
    s = strategy.lower()
    if s in ("single", "none"):
        return model, None
    from .flat_engine import EngineConfig, FlatShardedEngine
    shard = {"ddp": "NO_SHARD", "fsdp": "FULL_SHARD", "fsdp2": "FULL_SHARD", "zero3": "FULL_SHARD",
             "zero2": "SHARD_GRAD_OP", "shard_grad_op": "SHARD_GRAD_OP"}.get(s)
    if shard is None:
        raise ValueError(f"unknown strategy {strategy!r}")
    group = engine_kwargs.pop("process_group", None)
    eng = FlatShardedEngine(model, EngineConfig(sharding_strategy=shard, **engine_kwargs), process_group=group,
                            device=dev)
    return model, eng


def save_checkpoint_distributed(path, model=None, engine=None, extra: dict | None = None, *, state_dict=None,
                                state=None, barrier_after: bool = True) -> None:
    """Collective: rank 0 writes the full weights (+ `extra`), every rank writes its optimizer shard.  The reference's
    form `save_checkpoint_distributed(state_dict, path, state)` writes a ready state dict from rank 0 to the FILE `path`."""
    from ..ckpt import _to_cpu, atomic_torch_save
    from pathlib import Path
    if isinstance(path, dict) or state_dict is not None:
        sd, file = (path, model) if isinstance(path, dict) else (state_dict, path)
        on = dist.is_available() and dist.is_initialized()
        if not on or dist.get_rank() == 0:
            Path(file).parent.mkdir(parents=True, exist_ok=True)
            atomic_torch_save(_to_cpu(sd), Path(file))
        if on and barrier_after:
            dist.barrier()
        return
    path = Path(path)
    on = dist.is_available() and dist.is_initialized()
    rank, world = (dist.get_rank(), dist.get_world_size()) if on else (0, 1)
    sd = engine.full_model_state_dict() if engine is not None and hasattr(engine, "full_model_state_dict") \
        else model.state_dict()
    if rank == 0:
        atomic_torch_save({"model": _to_cpu(sd), "extra": extra or {}}, path / "model.pt")
    if engine is not None and hasattr(engine, "state_dict"):
        atomic_torch_save(_to_cpu(engine.state_dict()), path / "optim" / f"shard-{rank:05d}-of-{world:05d}.pt")
    if on:
        dist.barrier()


def load_checkpoint_distributed(path, model=None, engine=None, strict: bool = True, *, state=None, map_location="cpu"
                                ) -> dict:
    """Inverse of `save_checkpoint_distributed`; optimizer shards saved at another world size are re-sliced.  A `path`
    that is a file (the reference's form, `load_checkpoint_distributed(path, state, map_location)`) is read on every
    rank and returned as it is."""
    from ..ckpt import engine_layout, reshard_optimizer_state
    from pathlib import Path
    path = Path(path)
    if path.is_file():
        return torch.load(path, map_location=map_location, weights_only=False)
    blob = torch.load(path / "model.pt", map_location="cpu", weights_only=False)
    summon = engine.summon_full_params() if engine is not None and hasattr(engine, "summon_full_params") \
        else contextlib.nullcontext()
    with summon:
        own = dict(model.named_parameters())
        missing = [k for k in own if k not in blob["model"]]
        if strict and missing:
            raise KeyError(f"missing parameters in checkpoint: {missing[:6]}")
        with torch.no_grad():
            for k, v in blob["model"].items():
                if k in own:
                    own[k].copy_(v)
        if engine is not None and hasattr(engine, "units"):
            for u in engine.units:
                src = u.flat_param[u.shard_start:u.shard_start + u.shard_numel]
                if getattr(u, "resharded", False):
                    u.param_shard.copy_(src)
                u.master.copy_(src)
    if engine is not None and (path / "optim").exists():
        files = sorted((path / "optim").glob("shard-*.pt"))
        mine = path / "optim" / f"shard-{engine.rank:05d}-of-{engine.world:05d}.pt"
        if mine.exists():
            engine.load_state_dict(torch.load(mine, map_location="cpu", weights_only=False))
        elif files:
            shards = [torch.load(f, map_location="cpu", weights_only=False) for f in files]
            engine.load_state_dict(reshard_optimizer_state(shards, engine.rank, engine.world, engine_layout(engine)))
    return blob.get("extra", {})


# ------------------------------------------------------------------------------------------------ host-side fault injection
class InjectedFault(RuntimeError):
    """Raised by FaultInjector: stands for a rank that dies with a Python exception."""


class FaultInjector:
    """Failures made on the HOST, for tests of detection and recovery (nothing here touches a GPU):

        raise@K[:rankR]   raise InjectedFault at step K (on rank R only, else on every rank)
        exit@K[:rankR]    leave the process at step K without a word (os._exit), between steps
        sleep@K=S[:rankR] sleep S seconds at step K (a slow rank)
        mute@K[:rankR]    stop sending heartbeats from step K on (a rank whose messages are lost)

    The spec comes from the constructor or the TS_FAULT environment variable; several faults are separated by ','.
    Call `at_step(step)` between steps (never while a collective or kernel of this rank is in flight)."""

    def __init__(self, spec: str | None = None, rank: int | None = None):
        self.rank = int(os.environ.get("RANK", "0")) if rank is None else rank
        self.faults: list[tuple[str, int, float, int | None]] = []
        self.muted = False
        for item in filter(None, (spec if spec is not None else os.environ.get("TS_FAULT", "")).split(",")):
            head, _, who = item.partition(":rank")
            kind, _, rest = head.partition("@")
            step_s, _, arg = rest.partition("=")
            self.faults.append((kind.strip(), int(step_s), float(arg) if arg else 0.0, int(who) if who else None))

    def at_step(self, step: int) -> None:
        for kind, k, arg, who in self.faults:
            if who is not None and who != self.rank:
                continue
            if kind == "mute" and step >= k:
                self.muted = True
            if step != k:
                continue
            if kind == "raise":
                raise InjectedFault(f"injected failure on rank {self.rank} at step {step}")
            if kind == "exit":
                os._exit(17)
            if kind == "sleep":
                time.sleep(arg)

    def beat(self, monitor: HeartbeatMonitor) -> None:
        """Heartbeat unless this rank has been muted."""
        if not self.muted:
            monitor.beat()


# ------------------------------------------------------------------------------------------------ reference surface
class StatePhase(Enum):
    """Lifecycle of the distributed state (data_pipeline/trainer/distributed/sota_utils.py:655)."""
    UNINITIALIZED = 0
    INITIALIZING = 1
    READY = 2
    SHUTTING_DOWN = 3
    TERMINATED = 4
    ERROR = 5


class DistributedStateTransition(Enum):
    UNINITIALIZED_TO_INITIALIZING = (StatePhase.UNINITIALIZED, StatePhase.INITIALIZING)
    INITIALIZING_TO_READY = (StatePhase.INITIALIZING, StatePhase.READY)
    READY_TO_SHUTTING_DOWN = (StatePhase.READY, StatePhase.SHUTTING_DOWN)
    SHUTTING_DOWN_TO_TERMINATED = (StatePhase.SHUTTING_DOWN, StatePhase.TERMINATED)
    ANY_TO_ERROR = (None, StatePhase.ERROR)

    @classmethod
    def allowed(cls, src: StatePhase, dst: StatePhase) -> bool:
        return dst is StatePhase.ERROR or any(t.value == (src, dst) for t in cls)


class DistributedStrategy(Enum):
    NONE = "none"
    DDP = "ddp"
    FSDP = "fsdp"
    FSDP2 = "fsdp2"
    TENSOR_PARALLEL = "tensor_parallel"
    PIPELINE = "pipeline"


class GradientConfig(NamedTuple):
    max_norm: float = 1.0
    norm_type: float = 2.0
    clip_algorithm: str = "global"
    compression: str | None = None
    sync_before_clip: bool = False


def dist_scatter(tensor: torch.Tensor, scatter_list=None, src: int = 0, process_group=None) -> torch.Tensor:
    """Rank `src` hands element r of `scatter_list` to rank r; returns `tensor` (unchanged without a process group)."""
    if dist.is_available() and dist.is_initialized():
        dist.scatter(tensor, scatter_list=scatter_list if dist.get_rank(process_group) == src else None, src=src,
                     group=process_group)
    return tensor


@contextlib.contextmanager
def mixed_precision_context(enabled: bool = True, dtype: torch.dtype = torch.bfloat16, cache_enabled: bool = True):
    """torch autocast for modules OUTSIDE the framework (its own kernels compute in the dtype of their inputs and
    ignore autocast)."""
    if not enabled:
        yield
        return
    with torch.autocast("cuda" if torch.cuda.is_available() else "cpu", dtype=dtype, cache_enabled=cache_enabled):
        yield


def prepare_optimizer_for_distributed(optimizer, model, strategy=DistributedStrategy.DDP):
    """An optimizer built on the module's parameters needs nothing under DDP.  Under the sharded engine the ENGINE owns
    the update (fp32 master shards, fused AdamW): a torch optimizer passed here would update full-size parameters
    the engine overwrites, so that combination is refused."""
    kind = getattr(strategy, "value", strategy)
    if kind in ("fsdp", "fsdp2") and not hasattr(optimizer, "engine"):
        raise ValueError("with the sharded engine the optimizer step is engine.step(); build the engine with the "
                         "optimizer's hyper-parameters instead of wrapping a torch optimizer")
    return optimizer


def prepare_scheduler_for_distributed(scheduler, state=None):
    """Schedules depend on the step count only, which every rank shares: returned unchanged."""
    return scheduler


def print_rank_0(*args, flush: bool = True, **kwargs) -> None:
    if dist.is_available() and dist.is_initialized() and dist.get_rank() != 0:
        return
    print(*args, flush=flush, **kwargs)


@contextlib.contextmanager
def no_sync(model):
    """Suspend gradient synchronisation for the micro-batches of an accumulation window: uses the `no_sync()` of a
    torch DDP module or of this framework's engines (found on the object or on its `engine` attribute); a plain module
    needs nothing."""
    target = model if hasattr(model, "no_sync") else getattr(model, "engine", None)
    if target is not None and hasattr(target, "no_sync"):
        with target.no_sync():
            yield
    else:
        yield


def allreduce_conditional_embedding_grads(model, pp_group=None) -> None:
    """Parameters replicated on every pipeline stage (marked `pipeline_parallel = True`: timestep / label embedders of
    diffusion transformers) get their gradients summed over the stages.  `model` is a module or a list of module chunks
    (interleaved schedules); a name that occurs in several local chunks is summed locally first, reduced once and
    copied back to the other chunks (data_pipeline/trainer/distributed/finalize_grads.py:87)."""
    if pp_group is None or not dist.is_initialized() or dist.get_world_size(pp_group) <= 1:
        return
    chunks = list(model) if isinstance(model, (list, tuple)) else [model]
    by_name: dict[str, list[torch.Tensor]] = {}
    for chunk in chunks:
        for name, p in chunk.named_parameters():
            if not (p.requires_grad and getattr(p, "pipeline_parallel", False)):
                continue
            g = getattr(p, "main_grad", None)
            g = g if g is not None else p.grad
            if g is None:
                continue
            if name in by_name:
                by_name[name][0].add_(g)
            by_name.setdefault(name, []).append(g)
    for name in sorted(by_name):
        first = by_name[name][0]
        dist.all_reduce(first, group=pp_group)
        for other in by_name[name][1:]:
            other.copy_(first)


# ---- environment-driven defaults of data_pipeline/trainer/distributed/sota_utils.py
import os as _os  # noqa: E402

CACHE_LINE_SIZE = 64
NCCL_BUCKET_SIZE_MB = int(_os.environ.get("TRAINSCALE_BUCKET_SIZE_MB", "25"))
MAX_ASYNC_OPS = int(_os.environ.get("TRAINSCALE_MAX_ASYNC_OPS", "8"))
