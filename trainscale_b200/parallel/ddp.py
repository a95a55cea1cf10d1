"""Replicated data parallelism: the DDP engine surface, gradient-compression hooks and hierarchical all-reduce.

After data_pipeline/trainer/distributed/ddp.py:115-1953 (bucket-size table by interconnect, GradientCompression
NONE / FP16 / BF16 / POWERSGD / TOPK, comm hooks, `HierarchicalAllReduceManager`, `SOTADDPEngine.wrap_model /
no_sync / check_health`, `DDPInitializer.init_process_group`, `create_ddp_engine`).  The engine itself is the flat
engine in NO_SHARD mode (one contiguous gradient buffer per decoder layer = one bucket, all-reduced on a side stream
as soon as the layer's backward has been queued); hooks transform a bucket before / after its all-reduce.
"""
from __future__ import annotations

import contextlib
import datetime
import os
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable

import torch
import torch.distributed as dist
import torch.nn as nn

from ..utils.refargs import ANY, reference_kwargs

from ..core.types import Err, Ok, Result

BUCKET_MB = {"b200_nvlink": (80, 40), "h100_nvlink": (50, 25), "a100_nvlink": (40, 25), "pcie": (25, 25), "cpu": (25, 25)}


def detect_gpu_topology() -> str:
    if not torch.cuda.is_available():
        return "cpu"
    name = torch.cuda.get_device_name(0)
    for k in ("B200", "H100", "A100"):
        if k in name:
            return f"{k.lower()}_nvlink"
    return "pcie"


class GradientCompression(str, Enum):
    NONE = "none"
    FP16 = "fp16"
    BF16 = "bf16"
    FP8 = "fp8"
    POWERSGD = "powersgd"
    TOPK = "topk"
    ONEBIT = "onebit"


class SyncMode(str, Enum):
    SYNC = "sync"                    # reduce at the end of backward
    ASYNC = "async"                  # reduce every bucket on a side stream while backward continues
    LOCAL_SGD = "local_sgd"          # no gradient exchange; parameters are averaged every `local_sgd_period` steps


@dataclass
class DDPConfig:
    bucket_cap_mb: int | None = None
    gradient_compression: GradientCompression = GradientCompression.NONE
    gradient_as_bucket_view: bool = True
    static_graph: bool = True
    find_unused_parameters: bool = False
    broadcast_buffers: bool = True
    powersgd_rank: int = 4
    powersgd_start_iter: int = 10
    topk_ratio: float = 0.01
    timeout_seconds: int = 1800
    hierarchical: bool = False
    use_triton_kernels: bool = False   # accepted for file compatibility; unused

    def resolved_bucket_mb(self) -> int:
        return self.bucket_cap_mb or BUCKET_MB[detect_gpu_topology()][0]

    @classmethod
    def from_dict(cls, config_dict: dict) -> "Result":
        """Ok(DDPConfig) from a plain mapping (YAML section): enum fields accept their names or values in any case,
        unknown keys are an Err(ValueError) rather than silently dropped."""
        import dataclasses
        fields = {f.name: f for f in dataclasses.fields(cls)}
        unknown = sorted(set(config_dict) - set(fields))
        if unknown:
            return Err(ValueError(f"unknown DDP options: {unknown}"))
        kw = dict(config_dict)
        try:
            if isinstance(kw.get("gradient_compression"), str):
                v = kw["gradient_compression"]
                kw["gradient_compression"] = (GradientCompression[v.upper()] if v.upper() in GradientCompression.__members__
                                              else GradientCompression(v.lower()))
            return Ok(cls(**kw))
        except (KeyError, ValueError, TypeError) as e:
            return Err(ValueError(f"invalid DDP configuration: {e}"))


# ------------------------------------------------------------------------------------------------ hooks: bucket -> averaged bucket
def allreduce_hook(group, bucket: torch.Tensor) -> torch.Tensor:
    dist.all_reduce(bucket, group=group)
    return bucket.div_(dist.get_world_size(group))


class CastCompressionHook:
    """All-reduce in fp16 / bf16 (with a pre-scale by 1/world so the sum cannot overflow), then cast back."""

    def __init__(self, dtype: torch.dtype, process_group=None):
        """`process_group`: used when the hook is called with group None (the engines of this module always pass one)."""
        self.dtype, self.process_group = dtype, process_group

    def __call__(self, group, bucket: torch.Tensor) -> torch.Tensor:
        group = group if group is not None else self.process_group
        w = dist.get_world_size(group)
        low = (bucket / w).to(self.dtype)
        dist.all_reduce(low, group=group)
        bucket.copy_(low)
        return bucket


class PowerSGDHook:
    """Rank-r PowerSGD with error feedback on 2-D views of each bucket; plain all-reduce for the first iterations."""

    @reference_kwargs({"use_error_feedback": (True, None)}, matrix_rank="rank", warmup_steps="start_iter")
    def __init__(self, rank: int = 4, start_iter: int = 10, seed: int = 0, process_group=None):
        """Error feedback is always on (without it the low-rank projection does not converge); `process_group` is used
        when the hook is called with group None."""
        self.process_group = process_group
        self.rank, self.start_iter, self.iter = rank, start_iter, 0
        self.state: dict[int, dict] = {}
        self.gen = torch.Generator().manual_seed(seed)

    def reset(self):
        self.state.clear()
        self.iter = 0

    reset_state = reset

    def __call__(self, group, bucket: torch.Tensor, key: int = 0) -> torch.Tensor:
        self.iter += 1
        group = group if group is not None else self.process_group
        w = dist.get_world_size(group)
        if self.iter <= self.start_iter or bucket.numel() < 4 * self.rank * self.rank:
            dist.all_reduce(bucket, group=group)
            return bucket.div_(w)
        n = bucket.numel()
        rows = int(n ** 0.5)
        cols = (n + rows - 1) // rows
        st = self.state.setdefault(key, {})
        if "err" not in st or st["err"].numel() != rows * cols:
            st["err"] = torch.zeros(rows * cols, dtype=torch.float32, device=bucket.device)
            st["q"] = torch.randn(cols, self.rank, generator=self.gen).to(bucket.device)
        m = torch.zeros(rows * cols, dtype=torch.float32, device=bucket.device)
        m[:n] = bucket.float()
        m = (m + st["err"]).view(rows, cols)
        p = m @ st["q"]
        dist.all_reduce(p, group=group)
        p, _ = torch.linalg.qr(p / w)
        q = m.t() @ p
        dist.all_reduce(q, group=group)
        q = q / w
        approx = p @ q.t()
        st["err"] = (m - approx).reshape(-1)
        st["q"] = q
        bucket.copy_(approx.reshape(-1)[:n])
        return bucket


class TopKSparsificationHook:
    """Keep the largest-|g| fraction per rank (error feedback for the rest), exchange (index, value) pairs."""

    @reference_kwargs({"use_triton": ANY}, k_ratio="ratio")
    def __init__(self, ratio: float = 0.01, process_group=None):
        self.ratio, self.process_group = ratio, process_group
        self.err: dict[int, torch.Tensor] = {}

    def reset_state(self) -> None:
        self.err.clear()

    def __call__(self, group, bucket: torch.Tensor, key: int = 0) -> torch.Tensor:
        group = group if group is not None else self.process_group
        w = dist.get_world_size(group)
        g = bucket.float() + self.err.get(key, 0)
        k = max(1, int(g.numel() * self.ratio))
        vals, idx = g.abs().topk(k)
        sel = g[idx]
        rest = g.clone()
        rest[idx] = 0
        self.err[key] = rest
        all_idx = [torch.empty_like(idx) for _ in range(w)]
        all_val = [torch.empty_like(sel) for _ in range(w)]
        dist.all_gather(all_idx, idx, group=group)
        dist.all_gather(all_val, sel, group=group)
        out = torch.zeros_like(g)
        for i, v in zip(all_idx, all_val):
            out.index_add_(0, i, v)
        bucket.copy_(out / w)
        return bucket


class FP16CompressionHook(CastCompressionHook):
    @reference_kwargs({"use_triton": ANY, "initial_loss_scale": ANY})   # the pre-scale by 1 / world replaces a loss scale
    def __init__(self, process_group=None):
        super().__init__(torch.float16, process_group)


class BF16CompressionHook(CastCompressionHook):
    @reference_kwargs({"use_triton": ANY, "initial_loss_scale": ANY})
    def __init__(self, process_group=None):
        super().__init__(torch.bfloat16, process_group)


class FP8CompressionHook:
    """Per-bucket absmax-scaled E4M3 payload (a quarter of fp32 traffic).  Every rank's scaled bytes are all-gathered
    and summed in fp32 locally: 8-bit floats cannot be summed by the collective without losing the small addends."""

    def __call__(self, group, bucket: torch.Tensor, key: int = 0) -> torch.Tensor:
        w = dist.get_world_size(group)
        g = bucket.float()
        scale = g.abs().max().clamp(min=1e-12) / 448.0
        q = (g / scale).to(torch.float8_e4m3fn).view(torch.uint8)
        qs = [torch.empty_like(q) for _ in range(w)]
        ss = [torch.empty_like(scale) for _ in range(w)]
        dist.all_gather(qs, q, group=group)
        dist.all_gather(ss, scale, group=group)
        out = torch.zeros_like(g)
        for qi, si in zip(qs, ss):
            out += qi.view(torch.float8_e4m3fn).float() * si
        bucket.copy_(out / w)
        return bucket


class OneBitCompressionHook:
    """1-bit gradients with error feedback: sign(g + e) scaled by mean |g + e|; what the sign loses stays in e.
    Signs travel packed 8 per byte (all-gather), scales as one float per rank."""

    def __init__(self):
        self.err: dict[int, torch.Tensor] = {}

    def __call__(self, group, bucket: torch.Tensor, key: int = 0) -> torch.Tensor:
        w = dist.get_world_size(group)
        g = bucket.float() + self.err.get(key, 0)
        scale = g.abs().mean()
        sign = g >= 0
        self.err[key] = g - torch.where(sign, scale, -scale)
        n = g.numel()
        pad = (-n) % 8
        bits = torch.cat((sign, sign.new_zeros(pad))) if pad else sign
        packed = (bits.view(-1, 8).to(torch.uint8) << torch.arange(8, device=g.device, dtype=torch.uint8)).sum(1) \
            .to(torch.uint8)
        ps = [torch.empty_like(packed) for _ in range(w)]
        ss = [torch.empty_like(scale) for _ in range(w)]
        dist.all_gather(ps, packed, group=group)
        dist.all_gather(ss, scale, group=group)
        out = torch.zeros(n + pad, dtype=torch.float32, device=g.device)
        shifts = torch.arange(8, device=g.device, dtype=torch.uint8)
        for pi, si in zip(ps, ss):
            b = ((pi.unsqueeze(1) >> shifts) & 1).reshape(-1).float()
            out += (2 * b - 1) * si
        bucket.copy_(out[:n] / w)
        return bucket


def make_hook(cfg: DDPConfig) -> Callable | None:
    c = GradientCompression(cfg.gradient_compression)
    if c == GradientCompression.FP16:
        return FP16CompressionHook()
    if c == GradientCompression.BF16:
        return BF16CompressionHook()
    if c == GradientCompression.FP8:
        return FP8CompressionHook()
    if c == GradientCompression.ONEBIT:
        return OneBitCompressionHook()
    if c == GradientCompression.POWERSGD:
        return PowerSGDHook(cfg.powersgd_rank, cfg.powersgd_start_iter)
    if c == GradientCompression.TOPK:
        return TopKSparsificationHook(cfg.topk_ratio)
    return None


class CUDATimer:
    """Event-pair timer that never blocks the host: `stop()` records, `elapsed_ms()` reads once the events are done
    (None until then).  On CPU it is a wall clock."""

    def __init__(self, device: torch.device | str | None = None):
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self._a = self._b = None
        self._t0 = self._dt = None

    def start(self) -> "CUDATimer":
        if self.cuda:
            self._a, self._b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self._a.record()
        else:
            import time
            self._t0 = time.perf_counter()
        return self

    def stop(self) -> "CUDATimer":
        if self.cuda:
            self._b.record()
        else:
            import time
            self._dt = (time.perf_counter() - self._t0) * 1e3
        return self

    def elapsed_ms(self) -> float | None:
        if self.cuda:
            return self._a.elapsed_time(self._b) if self._b is not None and self._b.query() else None
        return self._dt

    def sync_and_elapsed_ms(self) -> float:
        """Waits for the stop event, then reads (the blocking form, for measurements outside the training loop)."""
        if self.cuda and self._b is not None:
            self._b.synchronize()
        return float(self.elapsed_ms() or 0.0)

    def elapsed_us(self) -> float | None:
        ms = self.elapsed_ms()
        return None if ms is None else ms * 1e3

    def elapsed_ns(self) -> int | None:
        ms = self.elapsed_ms()
        return None if ms is None else int(ms * 1e6)

    def __enter__(self) -> "CUDATimer":
        return self.start()

    def __exit__(self, *exc) -> None:
        self.stop()

    __enter__ = start

    def __exit__(self, *exc):
        self.stop()


@dataclass
class DDPMetrics:
    steps: int = 0
    allreduce_ms: float = 0.0
    backward_ms: float = 0.0
    bytes_reduced: int = 0
    compression_ratio: float = 1.0
    skipped_syncs: int = 0

    def record_allreduce(self, nbytes: int, ms: float | None) -> None:
        self.bytes_reduced += nbytes
        if ms is not None:
            self.allreduce_ms += ms

    def bus_bandwidth_gbs(self, world: int) -> float:
        """Ring all-reduce moves 2 (w-1)/w of the payload per rank."""
        if self.allreduce_ms <= 0 or world < 2:
            return 0.0
        return self.bytes_reduced * 2 * (world - 1) / world / (self.allreduce_ms * 1e6)

    def to_dict(self) -> dict:
        return dict(self.__dict__)

    def compute_avg_latency_ms(self) -> float:
        return self.allreduce_ms / self.steps if self.steps else 0.0

    def compute_bandwidth_gbps(self) -> float:
        """Payload bytes per second of all-reduce time, in GB/s."""
        return self.bytes_reduced / (self.allreduce_ms * 1e6) if self.allreduce_ms > 0 else 0.0

    def reset(self) -> None:
        self.__init__()


class MemoryPressureMonitor:
    """Watches allocated / total device memory; above `high` it asks for relief (smaller buckets, cache release),
    above `critical` it releases the allocator cache itself.  Readings come from torch's allocator (or from the
    injected `probe`, for tests): nothing on the device is configured."""

    @reference_kwargs(high_watermark_fraction="high", critical_watermark_fraction="critical")
    def __init__(self, device: torch.device | str | None = None, high: float = 0.85, critical: float = 0.95,
                 probe: Callable[[], tuple[int, int]] | None = None):
        self.device = torch.device(device) if device is not None else None
        self.high, self.critical = high, critical
        self._probe = probe
        self.events: list[tuple[str, float]] = []

    def usage(self) -> float:
        if self._probe is not None:
            used, total = self._probe()
        elif torch.cuda.is_available():
            free, total = torch.cuda.mem_get_info(self.device)
            used = total - free
        else:
            return 0.0
        return used / total if total else 0.0

    def level(self) -> str:
        u = self.usage()
        return "critical" if u >= self.critical else "high" if u >= self.high else "normal"

    def check(self) -> str:
        lvl = self.level()
        if lvl != "normal":
            self.events.append((lvl, self.usage()))
        if lvl == "critical" and torch.cuda.is_available() and self._probe is None:
            torch.cuda.empty_cache()
        return lvl

    def get_pressure_level(self) -> int:
        """0 normal, 1 high, 2 critical."""
        return {"normal": 0, "high": 1, "critical": 2}[self.level()]

    @property
    def allocated_bytes(self) -> int:
        return torch.cuda.memory_allocated(self.device) if torch.cuda.is_available() else 0

    @property
    def reserved_bytes(self) -> int:
        return torch.cuda.memory_reserved(self.device) if torch.cuda.is_available() else 0

    def emergency_free(self) -> int:
        """Release the allocator's cached blocks; returns the bytes that went back to the driver."""
        import gc
        gc.collect()
        if not torch.cuda.is_available():
            return 0
        before = torch.cuda.memory_reserved(self.device)
        torch.cuda.empty_cache()
        return before - torch.cuda.memory_reserved(self.device)

    def suggested_bucket_mb(self, base_mb: int) -> int:
        return {"normal": base_mb, "high": max(1, base_mb // 2), "critical": max(1, base_mb // 4)}[self.level()]


class HierarchicalAllReduceManager:
    """intra-node reduce -> inter-node all-reduce among node leaders -> intra-node broadcast."""

    @reference_kwargs({"global_group": (None,)})     # the hierarchy is always built over the default (world) group
    def __init__(self, local_world: int | None = None):
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        self.local_world = local_world or int(os.environ.get("LOCAL_WORLD_SIZE", self.world))
        self.node = self.rank // self.local_world
        n_nodes = self.world // self.local_world
        self.intra = self.inter = None
        for n in range(n_nodes):
            g = dist.new_group(list(range(n * self.local_world, (n + 1) * self.local_world)))
            if n == self.node:
                self.intra = g
        leaders = [n * self.local_world for n in range(n_nodes)]
        g = dist.new_group(leaders)
        self.inter = g if self.rank in leaders else None
        self.is_leader = self.rank in leaders
        self.leader = self.node * self.local_world

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        dist.reduce(t, self.leader, group=self.intra)
        if self.is_leader and self.inter is not None:
            dist.all_reduce(t, group=self.inter)
        dist.broadcast(t, self.leader, group=self.intra)
        return t.div_(self.world)

    def create_comm_hook(self):
        """Two forms of the same reduction.  `hook(group, flat_bucket) -> averaged bucket` is what the bucket engines of
        this module take; `hook(state, bucket)` with a torch `GradBucket` returns a completed Future of the averaged
        buffer, the signature of `DistributedDataParallel.register_comm_hook`."""
        def hook(state, bucket):
            if torch.is_tensor(bucket):
                return self.all_reduce(bucket)
            fut = torch.futures.Future()
            fut.set_result(self.all_reduce(bucket.buffer()))
            return fut
        return hook


class SOTADDPEngine:
    def __init__(self, config: DDPConfig | None = None, **kw):
        self.config = config or DDPConfig(**{k: v for k, v in kw.items() if k in DDPConfig.__dataclass_fields__})
        self.hook = make_hook(self.config)
        self.engine = None

    def wrap_model(self, model: nn.Module, lr: float = 2e-5, **engine_kw):
        """Builds the flat NO_SHARD engine around `model`; the compression hook (if any) replaces the bucket
        all-reduce. Returns the model (parameters now alias the engine's buffers)."""
        from .flat_engine import EngineConfig, FlatShardedEngine
        ec = EngineConfig(sharding_strategy="NO_SHARD", lr=lr, **engine_kw)
        self.engine = FlatShardedEngine(model, ec)
        if self.hook is not None and self.engine.world > 1:
            eng, hook = self.engine, self.hook

            def reduce_with_hook(u, cur):
                hook(eng.pg if eng.pg is not None else dist.group.WORLD, u.flat_grad)
                u.reduce_event = True
            eng._reduce_ddp = reduce_with_hook
        return model

    @contextlib.contextmanager
    def no_sync(self):
        with (self.engine.no_sync() if self.engine is not None else contextlib.nullcontext()):
            yield

    # ---- accessors of the reference's engine (data_pipeline/trainer/distributed/ddp.py:1587-1672)
    rank = property(lambda self: dist.get_rank() if dist.is_available() and dist.is_initialized() else 0)
    world_size = property(lambda self: dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1)
    is_rank_zero = property(lambda self: self.rank == 0)

    def _need_engine(self):
        if self.engine is None:
            raise RuntimeError("call wrap_model() first")
        return self.engine

    def get_module(self) -> nn.Module:
        """The module that was wrapped (the engine aliases its parameters; there is no wrapper module to peel off)."""
        return self._need_engine().model

    def clip_grad_norm_(self, max_norm: float, norm_type: float = 2.0) -> torch.Tensor:
        """Clip the gradients the engine holds; the engine's own `step()` already clips to its configured
        `max_grad_norm` on the device, this is for loops that step another optimizer."""
        eng = self._need_engine()
        params = [p for p in eng.model.parameters() if p.grad is not None or getattr(p, "main_grad", None) is not None]
        for p in params:
            if p.grad is None:
                p.grad = p.main_grad
        return torch.nn.utils.clip_grad_norm_(params, max_norm, norm_type)

    def get_metrics(self) -> "DDPMetrics":
        m = self.__dict__.setdefault("_metrics", DDPMetrics())
        if self.engine is not None:
            m.steps = getattr(self.engine, "step_count", m.steps)
        return m

    def reset_metrics(self) -> None:
        self.__dict__["_metrics"] = DDPMetrics()

    def reset_compression_state(self) -> None:
        """Forget the error-feedback / low-rank state of a compression hook (after loading a checkpoint the residuals of
        the old trajectory no longer apply)."""
        reset = getattr(self.hook, "reset_state", None)
        if reset is not None:
            reset()

    def check_health(self, timeout_s: float = 30.0) -> bool:
        if not dist.is_initialized():
            return True
        t = torch.ones(1, device=self.engine.device if self.engine else "cpu")
        try:
            dist.all_reduce(t)
            return bool(t.item() == dist.get_world_size())
        except RuntimeError:
            return False


class DDPInitializer:
    @staticmethod
    def init_process_group(backend: str = "nccl", timeout_seconds: int = 1800, init_method: str | None = None,
                           world_size: int | None = None, rank: int | None = None,
                           timeout_minutes: float | None = None) -> Result:
        """env:// rendezvous from torchrun variables (or `init_method` with explicit `world_size` / `rank`). NCCL debug
        output is enabled by DDP_DEBUG=1.  `timeout_minutes` is the reference's unit for the same limit."""
        if dist.is_initialized():
            return Ok(dist.get_world_size())
        if timeout_minutes is not None:
            timeout_seconds = int(timeout_minutes * 60)
        try:
            if backend == "nccl" and not torch.cuda.is_available():
                backend = "gloo"
            if os.environ.get("DDP_DEBUG"):
                os.environ.setdefault("NCCL_DEBUG", "INFO")
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            kw = {}
            if backend == "nccl":
                lr = int(os.environ.get("LOCAL_RANK", "0"))
                torch.cuda.set_device(lr)
                kw["device_id"] = torch.device("cuda", lr)
            if init_method:
                kw["init_method"] = init_method
            if world_size is not None:
                kw["world_size"] = int(world_size)
            if rank is not None:
                kw["rank"] = int(rank)
            dist.init_process_group(backend, timeout=datetime.timedelta(seconds=timeout_seconds), **kw)
            return Ok(dist.get_world_size())
        except Exception as e:   # noqa: BLE001
            return Err(e)

    @staticmethod
    def destroy_process_group() -> None:
        """Tear the default group down if there is one (after a barrier-free wait for this rank's own work)."""
        if dist.is_available() and dist.is_initialized():
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            dist.destroy_process_group()


def create_ddp_engine(**kw) -> Result:
    try:
        return Ok(SOTADDPEngine(**kw))
    except (TypeError, ValueError) as e:
        return Err(e)


# ------------------------------------------------------------------------------------------------ reference surface
from enum import IntEnum  # noqa: E402


class AllReduceAlgorithm(IntEnum):
    RING = 0
    RECURSIVE_HALVING = 1
    BUCKET_RECURSIVE = 2
    NCCL_AUTO = 3


class BucketSchedule(IntEnum):
    """Order in which gradient buckets are reduced: as they fill (FIFO), last layer first (REVERSE: the order backward
    produces them), largest first, or intra-node before inter-node."""
    FIFO = 0
    REVERSE = 1
    SIZE_PRIORITY = 2
    TOPOLOGY_AWARE = 3


class GradientCompressionHook:
    """Base of the bucket hooks: `hook(group, bucket) -> averaged bucket`.  Subclasses override `compress` /
    `decompress`; the base implementation all-reduces the compressed form and averages
    (data_pipeline/trainer/distributed/ddp.py:796-830)."""

    def __init__(self, process_group=None):
        ready = dist.is_available() and dist.is_initialized()
        self._process_group = process_group or (dist.group.WORLD if ready else None)
        self._world_size = dist.get_world_size(self._process_group) if ready else 1
        self._rank = dist.get_rank(self._process_group) if ready else 0
        self._metrics = DDPMetrics()
        self.__name__ = type(self).__name__

    def compress(self, bucket: torch.Tensor) -> torch.Tensor:
        return bucket

    def decompress(self, payload: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
        return payload.to(like.dtype)

    @property
    def metrics(self) -> DDPMetrics:
        """Bytes put on the wire (after compression) and the compression ratio of the last bucket."""
        return self._metrics

    def __call__(self, group, bucket: torch.Tensor) -> torch.Tensor:
        group = group if group is not None else self._process_group
        payload = self.compress(bucket)
        sent = payload.numel() * payload.element_size()
        self._metrics.record_allreduce(sent, None)
        self._metrics.compression_ratio = bucket.numel() * bucket.element_size() / max(sent, 1)
        if self._world_size > 1:
            dist.all_reduce(payload, group=group)
        bucket.copy_(self.decompress(payload, bucket).div_(self._world_size))
        return bucket


def create_ddp_from_yaml(config_path: str):
    """`SOTADDPEngine` from the `distributed.ddp` section of a YAML file, as a Result."""
    try:
        import yaml
        with open(config_path) as f:
            section = (yaml.safe_load(f) or {}).get("distributed", {}).get("ddp", {})
        return create_ddp_engine(**section)
    except Exception as e:   # noqa: BLE001 - reported through the Result
        return Err(e)


# ---- names of data_pipeline/trainer/distributed/ddp.py
from torch.nn.parallel import DistributedDataParallel as TorchDDP  # noqa: E402,F401

SOTADDP = SOTADDPEngine
