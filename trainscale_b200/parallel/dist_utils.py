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
import os
import random
import time
from dataclasses import dataclass
from enum import Enum

import numpy as np
import torch
import torch.distributed as dist

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
    def initialize(cls, backend: str | None = None, timeout_s: int = 1800) -> "DistributedState":
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

    def barrier(self):
        if dist.is_initialized():
            dist.barrier()

    def shutdown(self):
        if self.initialized_here and dist.is_initialized():
            dist.destroy_process_group()
            self.initialized_here = False


class NanoTimer:
    """Device timer: `with timer("fwd"):` records two CUDA events; durations are read by `flush()` for events that
    have completed (no synchronisation)."""

    def __init__(self):
        self.cuda = torch.cuda.is_available()
        self.pending: list[tuple[str, object, object]] = []
        self.totals: dict[str, float] = {}
        self.counts: dict[str, int] = {}

    @contextlib.contextmanager
    def __call__(self, name: str):
        if self.cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            yield
            b.record()
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


CUDATimer = NanoTimer


@torch.no_grad()
def fused_clip_grad_norm_(parameters, max_norm: float, group=None) -> torch.Tensor:
    """Global L2 norm over `.grad` (all-reduced over `group` for sharded grads), coefficient max_norm / (norm + 1e-6)
    clamped to 1, applied in place. The coefficient stays on the device."""
    grads = [p.grad for p in parameters if p.grad is not None]
    if not grads:
        return torch.zeros(())
    sq = torch.stack([g.float().pow(2).sum() for g in grads]).sum()
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(sq, group=group)
    norm = sq.sqrt()
    coef = (max_norm / (norm + 1e-6)).clamp(max=1.0)
    for g in grads:
        g.mul_(coef.to(g.dtype))
    return norm


def dist_reduce(t: torch.Tensor, op: str = "mean", group=None) -> torch.Tensor:
    if not (dist.is_initialized() and dist.get_world_size(group) > 1):
        return t
    t = t.clone()
    dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM, group=group)
    return t / dist.get_world_size(group) if op == "mean" else t


def dist_all_gather(t: torch.Tensor, group=None) -> list[torch.Tensor]:
    if not (dist.is_initialized() and dist.get_world_size(group) > 1):
        return [t]
    out = [torch.empty_like(t) for _ in range(dist.get_world_size(group))]
    dist.all_gather(out, t.contiguous(), group=group)
    return out


def set_deterministic_seed(seed: int, rank: int = 0, fully_deterministic: bool = False) -> int:
    s = seed + rank
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

    def state_dict(self):
        return {"scale": self.scale_value, "good": self._good}

    def load_state_dict(self, sd):
        self.scale_value, self._good = sd["scale"], sd["good"]


def log_rank_0(msg: str, level: int = logging.INFO):
    if not dist.is_initialized() or dist.get_rank() == 0:
        logger.log(level, msg)


@contextlib.contextmanager
def main_process_first():
    """Rank 0 runs the block first (e.g. dataset preprocessing with a cache), the others after it."""
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
