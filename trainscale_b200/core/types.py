"""Result type used by the data half of the API (`DataPipeline.from_config(...) -> Result`).

Same surface as data_pipeline/core/types.py:27-240 (Ok / Err / is_ok / unwrap / map_result / flat_map /
map_err), written as two small frozen dataclasses with methods, plus the free functions.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Generic, TypeVar, Union
from ..utils.refargs import ANY, reference_kwargs

T = TypeVar("T")
U = TypeVar("U")
E = TypeVar("E")
F = TypeVar("F")


@dataclass(frozen=True)
class Ok(Generic[T]):
    value: T

    def is_ok(self) -> bool:
        return True

    def is_err(self) -> bool:
        return False

    def unwrap(self) -> T:
        return self.value

    def unwrap_or(self, default):
        return self.value

    def map(self, fn):
        return Ok(fn(self.value))

    def and_then(self, fn):
        return fn(self.value)

    def map_err(self, fn):
        return self

    def __repr__(self):
        return f"Ok({self.value!r})"


@dataclass(frozen=True)
class Err(Generic[E]):
    error: E

    def is_ok(self) -> bool:
        return False

    def is_err(self) -> bool:
        return True

    def unwrap(self):
        if isinstance(self.error, BaseException):
            raise self.error
        raise ValueError(f"called unwrap on Err: {self.error!r}")

    def unwrap_or(self, default):
        return default

    def map(self, fn):
        return self

    def and_then(self, fn):
        return self

    def map_err(self, fn):
        return Err(fn(self.error))

    def __repr__(self):
        return f"Err({self.error!r})"


Result = Union[Ok[T], Err[E]]


@reference_kwargs(result="r")
def is_ok(r) -> bool:
    return isinstance(r, Ok)


@reference_kwargs(result="r")
def is_err(r) -> bool:
    return isinstance(r, Err)


@reference_kwargs(result="r")
def unwrap(r):
    return r.unwrap()


@reference_kwargs(result="r")
def unwrap_err(r):
    if isinstance(r, Err):
        return r.error
    raise ValueError(f"called unwrap_err on Ok: {r.value!r}")


@reference_kwargs(result="r")
def unwrap_or(r, default):
    return r.value if isinstance(r, Ok) else default


@reference_kwargs(result="r", f="fn")
def unwrap_or_else(r, fn: Callable):
    return r.value if isinstance(r, Ok) else fn(r.error)


@reference_kwargs(result="r", f="fn")
def map_result(r, fn: Callable):
    return Ok(fn(r.value)) if isinstance(r, Ok) else r


@reference_kwargs(result="r", f="fn")
def flat_map(r, fn: Callable):
    return fn(r.value) if isinstance(r, Ok) else r


@reference_kwargs(result="r", f="fn")
def map_err(r, fn: Callable):
    return Err(fn(r.error)) if isinstance(r, Err) else r


# ------------------------------------------------------------------------------------------------ training records
import enum  # noqa: E402
from typing import Dict, Optional  # noqa: E402


class WarmupType(str, enum.Enum):
    """How the learning rate ramps up (data_pipeline/trainer/core/types.py:440)."""
    NONE = "none"
    LINEAR = "linear"
    EXPONENTIAL = "exponential"
    CONSTANT = "constant"


class CheckpointStrategy(str, enum.Enum):
    STEPS = "steps"
    EPOCH = "epoch"
    BEST = "best"
    BEST_AND_LAST = "best_and_last"
    NO = "no"


@dataclass(frozen=True)
class GradientInfo:
    """Gradient statistics of one step (data_pipeline/trainer/core/types.py:652)."""
    global_norm: float
    max_norm: float
    min_norm: float
    clipped: bool
    overflow: bool
    scale_factor: float = 1.0
    layer_norms: Optional[Dict[str, float]] = None


@dataclass(frozen=True)
class StepMetrics:
    loss: float
    lr: float
    grad_norm: float
    throughput: float
    gpu_memory_mb: float
    step_time_ms: float
    component_losses: Optional[Dict[str, float]] = None


# ---- type variables and numeric defaults of data_pipeline/trainer/core/types.py
from typing import TypeVar as _TypeVar  # noqa: E402

ModelT = _TypeVar("ModelT")
OptimizerT = _TypeVar("OptimizerT")
CACHE_LINE_SIZE: int = 64                  # bytes, host L1 line
GPU_WARP_SIZE: int = 32                    # threads per warp
TPU_TILE_SIZE: int = 128                   # kept for scripts that import it; nothing here targets TPUs
MAX_GRADIENT_NORM: float = 1.0             # default clipping threshold of the trainer
DEFAULT_WARMUP_RATIO: float = 0.1
