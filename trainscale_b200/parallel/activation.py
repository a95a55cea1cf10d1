"""Activation checkpointing policies and activation offload to pinned host memory.

After data_pipeline/trainer/distributed/activation_checkpoint.py:85-2356 (modes NONE / SELECTIVE (every n-th layer) /
MEMORY_BUDGET / FULL / OFFLOAD / HIERARCHICAL, `MemoryProfiler`, `ActivationCheckpoint.apply`) and
activation_offload.py:92-910 (pinned `TensorPool`, saved-tensor hooks, d2h / h2d streams, byte summary).
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass, field
from enum import Enum
from typing import NamedTuple

import torch
import torch.nn as nn


class CheckpointMode(str, Enum):
    NONE = "none"
    SELECTIVE = "selective"
    OP_SELECTIVE = "op_selective"
    MEMORY_BUDGET = "memory_budget"
    FULL = "full"
    OFFLOAD = "offload"
    HIERARCHICAL = "hierarchical"


@dataclass
class ActivationCheckpointConfig:
    mode: CheckpointMode = CheckpointMode.SELECTIVE
    frequency: int = 2                 # SELECTIVE: recompute every n-th layer
    memory_budget_gb: float | None = None
    bytes_per_layer: float | None = None
    offload_min_bytes: int = 1 << 20
    hierarchical_group: int = 4


class MemoryProfiler:
    _inst = None

    def __new__(cls):
        if cls._inst is None:
            cls._inst = super().__new__(cls)
            cls._inst.snapshots = []
        return cls._inst

    def snapshot(self, tag: str = "") -> dict:
        if torch.cuda.is_available():
            s = {"tag": tag, "allocated": torch.cuda.memory_allocated(), "reserved": torch.cuda.memory_reserved(),
                 "peak": torch.cuda.max_memory_allocated()}
        else:
            s = {"tag": tag, "allocated": 0, "reserved": 0, "peak": 0}
        self.snapshots.append(s)
        return s

    def pressure(self) -> float:
        if not torch.cuda.is_available():
            return 0.0
        free, total = torch.cuda.mem_get_info()
        return 1.0 - free / total


class SelectiveCheckpointPolicy:
    def __init__(self, cfg: ActivationCheckpointConfig, num_layers: int):
        self.cfg, self.L = cfg, num_layers

    def layers_to_checkpoint(self) -> list[int]:
        m = CheckpointMode(self.cfg.mode)
        if m == CheckpointMode.NONE:
            return []
        if m in (CheckpointMode.FULL, CheckpointMode.OFFLOAD):
            return list(range(self.L))
        if m == CheckpointMode.MEMORY_BUDGET and self.cfg.memory_budget_gb and self.cfg.bytes_per_layer:
            keep = int(self.cfg.memory_budget_gb * 2 ** 30 // self.cfg.bytes_per_layer)
            return list(range(max(0, self.L - keep)))     # recompute the earliest layers, keep the latest
        if m == CheckpointMode.HIERARCHICAL:
            g = max(1, self.cfg.hierarchical_group)
            return [i for i in range(self.L) if i % g != g - 1]
        f = max(1, self.cfg.frequency)
        return [i for i in range(self.L) if i % f == 0]


class ActivationCheckpoint:
    def __init__(self, cfg: ActivationCheckpointConfig | None = None):
        self.cfg = cfg or ActivationCheckpointConfig()

    def apply(self, model) -> list[int]:
        """Configure the framework decoder (it recomputes layer i when i % checkpoint_every == 0) or wrap generic
        `nn.ModuleList` layers with torch's checkpoint wrapper. Returns the checkpointed layer indices."""
        inner = getattr(model, "model", model)
        layers = getattr(inner, "layers", None)
        if layers is None:
            return []
        if self.cfg.mode == CheckpointMode.OP_SELECTIVE and hasattr(model, "op_selective_recompute"):
            model.op_selective_recompute(True)      # no layer is re-run; norm / GLU outputs are rebuilt in backward
            if hasattr(inner, "gradient_checkpointing"):
                inner.gradient_checkpointing = False
            return []
        chosen = SelectiveCheckpointPolicy(self.cfg, len(layers)).layers_to_checkpoint()
        if hasattr(inner, "gradient_checkpointing"):
            inner.gradient_checkpointing = bool(chosen)
            inner.checkpoint_layers = set(chosen)
            if chosen:
                steps = sorted(set(b - a for a, b in zip(chosen, chosen[1:]))) or [1]
                inner.checkpoint_every = steps[0] if len(steps) == 1 and chosen[0] == 0 else 1
            return chosen
        from torch.distributed.algorithms._checkpoint.checkpoint_wrapper import checkpoint_wrapper
        for i in chosen:
            layers[i] = checkpoint_wrapper(layers[i])
        return chosen


def create_activation_checkpoint_from_config(d: dict | None) -> ActivationCheckpoint:
    d = dict(d or {})
    mode = d.get("ac_mode", d.get("mode", "selective"))
    return ActivationCheckpoint(ActivationCheckpointConfig(CheckpointMode(mode), int(d.get("ac_frequency", d.get("frequency", 2)))))


class PinnedTensorPool:
    """Reusable pinned host buffers keyed by (shape, dtype)."""

    def __init__(self):
        self.free: dict[tuple, list[torch.Tensor]] = {}
        self.bytes_allocated = 0

    def get(self, shape, dtype) -> torch.Tensor:
        key = (tuple(shape), dtype)
        lst = self.free.get(key)
        if lst:
            return lst.pop()
        t = torch.empty(shape, dtype=dtype, pin_memory=torch.cuda.is_available())
        self.bytes_allocated += t.numel() * t.element_size()
        return t

    def put(self, t: torch.Tensor) -> None:
        self.free.setdefault((tuple(t.shape), t.dtype), []).append(t)


class ActivationOffloader:
    """`with offloader.scope():` moves saved activations >= min_bytes to pinned host memory on a copy stream and
    brings them back on demand in backward (saved-tensor hooks)."""

    def __init__(self, min_bytes: int = 1 << 20):
        self.min_bytes = min_bytes
        self.pool = PinnedTensorPool()
        self.cuda = torch.cuda.is_available()
        self.d2h = torch.cuda.Stream() if self.cuda else None
        self.h2d = torch.cuda.Stream() if self.cuda else None
        self.offloaded_bytes = 0
        self.restored_bytes = 0

    def _pack(self, t: torch.Tensor):
        if not t.is_cuda or t.numel() * t.element_size() < self.min_bytes or isinstance(t, nn.Parameter) \
                or getattr(t, "_ts_unit", None) is not None or not t.is_contiguous():
            return t
        host = self.pool.get(t.shape, t.dtype)
        self.d2h.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.d2h):
            host.copy_(t, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.d2h)
        t.record_stream(self.d2h)
        self.offloaded_bytes += t.numel() * t.element_size()
        return ("offloaded", host, ev, t.device)

    def _unpack(self, obj):
        if not (isinstance(obj, tuple) and len(obj) == 4 and obj[0] == "offloaded"):
            return obj
        _, host, ev, dev = obj
        ev.synchronize()
        with torch.cuda.stream(self.h2d):
            out = host.to(dev, non_blocking=True)
        torch.cuda.current_stream().wait_stream(self.h2d)
        self.pool.put(host)
        self.restored_bytes += out.numel() * out.element_size()
        return out

    @contextlib.contextmanager
    def scope(self):
        if not self.cuda:
            yield self
            return
        with torch.autograd.graph.saved_tensors_hooks(self._pack, self._unpack):
            yield self

    def summary(self) -> str:
        return (f"offloaded {self.offloaded_bytes / 2 ** 30:.2f} GiB, restored {self.restored_bytes / 2 ** 30:.2f} GiB, "
                f"pinned pool {self.pool.bytes_allocated / 2 ** 30:.2f} GiB")


class ChunkOffloadHandler(ActivationOffloader):
    """Offloads the saved activations of one model chunk (a pipeline stage's micro-batch, a group of layers) and
    keeps per-chunk accounting, so that a pipeline schedule can offload chunk k while chunk k+1 computes and bring it
    back just before its backward (data_pipeline/trainer/distributed/activation_offload.py:358)."""

    def __init__(self, chunk_id: int = 0, min_bytes: int = 1 << 20):
        super().__init__(min_bytes)
        self.chunk_id = chunk_id


class PipelineOffloadManager:
    """One `ChunkOffloadHandler` per in-flight micro-batch of a pipeline stage
    (data_pipeline/trainer/distributed/activation_offload.py:531)."""

    def __init__(self, min_bytes: int = 1 << 20):
        self.min_bytes = min_bytes
        self.handlers: dict[int, ChunkOffloadHandler] = {}

    def scope(self, micro_batch: int):
        h = self.handlers.setdefault(micro_batch, ChunkOffloadHandler(micro_batch, self.min_bytes))
        return h.scope()

    def release(self, micro_batch: int) -> None:
        self.handlers.pop(micro_batch, None)

    def summary(self) -> str:
        return "; ".join(f"mb{k}: {h.summary()}" for k, h in sorted(self.handlers.items()))


def print_offload_summary(manager: "PipelineOffloadManager | ActivationOffloader") -> None:
    print(manager.summary())


# ------------------------------------------------------------------------------------------------ more of the policy surface
class ActivationPool:
    """Device buffers for recomputed activations, recycled by (shape, dtype): a layer's recomputation in step n reuses
    the storage its recomputation used in step n-1 instead of going through the allocator."""

    def __init__(self, max_bytes: int = 8 * 2 ** 30):
        self.max_bytes = max_bytes
        self._free: dict[tuple, list[torch.Tensor]] = {}
        self.bytes_cached = 0
        self.hits = self.misses = 0

    def get(self, shape, dtype: torch.dtype, device) -> torch.Tensor:
        key = (tuple(shape), dtype, str(device))
        lst = self._free.get(key)
        if lst:
            t = lst.pop()
            self.bytes_cached -= t.numel() * t.element_size()
            self.hits += 1
            return t
        self.misses += 1
        return torch.empty(shape, dtype=dtype, device=device)

    def put(self, t: torch.Tensor) -> None:
        nb = t.numel() * t.element_size()
        if self.bytes_cached + nb > self.max_bytes:
            return
        self._free.setdefault((tuple(t.shape), t.dtype, str(t.device)), []).append(t.detach())
        self.bytes_cached += nb

    def clear(self) -> None:
        self._free.clear()
        self.bytes_cached = 0


def _checkpoint_function():
    from .pipeline import CheckpointFunction as F
    return F


def __getattr__(name):          # `CheckpointFunction` lives in pipeline.py; exposed here without an import cycle
    if name == "CheckpointFunction":
        return _checkpoint_function()
    raise AttributeError(name)


class HierarchicalCheckpointManager:
    """Two-level recomputation for a chain of L layers: the chain is cut into groups of `group_size`; the forward keeps
    only each group's input (L / g tensors).  In backward a group is re-run once, and during that re-run each layer
    keeps only ITS input (g tensors), re-running itself when its turn comes.  Peak kept activations are about
    L / g + g layer inputs (minimal at g = sqrt(L)) for two extra forwards."""

    def __init__(self, layers, group_size: int | None = None, use_reentrant: bool = False):
        self.layers = list(layers)
        L = len(self.layers)
        self.group_size = group_size or max(1, int(round(L ** 0.5)))
        self.use_reentrant = use_reentrant
        self.groups = [self.layers[i:i + self.group_size] for i in range(0, L, self.group_size)]

    def kept_tensors(self) -> int:
        return len(self.groups) + self.group_size

    def _run_group(self, group, x, *args):
        from torch.utils.checkpoint import checkpoint
        for layer in group:
            x = checkpoint(layer, x, *args, use_reentrant=self.use_reentrant) if torch.is_grad_enabled() \
                else layer(x, *args)
        return x

    def forward(self, x, *args):
        from torch.utils.checkpoint import checkpoint
        for g in self.groups:
            if torch.is_grad_enabled():
                x = checkpoint(self._run_group, g, x, *args, use_reentrant=self.use_reentrant)
            else:
                x = self._run_group(g, x, *args)
        return x

    __call__ = forward


# ------------------------------------------------------------------------------------------------ reference surface
class CheckpointImpl(Enum):
    """Which checkpoint mechanism wraps a layer (data_pipeline/trainer/distributed/activation_checkpoint.py:109)."""
    NO_REENTRANT = "no_reentrant"
    REENTRANT = "reentrant"
    CUSTOM = "custom"


class OffloadTarget(Enum):
    GPU = "gpu"
    CPU_PINNED = "cpu_pinned"
    CPU_PAGED = "cpu_paged"
    NVME = "nvme"


class OperationType(Enum):
    """Kinds of operation a selective policy distinguishes: keep what is expensive to recompute (attention, GEMMs),
    recompute what is cheap and large (norms, activations, residual adds)."""
    ATTENTION = "attention"
    FFN = "ffn"
    LAYERNORM = "layernorm"
    EMBEDDING = "embedding"
    ACTIVATION = "activation"
    LINEAR = "linear"
    RESIDUAL = "residual"
    CUSTOM = "custom"


CHEAP_TO_RECOMPUTE = frozenset({OperationType.LAYERNORM, OperationType.ACTIVATION, OperationType.RESIDUAL})


class MemorySnapshot(NamedTuple):
    total_bytes: int
    allocated_bytes: int
    reserved_bytes: int
    free_bytes: int
    fragmentation_ratio: float
    timestamp_ns: int

    @classmethod
    def take(cls, device=None) -> "MemorySnapshot":
        import time
        if not torch.cuda.is_available():
            return cls(0, 0, 0, 0, 0.0, time.monotonic_ns())
        free, total = torch.cuda.mem_get_info(device)
        alloc, res = torch.cuda.memory_allocated(device), torch.cuda.memory_reserved(device)
        return cls(total, alloc, res, free, (res - alloc) / res if res else 0.0, time.monotonic_ns())


class CheckpointMetrics(NamedTuple):
    layer_name: str
    forward_time_ns: int
    recompute_time_ns: int
    memory_saved_bytes: int
    tensors_checkpointed: int
    tensors_recomputed: int


class LayerProfile(NamedTuple):
    name: str
    operation_type: OperationType
    activation_memory_bytes: int
    compute_flops: int
    recompute_cost: float
    is_attention: bool
    is_ffn: bool


@dataclass
class OffloadHandle:
    """Where an offloaded activation lives and how it comes back."""
    tensor_id: int
    shape: tuple
    dtype: torch.dtype
    device: torch.device
    target: OffloadTarget
    cpu_tensor: torch.Tensor | None = None
    nvme_path: str | None = None
    is_prefetching: bool = False
    prefetch_stream: object = None
    prefetch_event: object = None

    def __post_init__(self):
        if self.target is OffloadTarget.NVME and self.nvme_path is None:
            raise ValueError("an NVMe offload handle needs `nvme_path`")
        if self.target in (OffloadTarget.CPU_PINNED, OffloadTarget.CPU_PAGED) and self.cpu_tensor is None:
            raise ValueError("a CPU offload handle needs `cpu_tensor`")

    @classmethod
    def offload(cls, tensor_id: int, t: torch.Tensor, target: OffloadTarget = OffloadTarget.CPU_PINNED,
                nvme_path: str | None = None) -> "OffloadHandle":
        if target is OffloadTarget.NVME:
            torch.save(t.detach().cpu(), nvme_path)
            return cls(tensor_id, tuple(t.shape), t.dtype, t.device, target, nvme_path=nvme_path)
        if target is OffloadTarget.GPU:
            return cls(tensor_id, tuple(t.shape), t.dtype, t.device, target, cpu_tensor=None)
        host = torch.empty(t.shape, dtype=t.dtype, pin_memory=target is OffloadTarget.CPU_PINNED and t.is_cuda)
        host.copy_(t.detach(), non_blocking=t.is_cuda)
        return cls(tensor_id, tuple(t.shape), t.dtype, t.device, target, cpu_tensor=host)

    def restore(self) -> torch.Tensor:
        if self.target is OffloadTarget.NVME:
            return torch.load(self.nvme_path, weights_only=True).to(self.device)
        return self.cpu_tensor.to(self.device, non_blocking=True)


class CheckpointSegment:
    """Layers [start_layer, end_layer) treated as one recomputation unit at `level` of a hierarchy (0 = finest)."""

    def __init__(self, segment_id: int, start_layer: int, end_layer: int, level: int = 0):
        if end_layer <= start_layer:
            raise ValueError("a segment needs at least one layer")
        self.segment_id, self.start_layer, self.end_layer, self.level = segment_id, start_layer, end_layer, level
        self.children: list[CheckpointSegment] = []

    def __len__(self) -> int:
        return self.end_layer - self.start_layer

    def __contains__(self, layer: int) -> bool:
        return self.start_layer <= layer < self.end_layer

    def split(self, parts: int) -> list["CheckpointSegment"]:
        """Cut into `parts` nearly equal child segments one level down."""
        n, parts = len(self), max(1, min(parts, len(self)))
        cuts = [self.start_layer + (n * i) // parts for i in range(parts + 1)]
        self.children = [CheckpointSegment(self.segment_id * parts + i, a, b, max(0, self.level - 1))
                         for i, (a, b) in enumerate(zip(cuts, cuts[1:]))]
        return self.children

    def run(self, layers, x, *args, use_reentrant: bool = False):
        """Run the segment's layers as one checkpointed unit (plainly when recomputation is switched off)."""
        def body(h, *a):
            for layer in layers[self.start_layer:self.end_layer]:
                h = layer(h, *a)
            return h
        return checkpoint(body, x, *args, use_reentrant=use_reentrant)


class OperationCheckpointContext:
    """`with OperationCheckpointContext(policy, "attention") as ctx: y = ctx.run(fn, x)`: runs `fn` under a checkpoint
    when the operation kind is cheap to recompute (or the policy says so), plainly otherwise; contexts nest and the
    stack of active operation names is kept per thread."""
    _active: dict = {}

    def __init__(self, policy=None, op_name: str = "custom", enabled: bool = True):
        self.policy, self.op_name, self.enabled = policy, op_name, enabled
        try:
            self.op_type = OperationType(op_name.lower())
        except ValueError:
            self.op_type = OperationType.CUSTOM

    def should_checkpoint(self) -> bool:
        if not self.enabled or not torch.is_grad_enabled():
            return False
        decide = getattr(self.policy, "should_checkpoint_op", None)
        return bool(decide(self.op_type)) if decide is not None else self.op_type in CHEAP_TO_RECOMPUTE

    def run(self, fn, *args, **kwargs):
        return checkpoint(fn, *args, **kwargs) if self.should_checkpoint() else fn(*args, **kwargs)

    @classmethod
    def active(cls) -> list[str]:
        import threading
        return [c.op_name for c in cls._active.get(threading.get_ident(), [])]

    def __enter__(self):
        import threading
        self._active.setdefault(threading.get_ident(), []).append(self)
        return self

    def __exit__(self, *exc):
        import threading
        self._active[threading.get_ident()].pop()
        return False


def checkpoint(function, *args, use_reentrant: bool = False, preserve_rng_state: bool = True, **kwargs):
    """torch's activation checkpoint with keyword arguments allowed for `function`, obeying `no_checkpoint()`."""
    from ..utils import recompute
    if recompute.override() is False or not torch.is_grad_enabled():
        return function(*args, **kwargs)
    from torch.utils.checkpoint import checkpoint as _ckpt
    fn = (lambda *a: function(*a, **kwargs)) if kwargs else function
    return _ckpt(fn, *args, use_reentrant=use_reentrant, preserve_rng_state=preserve_rng_state)


def no_checkpoint():
    """Context manager: layers configured for recomputation run plainly (framework decoder, `checkpoint` above,
    `CheckpointSegment`, `OperationCheckpointContext`)."""
    from ..utils import recompute
    return recompute.scoped(False)


def force_checkpoint():
    """Context manager: layers configured for recomputation are checkpointed even when the model is in eval mode
    (gradients must be enabled for a checkpoint to mean anything)."""
    from ..utils import recompute
    return recompute.scoped(True)


def create_activation_checkpoint(mode: str = "selective", frequency: int = 2, memory_budget: float = 0.7,
                                 **kwargs) -> ActivationCheckpoint:
    """`ActivationCheckpoint` from a mode name: none | full | selective | memory_budget | op_selective | hierarchical |
    offload.  `memory_budget` is the fraction of the device's memory activations may use (memory_budget mode)."""
    cfg = ActivationCheckpointConfig(CheckpointMode(mode), int(frequency))
    if CheckpointMode(mode) is CheckpointMode.MEMORY_BUDGET:
        total = torch.cuda.mem_get_info()[1] if torch.cuda.is_available() else 0
        cfg.memory_budget_gb = kwargs.pop("memory_budget_gb", memory_budget * total / 2 ** 30 if total else None)
    for k, v in kwargs.items():
        if hasattr(cfg, k):
            setattr(cfg, k, v)
    return ActivationCheckpoint(cfg)


def activation_checkpoint(fn, *args, use_reentrant: bool = False, **kwargs):
    """Run `fn(*args, **kwargs)` under a checkpoint (data_pipeline/trainer/distributed/__init__.py:629)."""
    return checkpoint(fn, *args, use_reentrant=use_reentrant, **kwargs)


def wrap_activation_checkpointing(model: nn.Module, layer_cls) -> nn.Module:
    """Every submodule of type `layer_cls` recomputes its forward in backward from now on; obeys `no_checkpoint()`."""
    import functools
    for module in model.modules():
        if isinstance(module, layer_cls) and not getattr(module, "_ts_checkpointed", False):
            original = module.forward

            @functools.wraps(original)
            def checkpointed_forward(*a, _original=original, **k):
                return activation_checkpoint(_original, *a, **k)
            module.forward = checkpointed_forward
            module._ts_checkpointed = True
    return model


@dataclass
class ActivationOffloadConfig:
    """Options of activation offload (data_pipeline/trainer/distributed/activation_offload.py:67): tensors below
    `min_offload_tensor_size` ELEMENTS stay on the GPU, `offload_margin` trailing groups are never offloaded (they are
    needed again at once when backward starts)."""
    min_offload_tensor_size: int = 1 << 20
    use_pinned_memory: bool = True
    offload_margin: int = 0
    enable_warmup_stats: bool = True

    def build(self, bytes_per_element: int = 2) -> ActivationOffloader:
        return ActivationOffloader(self.min_offload_tensor_size * bytes_per_element)


class OffloadTensorGroup:
    """Tensors offloaded and reloaded together (one group per layer part: "attention", "mlp", ...), with one event per
    direction so that a consumer waits once per group."""

    def __init__(self, name: str, offload: bool = True):
        self.name, self.offload = name, offload
        self._tensors: dict = {}
        self._handles: dict = {}
        self.total_offload_bytes = 0
        self.total_tensor_count = 0
        cuda = torch.cuda.is_available()
        self._offload_event = torch.cuda.Event() if cuda else None
        self._reload_event = torch.cuda.Event() if cuda else None

    def add(self, key, t: torch.Tensor) -> None:
        self._tensors[key] = t
        self.total_tensor_count += 1

    def offload_all(self, target: OffloadTarget = OffloadTarget.CPU_PINNED, min_elements: int = 0) -> int:
        """Move the group's tensors (those of at least `min_elements`) to the host; returns the bytes moved."""
        if not self.offload:
            return 0
        moved = 0
        for i, (key, t) in enumerate(list(self._tensors.items())):
            if t.numel() < min_elements:
                continue
            self._handles[key] = OffloadHandle.offload(i, t, target)
            moved += t.numel() * t.element_size()
            del self._tensors[key]
        if self._offload_event is not None:
            self._offload_event.record()
        self.total_offload_bytes += moved
        return moved

    def reload_all(self) -> dict:
        if self._offload_event is not None:
            self._offload_event.synchronize()
        for key, h in list(self._handles.items()):
            self._tensors[key] = h.restore()
            del self._handles[key]
        if self._reload_event is not None:
            self._reload_event.record()
        return dict(self._tensors)

    def get(self, key) -> torch.Tensor:
        if key in self._handles:
            self.reload_all()
        return self._tensors[key]
