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

from ..utils.refargs import ANY, reference_kwargs


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
    # operation-level policy and hierarchy (data_pipeline/trainer/distributed/activation_checkpoint.py:219-378)
    memory_budget_fraction: float = 0.70
    checkpoint_attention: bool = True
    checkpoint_ffn: bool = True
    checkpoint_layernorm: bool = False
    checkpoint_residual: bool = False
    min_recompute_cost_threshold: float = 0.1
    max_memory_threshold_bytes: int = 100 * 2 ** 20
    hierarchy_levels: int = 2
    segment_size: int = 4
    use_reentrant: bool = False

    def with_mode(self, mode) -> "ActivationCheckpointConfig":
        import dataclasses
        return dataclasses.replace(self, mode=CheckpointMode(mode))


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

    get_memory_pressure = pressure

    @staticmethod
    def estimate_activation_memory(batch_size: int, seq_len: int, hidden_size: int, num_layers: int,
                                   num_attention_heads: int, intermediate_size: int,
                                   dtype: torch.dtype = torch.bfloat16, num_kv_heads: int | None = None,
                                   flash_attention: bool = True) -> int:
        """Bytes that a decoder of this shape keeps for backward without recomputation, +10 % for temporaries.
        Per layer and token: the residual stream into each of the two norms (2 H), the two normalised inputs (2 H),
        q / k / v after RoPE ((nh + 2 nkv) d), the attention output (H), gate and up (2 I) and the GLU product (I).
        With `flash_attention` the S x S probabilities are not kept (only a per-row log-sum-exp, 4 bytes per head and
        token); without it they are, which is the term that dominates the reference's estimate
        (data_pipeline/trainer/distributed/activation_checkpoint.py:487-570)."""
        e = torch.finfo(dtype).bits // 8 if dtype.is_floating_point else torch.iinfo(dtype).bits // 8
        nh, nkv = num_attention_heads, num_kv_heads or num_attention_heads
        d = hidden_size // nh
        tokens = batch_size * seq_len
        per_token = (5 * hidden_size + (nh + 2 * nkv) * d + 3 * intermediate_size) * e
        attn = batch_size * nh * seq_len * (4 if flash_attention else seq_len * e)
        return int((tokens * per_token + attn) * num_layers * 1.1)

    def profile_layer(self, module: nn.Module, name: str, input_tensor: torch.Tensor) -> "LayerProfile":
        """Measures what `module` keeps for backward on `input_tensor` (saved-tensor hooks around one forward; weights
        excluded) and classifies it by its class name; when the forward cannot be run with this input alone the
        estimate is twice the input's size."""
        cls = type(module).__name__.lower()
        kind = (OperationType.ATTENTION if "attn" in cls or "attention" in cls else
                OperationType.FFN if any(k in cls for k in ("mlp", "ffn", "feedforward", "moe")) else
                OperationType.LAYERNORM if "norm" in cls else
                OperationType.EMBEDDING if "embed" in cls else OperationType.CUSTOM)
        weights = {p.data_ptr() for p in module.parameters()}      # by address: autograd saves views of weights
        seen, saved = set(), [0]

        def pack(t):
            if t.data_ptr() not in weights and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                saved[0] += t.numel() * t.element_size()
            return t

        try:
            with torch.enable_grad(), torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t):
                module(input_tensor.detach().requires_grad_(input_tensor.is_floating_point()))
            act = saved[0]
        except Exception:   # noqa: BLE001 - modules that need more than one input
            act = 2 * input_tensor.numel() * input_tensor.element_size()
        params = sum(p.numel() for p in module.parameters())
        tokens = input_tensor.numel() // max(1, input_tensor.shape[-1]) if input_tensor.dim() > 1 else input_tensor.numel()
        cost = {OperationType.ATTENTION: 0.8, OperationType.FFN: 0.6, OperationType.LAYERNORM: 0.05,
                OperationType.ACTIVATION: 0.02}.get(kind, 0.5)
        prof = LayerProfile(name, kind, act, 2 * params * tokens, cost, kind is OperationType.ATTENTION,
                            kind is OperationType.FFN)
        self.__dict__.setdefault("layer_profiles", {})[name] = prof
        return prof

    def record_checkpoint_metrics(self, metrics: "CheckpointMetrics") -> None:
        lst = self.__dict__.setdefault("checkpoint_metrics", [])
        lst.append(metrics)
        if len(lst) > 10000:
            del lst[:5000]

    def get_statistics(self) -> dict:
        ms = self.__dict__.get("checkpoint_metrics", [])
        return {"peak_memory_bytes": max((x["peak"] for x in self.snapshots), default=0),
                "snapshot_count": len(self.snapshots), "profiled_layers": len(self.__dict__.get("layer_profiles", {})),
                "checkpoint_operations": len(ms), "total_memory_saved_bytes": sum(m.memory_saved_bytes for m in ms),
                "total_recompute_time_ns": sum(m.recompute_time_ns for m in ms)}

    def clear(self) -> None:
        self.snapshots.clear()
        self.__dict__.get("layer_profiles", {}).clear()
        self.__dict__.get("checkpoint_metrics", []).clear()


class SelectiveCheckpointPolicy:
    """Which layers are recomputed (`layers_to_checkpoint`) and, inside a layer, which kinds of operation
    (`should_checkpoint`, `should_checkpoint_op`)."""

    _KINDS = {"attention": ("attention", "attn"), "ffn": ("mlp", "ffn", "feed_forward", "feedforward"),
              "layernorm": ("layernorm", "layer_norm", "rmsnorm", "rms_norm"), "residual": ("residual", "skip")}

    @reference_kwargs(config="cfg")
    def __init__(self, cfg: ActivationCheckpointConfig | None = None, num_layers: int = 0):
        self.cfg, self.L = cfg or ActivationCheckpointConfig(), num_layers
        self.config = self.cfg
        self._decisions: dict[str, bool] = {}
        for kind, words in self._KINDS.items():
            for w in words:
                self._decisions[w] = bool(getattr(self.cfg, f"checkpoint_{kind}"))

    def should_checkpoint(self, op_name: str, activation_size_bytes: int = 0, recompute_cost: float = 0.5,
                          memory_pressure: float | None = None) -> bool:
        """A named operation is recomputed when its kind is switched on and it is not trivially cheap; an operation of
        no known kind when it keeps more than `max_memory_threshold_bytes`, or - unless cheap - when device memory is
        more than 85 % in use (data_pipeline/trainer/distributed/activation_checkpoint.py:1283-1324)."""
        low = op_name.lower()
        cheap = recompute_cost < self.cfg.min_recompute_cost_threshold
        for word in sorted(self._decisions, key=len, reverse=True):
            if word in low:
                return self._decisions[word] and not cheap
        if activation_size_bytes > self.cfg.max_memory_threshold_bytes:
            return True
        if cheap:
            return False
        pressure = MemoryProfiler().pressure() if memory_pressure is None else memory_pressure
        return pressure > 0.85

    def should_checkpoint_op(self, op_type) -> bool:
        return self.should_checkpoint(getattr(op_type, "value", str(op_type)))

    def update_from_profile(self, layer_profile) -> None:
        """A layer seen to keep more than twice the size threshold is always recomputed from now on; one whose
        recomputation is nearly free never is."""
        if layer_profile.activation_memory_bytes > 2 * self.cfg.max_memory_threshold_bytes:
            self._decisions[layer_profile.name.lower()] = True
        elif layer_profile.recompute_cost < self.cfg.min_recompute_cost_threshold / 2:
            self._decisions[layer_profile.name.lower()] = False

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
    @reference_kwargs(config="cfg")
    def __init__(self, cfg: ActivationCheckpointConfig | None = None):
        self.cfg = cfg or ActivationCheckpointConfig()
        self.config = self.cfg
        self.profiler = MemoryProfiler()
        self._stats = {"layers_wrapped": 0, "applications": 0}

    # ---- one-call forms (data_pipeline/trainer/distributed/activation_checkpoint.py:2079-2170): return the model
    @staticmethod
    def _applied(model, cfg: ActivationCheckpointConfig):
        ac = ActivationCheckpoint(cfg)
        model._ts_checkpointed_layers = ac.apply(model)
        model._ts_activation_checkpoint = ac
        return model

    @staticmethod
    def apply_full(model):
        return ActivationCheckpoint._applied(model, ActivationCheckpointConfig(CheckpointMode.FULL))

    @staticmethod
    def apply_selective(model, frequency: int = 2):
        return ActivationCheckpoint._applied(model, ActivationCheckpointConfig(CheckpointMode.SELECTIVE, int(frequency)))

    @staticmethod
    def apply_memory_budget(model, budget: float = 0.7, batch_size: int = 1, seq_len: int = 4096,
                            total_bytes: int | None = None):
        """Recompute as many of the earliest layers as needed for the kept activations to fit `budget` x device memory
        (`total_bytes` replaces the device's size, e.g. off-GPU) after the weights; the per-layer size comes from
        `MemoryProfiler.estimate_activation_memory` for the model's own shape."""
        c = model.config
        per_layer = MemoryProfiler.estimate_activation_memory(batch_size, seq_len, c.hidden_size, 1, c.num_attention_heads,
                                                              c.intermediate_size, torch.bfloat16,
                                                              getattr(c, "num_key_value_heads", None))
        if total_bytes is None:
            total_bytes = torch.cuda.mem_get_info()[1] if torch.cuda.is_available() else 0
        weights = sum(p.numel() * p.element_size() for p in model.parameters())
        room = max(0.0, budget * total_bytes - weights)
        cfg = ActivationCheckpointConfig(CheckpointMode.MEMORY_BUDGET, memory_budget_gb=max(room, 1.0) / 2 ** 30,
                                         bytes_per_layer=per_layer, memory_budget_fraction=budget)
        return ActivationCheckpoint._applied(model, cfg)

    @staticmethod
    def apply_hierarchical(model, levels: int = 2, segment_size: int = 4):
        cfg = ActivationCheckpointConfig(CheckpointMode.HIERARCHICAL, hierarchical_group=int(segment_size),
                                         hierarchy_levels=int(levels), segment_size=int(segment_size))
        return ActivationCheckpoint._applied(model, cfg)

    def get_statistics(self) -> dict:
        return {**self._stats, "profiler_stats": self.profiler.get_statistics(),
                "config": {"mode": CheckpointMode(self.cfg.mode).name, "frequency": self.cfg.frequency,
                           "memory_budget_fraction": self.cfg.memory_budget_fraction}}

    def clear_profiling_data(self) -> None:
        self.profiler.clear()
        self._stats = {"layers_wrapped": 0, "applications": 0}

    def apply(self, model, batch_size: int | None = None, seq_len: int | None = None):
        """Configure the framework decoder (it recomputes layer i when i % checkpoint_every == 0) or wrap generic
        `nn.ModuleList` layers with torch's checkpoint wrapper. Returns the checkpointed layer indices.

        `apply(model, batch_size, seq_len)` is the reference's form: the expected activation size of a layer is
        recorded in the statistics and the (modified) MODEL is returned, its chosen layers in
        `model._ts_checkpointed_layers` (data_pipeline/trainer/distributed/activation_checkpoint.py:1875)."""
        if batch_size is not None or seq_len is not None:
            chosen = self.apply(model)
            hidden = getattr(getattr(model, "config", None), "hidden_size", None)
            if hidden:
                self._stats["layer_activation_bytes"] = self.profiler.estimate_activation_memory(
                    int(batch_size or 1), int(seq_len or 4096), int(hidden))
            model._ts_checkpointed_layers, model._ts_activation_checkpoint = chosen, self
            return model
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
        self._stats["layers_wrapped"] += len(chosen)
        self._stats["applications"] += 1
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


@reference_kwargs(config="d")
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

    def __init__(self, min_bytes: "int | ActivationCheckpointConfig" = 1 << 20, device=None, *, config=None):
        """`ActivationOffloader(min_bytes)`, or the reference's `(config, device)`: tensors below the configuration's
        `offload_min_bytes` (1 MiB when it has none) stay on the device."""
        if isinstance(min_bytes, ActivationCheckpointConfig):
            config, min_bytes = min_bytes, None
        if config is not None and min_bytes is None or config is not None and min_bytes == 1 << 20:
            min_bytes = int(getattr(config, "offload_min_bytes", 1 << 20))
        self.config, self.device = config, device
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

    # ---- explicit, handle-addressed use (data_pipeline/trainer/distributed/activation_checkpoint.py:860-1056)
    def offload(self, tensor: torch.Tensor) -> int:
        """Copy `tensor` to a pooled host buffer (on the copy stream for a device tensor); returns the handle id."""
        table = self.__dict__.setdefault("_handles", {})
        hid = self.__dict__["_next_id"] = self.__dict__.get("_next_id", 0) + 1
        host = self.pool.get(tensor.shape, tensor.dtype)
        ev = None
        if tensor.is_cuda:
            self.d2h.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.d2h):
                host.copy_(tensor.detach(), non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.d2h)
            tensor.record_stream(self.d2h)
        else:
            host.copy_(tensor.detach())
        table[hid] = {"host": host, "event": ev, "device": tensor.device, "ready": None}
        self.offloaded_bytes += tensor.numel() * tensor.element_size()
        return hid

    def prefetch(self, handle_id: int) -> None:
        """Start bringing the tensor back on the host-to-device stream; `reload` then only waits for it."""
        h = self._handles[handle_id]
        if h["ready"] is not None:
            return
        if h["device"].type == "cuda":
            if h["event"] is not None:
                self.h2d.wait_event(h["event"])
            with torch.cuda.stream(self.h2d):
                out = h["host"].to(h["device"], non_blocking=True)
                done = torch.cuda.Event()
                done.record(self.h2d)
            h["ready"] = (out, done)
        else:
            h["ready"] = (h["host"].clone(), None)

    def reload(self, handle_id: int) -> torch.Tensor:
        self.prefetch(handle_id)
        out, done = self._handles[handle_id]["ready"]
        if done is not None:
            torch.cuda.current_stream().wait_event(done)
            out.record_stream(torch.cuda.current_stream())
        self.restored_bytes += out.numel() * out.element_size()
        return out

    def release(self, handle_id: int) -> None:
        """Give the host buffer back to the pool.  A reload in flight is waited for first."""
        h = self.__dict__.get("_handles", {}).pop(handle_id, None)
        if h is None:
            return
        if h["ready"] is not None and h["ready"][1] is not None:
            h["ready"][1].synchronize()
        elif h["event"] is not None:
            h["event"].synchronize()
        self.pool.put(h["host"])

    def clear(self) -> None:
        for hid in list(self.__dict__.get("_handles", {})):
            self.release(hid)


class ChunkOffloadHandler(ActivationOffloader):
    """Offloads the saved activations of one model chunk (a pipeline stage's micro-batch, a group of layers) and
    keeps per-chunk accounting, so that a pipeline schedule can offload chunk k while chunk k+1 computes and bring it
    back just before its backward (data_pipeline/trainer/distributed/activation_offload.py:358).

    `tensor_push` / `tensor_pop` are the pack / unpack pair of saved-tensor hooks: a tensor below
    `min_offload_tensor_size` ELEMENTS travels as ("direct", tensor); a larger one is copied to a pooled host buffer on
    the device-to-host stream and travels as ("offloaded", state).  Host tensors take the same path without streams, so
    the bookkeeping is testable without a GPU.  Tensors are filed under the group opened last by `begin_group`."""

    def __init__(self, chunk_id: int = 0, min_bytes: int = 1 << 20, min_offload_tensor_size: int | None = None,
                 cpu_tensor_pool: "PinnedTensorPool | None" = None, d2h_stream=None, h2d_stream=None):
        super().__init__(min_bytes)
        self.chunk_id = chunk_id
        self.min_offload_tensor_size = min_offload_tensor_size if min_offload_tensor_size is not None else max(1, min_bytes // 2)
        if cpu_tensor_pool is not None:
            self.pool = cpu_tensor_pool
        if d2h_stream is not None:
            self.d2h = d2h_stream
        if h2d_stream is not None:
            self.h2d = h2d_stream
        self.cpu_tensor_pool = self.pool
        self.do_offload = True
        self.vpp_rank = 0
        self.is_warmup = True
        self.offload_groups: list[OffloadTensorGroup] = []
        self._reloaded: set[int] = set()          # ids of groups whose tensors have all come back
        self._pending: dict[int, int] = {}        # group id -> tensors still on the host
        self.torch_tensor_count = 0

    @property
    def d2h_stream(self):
        return self.d2h

    @property
    def h2d_stream(self):
        return self.h2d

    def begin_group(self, name: str) -> "OffloadTensorGroup":
        g = OffloadTensorGroup(name)
        self.offload_groups.append(g)
        return g

    def reset(self) -> None:
        """Forget the groups of the finished iteration; the host pool keeps its buffers."""
        self.offload_groups, self._reloaded, self._pending = [], set(), {}
        self.torch_tensor_count = 0

    @reference_kwargs(src_tensor="src")
    def offload_tensor(self, src: torch.Tensor, use_cpu_pool: bool = True):
        """Copy `src` to the host; returns the state that `reload_tensor` takes: (device, host tensor, pooled, group)."""
        host = self.pool.get(src.shape, src.dtype) if use_cpu_pool else torch.empty(src.shape, dtype=src.dtype)
        ev = None
        if src.is_cuda:
            self.d2h.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.d2h):
                host.copy_(src.detach(), non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.d2h)
            src.record_stream(self.d2h)
        else:
            host.copy_(src.detach())
        g = self.offload_groups[-1] if self.offload_groups else self.begin_group("default")
        g.update_stats(src)
        self._pending[id(g)] = self._pending.get(id(g), 0) + 1
        self.offloaded_bytes += src.numel() * src.element_size()
        return (src.device, host, use_cpu_pool, g, ev)

    def reload_tensor(self, state) -> torch.Tensor:
        dev, host, pooled, g, ev = state
        if ev is not None:
            ev.synchronize()
        if dev.type == "cuda":
            with torch.cuda.stream(self.h2d):
                out = host.to(dev, non_blocking=True)
            torch.cuda.current_stream().wait_stream(self.h2d)
        else:
            out = host.clone()
        if pooled:
            self.pool.put(host)
        self.restored_bytes += out.numel() * out.element_size()
        left = self._pending.get(id(g), 1) - 1
        self._pending[id(g)] = left
        if left <= 0:
            self._reloaded.add(id(g))
        return out

    def tensor_push(self, tensor: torch.Tensor):
        self.torch_tensor_count += 1
        if (not self.do_offload or tensor.numel() < self.min_offload_tensor_size or isinstance(tensor, nn.Parameter)
                or getattr(tensor, "_ts_unit", None) is not None):
            return ("direct", tensor)
        return ("offloaded", self.offload_tensor(tensor.contiguous()))

    def tensor_pop(self, saved_state) -> torch.Tensor:
        tag, data = saved_state
        if tag == "direct":
            return data
        if tag == "offloaded":
            return self.reload_tensor(data)
        raise ValueError(f"unknown saved-state tag {tag!r}")

    def is_empty_chunk(self, name: str | None = None) -> bool:
        groups = [g for g in self.offload_groups if name is None or g.name == name]
        return not any(g.total_tensor_count for g in groups)

    def finish_all_groups(self, name: str | None = None) -> bool:
        """True when every group (of that name) that offloaded something has been reloaded in full."""
        return all(id(g) in self._reloaded for g in self.offload_groups
                   if (name is None or g.name == name) and g.total_tensor_count)

    def get_max_deduplicated_groups(self) -> int:
        return len({g.name for g in self.offload_groups})


class PipelineOffloadManager:
    """Activation offload for a pipeline stage: one `ChunkOffloadHandler` per in-flight micro-batch (and virtual stage),
    all sharing two copy streams and one pinned host pool (data_pipeline/trainer/distributed/activation_offload.py:531).

    Two ways to use it.  `with mgr.scope(mb):` around a micro-batch's forward (handlers keyed by micro-batch).  Or the
    schedule-driven protocol: `init_model_chunk_offload_handler(vp_size, vp_stage)` before each forward chunk,
    `with mgr:` around its forward, `pop_backward_chunk()` before each backward chunk, `reset()` between iterations.
    The order in which chunks are handed to backward is learnt in the first iteration: per virtual stage in forward
    order, later virtual stages first."""

    _instance: "PipelineOffloadManager | None" = None

    @classmethod
    def get_instance(cls) -> "PipelineOffloadManager":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    @classmethod
    def reset_instance(cls) -> None:
        cls._instance = None

    def __init__(self, min_bytes: int = 1 << 20):
        self.min_bytes = min_bytes
        self.handlers: dict[int, ChunkOffloadHandler] = {}
        cuda = torch.cuda.is_available()
        self._d2h = torch.cuda.Stream() if cuda else None
        self._h2d = torch.cuda.Stream() if cuda else None
        self._pool = PinnedTensorPool()
        self.do_offload = True
        self._warm = True
        self._vpp = 1
        self._stages: list[list[ChunkOffloadHandler]] | None = None
        self._forward: list[ChunkOffloadHandler] = []       # chunks in forward order (learnt in the first iteration)
        self._backward: list[ChunkOffloadHandler] = []      # the same chunks in backward order
        self._fi = self._bi = 0
        self._cur_f: ChunkOffloadHandler | None = None
        self._cur_b: ChunkOffloadHandler | None = None
        self._hooks = None

    # ---- keyed use
    def scope(self, micro_batch: int):
        h = self.handlers.get(micro_batch)
        if h is None:
            h = self.handlers[micro_batch] = ChunkOffloadHandler(micro_batch, self.min_bytes, cpu_tensor_pool=self._pool,
                                                                 d2h_stream=self._d2h, h2d_stream=self._h2d)
        return h.scope()

    def release(self, micro_batch: int) -> None:
        self.handlers.pop(micro_batch, None)

    def summary(self) -> str:
        return "; ".join(f"mb{k}: {h.summary()}" for k, h in sorted(self.handlers.items()))

    # ---- shared resources and totals
    @property
    def d2h_stream(self):
        return self._d2h

    @property
    def h2d_stream(self):
        return self._h2d

    @property
    def cpu_tensor_pool(self) -> PinnedTensorPool:
        return self._pool

    def _all_chunks(self):
        return list(self.handlers.values()) + self._forward

    @property
    def offload_summary_bytes(self) -> dict[str, int]:
        """Bytes offloaded so far per group name."""
        out: dict[str, int] = {}
        for h in self._all_chunks():
            for g in h.offload_groups:
                out[g.name] = out.get(g.name, 0) + g.total_offload_bytes
        return out

    @property
    def offload_summary_total_bytes(self) -> int:
        return sum(h.offloaded_bytes for h in self._all_chunks())

    def disable_offload(self) -> None:
        self.do_offload = False
        for h in self._all_chunks():
            h.do_offload = False

    def enable_offload(self) -> None:
        self.do_offload = True
        for h in self._all_chunks():
            h.do_offload = True

    # ---- schedule-driven protocol
    def reset(self) -> None:
        """Between iterations: the chunk order learnt in the first iteration is kept and replayed."""
        if self._hooks is not None:
            self.__exit__(None, None, None)
        if self._warm and self._forward:
            self._flush(final=True)
            self._warm = False
            for h in self._forward:
                h.is_warmup = False
        self._fi = self._bi = 0
        self._cur_f = self._cur_b = None
        for h in self._forward:
            h.reset()

    def _flush(self, final: bool = False) -> None:
        st = self._stages
        if st is None or not any(st):
            return
        if not final and len({len(x) for x in st}) != 1:
            return                                            # a round over the virtual stages is not complete yet
        for chunks in reversed(st):
            self._backward.extend(chunks)
        self._stages = [[] for _ in range(self._vpp)]

    def init_model_chunk_offload_handler(self, vp_size: int | None = None, vp_stage: int | None = None,
                                         min_offload_tensor_size: int = 1 << 20) -> None:
        if not self._warm:                                    # replay: next chunk of the learnt forward order
            self._cur_f = self._forward[self._fi % len(self._forward)]
            self._fi += 1
            return
        vp = 1 if vp_size is None else int(vp_size)
        if self._stages is None:
            self._vpp, self._stages = vp, [[] for _ in range(vp)]
        rank = 0 if vp_stage is None else int(vp_stage)
        if not 0 <= rank < self._vpp:
            raise ValueError(f"vp_stage {rank} outside [0, {self._vpp})")
        h = ChunkOffloadHandler(len(self._forward), min_offload_tensor_size=min_offload_tensor_size,
                                cpu_tensor_pool=self._pool, d2h_stream=self._d2h, h2d_stream=self._h2d)
        h.vpp_rank, h.do_offload = rank, self.do_offload
        self._stages[rank].append(h)
        if rank == self._vpp - 1:
            self._flush()
        self._cur_f = h
        self._forward.append(h)

    def pop_backward_chunk(self, name: str | None = None) -> None:
        """Make the next chunk that holds tensors (of group `name`) the current backward chunk."""
        if self._warm:
            self._flush(final=True)
        self._cur_b = None
        if not self.do_offload:
            return                                            # nothing was offloaded: there is no chunk to wait for
        while self._bi < len(self._backward):
            h = self._backward[self._bi]
            self._bi += 1
            if not h.is_empty_chunk(name):
                self._cur_b = h
                return
        raise RuntimeError("no non-empty backward chunk left")

    def cur_forward_chunk(self) -> "ChunkOffloadHandler | None":
        return self._cur_f

    def cur_backward_chunk(self) -> "ChunkOffloadHandler | None":
        return self._cur_b

    def __enter__(self) -> "PipelineOffloadManager":
        h = self._cur_f
        if h is None or not h.do_offload:
            return self
        self._hooks = torch.autograd.graph.saved_tensors_hooks(
            h.tensor_push, lambda st: st if isinstance(st, torch.Tensor) else h.tensor_pop(st))
        self._hooks.__enter__()
        return self

    def __exit__(self, *exc) -> None:
        if self._hooks is not None:
            hooks, self._hooks = self._hooks, None
            hooks.__exit__(*exc)


def print_offload_summary(manager=None, *, total_offload_bytes: dict | None = None) -> None:
    """Print what was offloaded.  `manager`: an offloader / pipeline manager (its `summary()`), or the reference's
    {group name: bytes} mapping (also as `total_offload_bytes=`), printed as a table; in a distributed job the bytes are
    summed over the ranks first and rank 0 prints."""
    table = total_offload_bytes if total_offload_bytes is not None else (manager if isinstance(manager, dict) else None)
    if table is None:
        print(manager.summary())
        return
    import torch.distributed as dist
    names, vals = sorted(table), torch.tensor([float(table[k]) for k in sorted(table)], dtype=torch.float64)
    on = dist.is_available() and dist.is_initialized()
    if on and dist.get_world_size() > 1:
        dist.all_reduce(vals)
    if not on or dist.get_rank() == 0:
        width = max([len(n) for n in names] + [5])
        print(f"{'group':<{width}}  {'MiB':>12}")
        for n, v in zip(names, vals.tolist()):
            print(f"{n:<{width}}  {v / 2 ** 20:>12.2f}")
        print(f"{'total':<{width}}  {float(vals.sum()) / 2 ** 20:>12.2f}")


# ------------------------------------------------------------------------------------------------ more of the policy surface
class ActivationPool:
    """Device buffers for recomputed activations, recycled by (shape, dtype): a layer's recomputation in step n reuses
    the storage its recomputation used in step n-1 instead of going through the allocator."""

    def __init__(self, max_bytes: int = 8 * 2 ** 30, *, initial_capacity: int | None = None,
                 max_capacity: int | None = None, device=None):
        """`max_bytes` bounds the bytes kept; `max_capacity` (the reference's bound) the NUMBER of buffers kept;
        `device`: where `acquire` allocates by default; `initial_capacity` is a hint only (buffers appear on release)."""
        self.max_bytes = max_bytes
        self.max_capacity, self.initial_capacity, self.device = max_capacity, initial_capacity, device
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
        if self.max_capacity is not None and sum(len(v) for v in self._free.values()) >= self.max_capacity:
            return
        self._free.setdefault((tuple(t.shape), t.dtype, str(t.device)), []).append(t.detach())
        self.bytes_cached += nb

    def clear(self) -> None:
        self._free.clear()
        self.bytes_cached = 0

    def acquire(self, shape, dtype: torch.dtype = torch.bfloat16, device=None) -> torch.Tensor:
        return self.get(shape, dtype, device if device is not None else (self.device if self.device is not None else "cpu"))

    @reference_kwargs(tensor="t")
    def release(self, t: torch.Tensor) -> None:
        self.put(t)

    @property
    def hit_rate(self) -> float:
        n = self.hits + self.misses
        return self.hits / n if n else 0.0

    def get_stats(self) -> dict:
        return {"hits": self.hits, "misses": self.misses, "hit_rate": self.hit_rate, "bytes_cached": self.bytes_cached,
                "max_bytes": self.max_bytes, "buffers_cached": sum(len(v) for v in self._free.values())}


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

    def __init__(self, layers=None, group_size: int | None = None, use_reentrant: bool = False, levels: int | None = None,
                 *, config: "ActivationCheckpointConfig | None" = None, num_layers: int | None = None):
        """`layers`: the modules of the chain.  The planning-only form `HierarchicalCheckpointManager(config,
        num_layers)` (data_pipeline/trainer/distributed/activation_checkpoint.py:1466) builds the segment hierarchy
        without modules: `segment_size` x 2^level layers per segment at each of `hierarchy_levels` levels."""
        if config is not None:
            layers, group_size = config, (num_layers if num_layers is not None else group_size)
        if isinstance(layers, ActivationCheckpointConfig):
            cfg, L = layers, int((num_layers if num_layers is not None else group_size) or 0)
            self.layers, group_size, levels = [], cfg.segment_size, cfg.hierarchy_levels
            use_reentrant = cfg.use_reentrant
        else:
            self.layers = list(layers)
            L = len(self.layers)
        self.num_layers = L
        self.group_size = group_size or max(1, int(round(L ** 0.5)))
        self.use_reentrant = use_reentrant
        self.groups = [self.layers[i:i + self.group_size] for i in range(0, L, self.group_size)]
        self.hierarchy_levels = max(1, levels or 2)
        self.segments: dict[int, list] = {}
        self.active_level = 0

    def _level(self, level: int) -> list:
        if level not in self.segments:
            size = self.group_size * 2 ** level
            base = sum(-(-self.num_layers // (self.group_size * 2 ** l)) for l in range(level))
            self.segments[level] = [CheckpointSegment(base + i, a, min(a + size, self.num_layers), level)
                                    for i, a in enumerate(range(0, self.num_layers, size))]
        return self.segments[level]

    def get_segment_for_layer(self, layer_idx: int, level: int | None = None) -> "CheckpointSegment":
        level = self.active_level if level is None else level
        if not 0 <= level < self.hierarchy_levels:
            raise ValueError(f"level {level} outside [0, {self.hierarchy_levels})")
        for seg in self._level(level):
            if layer_idx in seg:
                return seg
        raise ValueError(f"no segment holds layer {layer_idx} at level {level}")

    def should_checkpoint_layer(self, layer_idx: int) -> bool:
        """True for the last layer of each segment at the active level: its output is what the forward keeps."""
        return layer_idx == self.get_segment_for_layer(layer_idx).end_layer - 1

    def adjust_level_for_memory(self, pressure: float | None = None) -> int:
        """Finest segments above 95 % memory in use, the middle level above 85 %, the coarsest otherwise."""
        p = MemoryProfiler().pressure() if pressure is None else pressure
        self.active_level = 0 if p > 0.95 else min(1, self.hierarchy_levels - 1) if p > 0.85 else self.hierarchy_levels - 1
        return self.active_level

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

    @property
    def memory_bytes(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n * torch.empty((), dtype=self.dtype).element_size()

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

    @property
    def num_layers(self) -> int:
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

    @property
    def checkpointing(self) -> bool:
        return self.should_checkpoint()

    @classmethod
    def get_current(cls) -> "OperationCheckpointContext | None":
        """The innermost context entered by this thread."""
        import threading
        stack = cls._active.get(threading.get_ident(), [])
        return stack[-1] if stack else None

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

    # ---- tag-addressed storage and per-direction events (data_pipeline/trainer/distributed/activation_offload.py:324-355)
    def push_tensor(self, tag, tensor: torch.Tensor) -> None:
        self._tensors[tag] = tensor

    def pop_tensor(self, tag) -> torch.Tensor:
        if tag in self._handles:
            self.reload_all()
        return self._tensors.pop(tag)

    def record_offload_event(self, stream) -> None:
        if self._offload_event is not None:
            self._offload_event.record(stream)

    def wait_offload_event(self, stream) -> None:
        if self._offload_event is not None:
            stream.wait_event(self._offload_event)

    def record_reload_event(self, stream) -> None:
        if self._reload_event is not None:
            self._reload_event.record(stream)

    def wait_reload_event(self, stream) -> None:
        if self._reload_event is not None:
            stream.wait_event(self._reload_event)

    def update_stats(self, tensor: torch.Tensor) -> None:
        self.total_offload_bytes += tensor.numel() * tensor.element_size()
        self.total_tensor_count += 1


# ---- names of data_pipeline/trainer/distributed/{activation_checkpoint,activation_offload}.py: the thresholds are the
# ones `MemoryProfiler.get_memory_pressure` and the memory-budget policy use, the costs the relative recompute cost of a
# block kind (attention = 1)
from typing import Tuple as _Tuple, Union as _Union  # noqa: E402

from torch.utils.checkpoint import checkpoint as torch_checkpoint  # noqa: E402,F401

from .dist_utils import TensorPool as OffloadTensorPool  # noqa: E402,F401

TensorOrTensors = _Union[torch.Tensor, _Tuple[torch.Tensor, ...]]
PoolKey = _Tuple[_Tuple[int, ...], torch.dtype]
CACHE_LINE_BYTES, WARP_SIZE = 64, 32
PAGE_SIZE_BYTES = 4096
HBM_BANK_SIZE = 256
CHECKPOINT_ALIGNMENT = 512
MEMORY_CRITICAL_THRESHOLD, MEMORY_WARNING_THRESHOLD, MEMORY_COMFORTABLE_THRESHOLD = 0.95, 0.85, 0.70
RECOMPUTE_COST_ATTENTION, RECOMPUTE_COST_FFN, RECOMPUTE_COST_LAYERNORM, RECOMPUTE_COST_ACTIVATION = 1.0, 0.5, 0.05, 0.01
