"""Contiguous parameter / gradient buffers with bucketed collectives and a ZeRO-1 sharded optimizer on top.

The same building blocks as data_pipeline/trainer/distributed/grad_buffer.py:87-1096 (`shard_buffer`,
`ParamAndGradBucket`, `ParamAndGradBucketGroup` with `start_param_sync` / `start_grad_sync` / `register_grad_ready`,
`ParamAndGradBuffer` with padded, aligned buckets and host offload, `partition_buckets`), plus the optimizer that the
reference leaves to the caller: `DistributedOptimizer` keeps fp32 master weights and AdamW moments only for this rank's
shard of every bucket, steps them with the flat AdamW kernel and all-gathers the updated bf16 parameters.

The trainer's own data-parallel path is `flat_engine.FlatShardedEngine` (per-layer units, collectives fused into
kernels over peer memory); this module is the library-level API for models that do not go through the trainer.
"""
from __future__ import annotations

from enum import Enum
from typing import Iterable, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import optim as K

ALIGN_ELEMS = 64          # 128 bytes of bf16: every parameter starts on a 128-byte boundary


class BufferType(Enum):
    PARAM = "param"
    GRAD = "grad"


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def _rank(group) -> int:
    return dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0


def shard_buffer(buffer: torch.Tensor, data_parallel_world_size: int) -> list[torch.Tensor]:
    """Equal views of a 1-D buffer, one per data-parallel rank (numel must divide)."""
    if buffer.dim() != 1 or buffer.numel() % data_parallel_world_size:
        raise ValueError(f"a 1-D buffer whose length divides by {data_parallel_world_size} is required")
    n = buffer.numel() // data_parallel_world_size
    return [buffer[r * n:(r + 1) * n] for r in range(data_parallel_world_size)]


class ParamAndGradBucket:
    """A contiguous slice of a buffer: the unit of one collective."""

    __slots__ = ("params_list", "params", "param_data", "grad_data", "offset", "numel_unpadded",
                 "gradient_scaling_factor", "bucket_id", "param_to_index")

    def __init__(self, params: Sequence[nn.Parameter], param_data: torch.Tensor | None, grad_data: torch.Tensor,
                 offset: int, numel_unpadded: int, gradient_scaling_factor: float, bucket_id: int,
                 param_to_index: dict):
        self.params_list = list(params)
        self.params = set(params)
        self.param_data, self.grad_data = param_data, grad_data
        self.offset, self.numel_unpadded = offset, numel_unpadded
        self.gradient_scaling_factor = gradient_scaling_factor
        self.bucket_id = bucket_id
        self.param_to_index = param_to_index      # param -> (start, end) inside this bucket

    @property
    def numel(self) -> int:
        return self.grad_data.numel()


def _is_ddp_config(x) -> bool:
    """A data-parallel configuration object (any class carrying the switches), as opposed to a process group."""
    return x is not None and any(hasattr(x, n) for n in ("use_distributed_optimizer", "overlap_grad_reduce",
                                                          "average_in_collective", "overlap_param_gather"))


class ParamAndGradBucketGroup:
    """Buckets whose collectives are issued together.  Gradient side: all-reduce, or reduce-scatter into this rank's
    shard when the distributed optimizer is on.  Parameter side: all-gather of the updated shards."""

    def __init__(self, buckets: Sequence[ParamAndGradBucket], group=None, use_distributed_optimizer: bool = False,
                 overlap_grad_reduce: bool = True, overlap_param_gather: bool = False, average: bool = True, *,
                 ddp_config=None, collective_group=None, collective_group_size: int | None = None):
        """`ParamAndGradBucketGroup(buckets, group, use_distributed_optimizer, ...)`, or the reference's `(buckets,
        ddp_config, collective_group, collective_group_size)`: the switches are then read from the configuration object
        (`use_distributed_optimizer`, `overlap_grad_reduce`, `overlap_param_gather`, `average_in_collective`)
        (data_pipeline/trainer/distributed/grad_buffer.py:262)."""
        if _is_ddp_config(group):                                        # positional (buckets, ddp_config, group, size)
            ddp_config, group = group, None
            if not isinstance(use_distributed_optimizer, bool):
                collective_group, use_distributed_optimizer = use_distributed_optimizer, False
            if not isinstance(overlap_grad_reduce, bool):
                collective_group_size, overlap_grad_reduce = int(overlap_grad_reduce), True
        if ddp_config is not None:
            use_distributed_optimizer = bool(getattr(ddp_config, "use_distributed_optimizer", False))
            overlap_grad_reduce = bool(getattr(ddp_config, "overlap_grad_reduce", False))
            overlap_param_gather = bool(getattr(ddp_config, "overlap_param_gather", False))
            average = bool(getattr(ddp_config, "average_in_collective", True))
        group = collective_group if collective_group is not None else group
        if collective_group_size is not None and int(collective_group_size) != _world(group):
            raise ValueError(f"collective_group_size={collective_group_size} but the group has {_world(group)} ranks")
        self.ddp_config = ddp_config
        self.buckets = list(buckets)
        self.group = group
        self.world, self.rank = _world(group), _rank(group)
        self.use_distributed_optimizer = use_distributed_optimizer
        self.overlap_grad_reduce, self.overlap_param_gather = overlap_grad_reduce, overlap_param_gather
        self.average = average
        self.params = set().union(*[b.params for b in self.buckets]) if self.buckets else set()
        self.params_with_grad: set = set()
        self.grad_handles: list = []
        self.param_handles: list = []
        self.is_last_microbatch = True
        self.next_param_gather_bucket_group: "ParamAndGradBucketGroup | None" = None
        self.grad_sync_dispatched = False

    def reset(self) -> None:
        self.params_with_grad.clear()
        self.grad_handles.clear()
        self.grad_sync_dispatched = False
        self.is_last_microbatch = True

    def check_grads(self, check_for_nan_or_inf: bool = True, check_for_large: bool = False,
                    large_threshold: float = 1e6) -> None:
        for b in self.buckets:
            n = b.grad_data.float().norm()
            if check_for_nan_or_inf and not torch.isfinite(n):
                raise FloatingPointError(f"non-finite gradient norm in bucket {b.bucket_id} before its collective")
            if check_for_large and float(n) > large_threshold:
                raise FloatingPointError(f"gradient norm {float(n):.3e} in bucket {b.bucket_id} exceeds "
                                         f"{large_threshold:.1e}")

    # ---------------------------------------------------------------- parameters
    def start_param_sync(self, force_sync: bool = False) -> None:
        """All-gather every bucket's parameter shards (distributed optimizer only)."""
        if not self.use_distributed_optimizer:
            return
        async_op = self.overlap_param_gather and not force_sync
        self.param_handles = []
        for b in self.buckets:
            if self.world == 1:
                continue
            mine = shard_buffer(b.param_data, self.world)[self.rank]
            h = dist.all_gather_into_tensor(b.param_data, mine.clone(), group=self.group, async_op=async_op)
            if async_op:
                self.param_handles.append(h)

    def finish_param_sync(self, skip_next_bucket_dispatch: bool = False) -> None:
        for h in self.param_handles:
            h.wait()
        self.param_handles = []
        nxt = self.next_param_gather_bucket_group
        if nxt is not None and not skip_next_bucket_dispatch and not nxt.param_handles:
            nxt.start_param_sync()

    # ---------------------------------------------------------------- gradients
    def start_grad_sync(self, force_all_reduce: bool = False) -> None:
        """Scale, then reduce-scatter (distributed optimizer) or all-reduce every bucket."""
        if self.grad_sync_dispatched:
            raise RuntimeError("gradient sync of this bucket group was already dispatched in this step")
        async_op = self.overlap_grad_reduce
        for b in self.buckets:
            f = b.gradient_scaling_factor * ((1.0 / self.world) if self.average else 1.0)
            if f != 1.0:
                b.grad_data.mul_(f)
            if self.world == 1:
                continue
            if self.use_distributed_optimizer and not force_all_reduce:
                mine = shard_buffer(b.grad_data, self.world)[self.rank]
                h = dist.reduce_scatter_tensor(mine, b.grad_data, group=self.group, async_op=async_op)
            else:
                h = dist.all_reduce(b.grad_data, group=self.group, async_op=async_op)
            if async_op:
                self.grad_handles.append(h)
        self.grad_sync_dispatched = True

    def finish_grad_sync(self, force_all_reduce: bool = False) -> None:
        if not self.grad_sync_dispatched:
            self.start_grad_sync(force_all_reduce)
        for h in self.grad_handles:
            h.wait()
        self.grad_handles = []

    def register_grad_ready(self, param: nn.Parameter, force_all_reduce: bool = False) -> None:
        """Called from the gradient hook of `param`; the last one of the group (on the last micro-batch) fires the
        collective while the rest of the backward is still running."""
        if not self.overlap_grad_reduce:
            return
        if param not in self.params:
            raise KeyError("parameter does not belong to this bucket group")
        if not self.is_last_microbatch:
            return
        self.params_with_grad.add(param)
        if len(self.params_with_grad) == len(self.params):
            self.start_grad_sync(force_all_reduce)


class ParamAndGradBuffer:
    """One flat parameter buffer (optional) and one flat gradient buffer for a set of parameters of one dtype.

    Parameters are laid out in REVERSE order (backward produces the last layers' gradients first, so bucket 0 fills
    first), each starting on a 128-byte boundary; a bucket closes once it holds `bucket_size` elements and is padded to
    a multiple of world * 64 elements so that it shards evenly.  `p.data` is re-pointed into the parameter buffer and
    `p.main_grad` is a view of the gradient buffer; backward hooks add `p.grad` into it."""

    def __init__(self, params: Iterable[nn.Parameter], param_dtype: torch.dtype = torch.bfloat16,
                 grad_dtype: torch.dtype = torch.float32, group=None, bucket_size: int | None = 40_000_000,
                 use_distributed_optimizer: bool = False, gradient_scaling_factor: float = 1.0,
                 device: torch.device | str | None = None, install_hooks: bool = True, *, ddp_config=None,
                 data_parallel_group=None, param_to_name: dict | None = None):
        """`ParamAndGradBuffer(params, param_dtype, grad_dtype, group, bucket_size, ...)`, or the reference's
        `(ddp_config, param_dtype, grad_dtype, params, data_parallel_group, bucket_size, param_to_name,
        gradient_scaling_factor)`: `use_distributed_optimizer` then comes from the configuration object, and
        `param_to_name` labels parameters in error messages (data_pipeline/trainer/distributed/grad_buffer.py:703)."""
        if _is_ddp_config(params):                                       # the reference's positional order
            ref = (params, group, bucket_size, use_distributed_optimizer, gradient_scaling_factor, device)
            ddp_config, params = ref[0], ref[1]
            data_parallel_group = ref[2] if not isinstance(ref[2], int) else data_parallel_group
            bucket_size = ref[3] if isinstance(ref[3], int) and not isinstance(ref[3], bool) else \
                (ref[2] if isinstance(ref[2], int) else 40_000_000)
            if isinstance(ref[4], dict):
                param_to_name, gradient_scaling_factor = ref[4], (ref[5] if isinstance(ref[5], (int, float)) else 1.0)
            use_distributed_optimizer, group = False, None
            device = None if not isinstance(device, (str, torch.device)) or isinstance(ref[5], (int, float)) else device
        if ddp_config is not None:
            use_distributed_optimizer = bool(getattr(ddp_config, "use_distributed_optimizer", use_distributed_optimizer))
        group = data_parallel_group if data_parallel_group is not None else group
        self.ddp_config, self.param_to_name = ddp_config, dict(param_to_name or {})
        self.params = [p for p in params if p.requires_grad]
        if not self.params:
            raise ValueError("no trainable parameters")
        self.param_dtype, self.grad_dtype, self.group = param_dtype, grad_dtype, group
        self.world, self.rank = _world(group), _rank(group)
        self.use_distributed_optimizer = use_distributed_optimizer
        self.gradient_scaling_factor = gradient_scaling_factor
        self.device = torch.device(device) if device is not None else self.params[0].device
        pad_to = self.world * ALIGN_ELEMS

        def up(x, m):
            return (x + m - 1) // m * m

        layout, bucket_bounds = [], []
        off, start, bucket_params = 0, 0, 0
        for p in reversed(self.params):
            off = up(off, ALIGN_ELEMS)
            layout.append((p, off, off + p.numel()))
            off += p.numel()
            bucket_params += p.numel()
            if bucket_size is not None and bucket_params >= bucket_size:
                end = up(off, pad_to)
                bucket_bounds.append((start, end, off))
                off = start = end
                bucket_params = 0
        if off > start:
            end = up(off, pad_to)
            bucket_bounds.append((start, end, off))
            off = end
        self.numel = off
        self.numel_unpadded = sum(p.numel() for p in self.params)
        self.grad_data = torch.zeros(self.numel, dtype=grad_dtype, device=self.device)
        self.param_data = torch.zeros(self.numel, dtype=param_dtype, device=self.device)
        self.param_index_map: dict = {}
        with torch.no_grad():
            for p, a, b in layout:
                self.param_data[a:b].copy_(p.data.reshape(-1))
                p.data = self.param_data[a:b].view(p.shape)
                p.main_grad = self.grad_data[a:b].view(p.shape)
                self.param_index_map[p] = (a, b)
        self.buckets: list[ParamAndGradBucket] = []
        for bid, (a, b, used_end) in enumerate(bucket_bounds):
            ps = [p for p, s, e in layout if a <= s < b]
            idx = {p: (self.param_index_map[p][0] - a, self.param_index_map[p][1] - a) for p in ps}
            self.buckets.append(ParamAndGradBucket(ps, self.param_data[a:b], self.grad_data[a:b], a,
                                                   sum(p.numel() for p in ps), gradient_scaling_factor, bid, idx))
        self.param_to_bucket = {p: b for b in self.buckets for p in b.params_list}
        self.bucket_groups: list[ParamAndGradBucketGroup] = []
        self._hooks = []
        self._offloaded: dict | None = None
        if install_hooks:
            self._install_hooks()

    def _install_hooks(self) -> None:
        def make(p):
            def hook(*_):
                if p.grad is not None:
                    p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                    p.grad = None
                for g in self.bucket_groups:
                    if p in g.params:
                        g.register_grad_ready(p)
            return hook
        for p in self.params:
            self._hooks.append(p.register_post_accumulate_grad_hook(make(p)))

    def scale_gradients(self, factor: float) -> None:
        self.grad_data.mul_(factor)

    def reset(self) -> None:
        """Zero the gradient buffer for the next step."""
        self.grad_data.zero_()
        for g in self.bucket_groups:
            g.reset()

    def offload_to_cpu(self, move_params: bool = True, move_grads: bool = True) -> int:
        """Moves the buffers' storage to (pinned) host memory and shrinks the device storage to zero; views held by the
        parameters stay valid objects and come back with `reload_from_cpu`.  Returns the bytes released."""
        freed = 0
        self._offloaded = self._offloaded or {}
        for name, flag in (("param_data", move_params), ("grad_data", move_grads)):
            t = getattr(self, name)
            if not flag or name in self._offloaded or t.untyped_storage().size() == 0:
                continue
            host = torch.empty(t.shape, dtype=t.dtype, pin_memory=t.is_cuda)
            host.copy_(t)
            self._offloaded[name] = host
            freed += t.untyped_storage().nbytes()
            t.untyped_storage().resize_(0)
        return freed

    def reload_from_cpu(self, move_params: bool = True, move_grads: bool = True) -> None:
        if not self._offloaded:
            return
        for name, flag in (("param_data", move_params), ("grad_data", move_grads)):
            host = self._offloaded.get(name)
            if not flag or host is None:
                continue
            t = getattr(self, name)
            t.untyped_storage().resize_(host.numel() * host.element_size())
            t.copy_(host, non_blocking=True)
            del self._offloaded[name]


def partition_buckets(buffers: Sequence[ParamAndGradBuffer], force_single_bucket_group: bool = False,
                      overlap_grad_reduce: bool = True, overlap_param_gather: bool = False,
                      average: bool = True) -> list[ParamAndGradBucketGroup]:
    """One group per bucket (maximum overlap) or a single group over everything (fewest launches).  The groups are
    chained for the parameter all-gather so that finishing one dispatches the next."""
    groups: list[ParamAndGradBucketGroup] = []
    if force_single_bucket_group:
        b0 = buffers[0]
        groups.append(ParamAndGradBucketGroup([b for buf in buffers for b in buf.buckets], b0.group,
                                              b0.use_distributed_optimizer, overlap_grad_reduce, overlap_param_gather,
                                              average))
    else:
        for buf in buffers:
            for b in buf.buckets:
                groups.append(ParamAndGradBucketGroup([b], buf.group, buf.use_distributed_optimizer,
                                                      overlap_grad_reduce, overlap_param_gather, average))
    # forward uses the parameters in the opposite order of the buckets (bucket 0 = last layers)
    for later, earlier in zip(groups[:-1], groups[1:]):
        earlier.next_param_gather_bucket_group = later
    for buf in buffers:
        buf.bucket_groups = [g for g in groups if any(b in buf.buckets for b in g.buckets)]
    return groups


class DistributedOptimizer:
    """ZeRO-1: every rank owns 1/world of each bucket.  Step = finish the reduce-scatter, clip by the global norm
    (one all-reduce of a scalar), AdamW on the owned fp32 master / moment shards with the low-precision write-back
    into the parameter buffer (one fused kernel per bucket on CUDA), then all-gather the parameter buffer."""

    def __init__(self, buffers: Sequence[ParamAndGradBuffer], lr: float = 1e-4, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, max_grad_norm: float | None = 1.0,
                 bucket_groups: Sequence[ParamAndGradBucketGroup] | None = None):
        self.buffers = list(buffers)
        for b in self.buffers:
            if not b.use_distributed_optimizer:
                raise ValueError("buffers must be built with use_distributed_optimizer=True")
        self.groups = list(bucket_groups) if bucket_groups is not None else partition_buckets(self.buffers)
        self.param_groups = [{"lr": lr, "betas": tuple(betas), "eps": eps, "weight_decay": weight_decay}]
        self.max_grad_norm = max_grad_norm
        self.step_count = 0
        self.shards = []            # (bucket, master, exp_avg, exp_avg_sq)
        for buf in self.buffers:
            for b in buf.buckets:
                mine = shard_buffer(b.param_data, buf.world)[buf.rank]
                self.shards.append((buf, b, mine.float().clone(), torch.zeros_like(mine, dtype=torch.float32),
                                    torch.zeros_like(mine, dtype=torch.float32)))

    def zero_grad(self) -> None:
        for buf in self.buffers:
            buf.reset()

    @torch.no_grad()
    def step(self) -> torch.Tensor:
        """Returns the global gradient norm (a tensor on the buffers' device)."""
        for g in self.groups:
            g.finish_grad_sync()
        dev = self.buffers[0].device
        sq = torch.zeros(1, dtype=torch.float32, device=dev)
        for buf, b, *_ in self.shards:
            gs = shard_buffer(b.grad_data, buf.world)[buf.rank]
            K.sumsq_(sq, gs)
        grp = self.buffers[0].group
        if _world(grp) > 1:
            dist.all_reduce(sq, group=grp)
        self.step_count += 1
        pg = self.param_groups[0]
        for buf, b, master, m, v in self.shards:
            gs = shard_buffer(b.grad_data, buf.world)[buf.rank]
            ps = shard_buffer(b.param_data, buf.world)[buf.rank]
            lowp = ps if ps.dtype != torch.float32 else None
            K.adamw_flat_(master, m, v, gs, lowp if lowp is not None and lowp.dtype == torch.bfloat16 else None,
                          lr=pg["lr"], beta1=pg["betas"][0], beta2=pg["betas"][1], eps=pg["eps"],
                          weight_decay=pg["weight_decay"], step=self.step_count, sumsq=sq,
                          max_norm=self.max_grad_norm or 0.0)
            if lowp is None or lowp.dtype != torch.bfloat16:
                ps.copy_(master)
        for g in self.groups:
            g.start_param_sync(force_sync=True)
        return sq.sqrt()

    def state_dict(self) -> dict:
        return {"step": self.step_count, "param_groups": [dict(g) for g in self.param_groups],
                "shards": [{"master": ms.cpu(), "exp_avg": m.cpu(), "exp_avg_sq": v.cpu()}
                           for _, _, ms, m, v in self.shards]}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = sd["step"]
        for (_, _, ms, m, v), s in zip(self.shards, sd["shards"]):
            ms.copy_(s["master"])
            m.copy_(s["exp_avg"])
            v.copy_(s["exp_avg_sq"])
        for g, s in zip(self.param_groups, sd.get("param_groups", [])):
            g.update(s)
