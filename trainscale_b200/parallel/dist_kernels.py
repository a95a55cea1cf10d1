"""Collective-communication helpers of the kernel layer: side streams, tensor bucketing, gradient compression
(bf16 / fp16 cast, PowerSGD, top-k with error feedback), a `DistributedKernels` facade over the collectives used by
data / tensor / sequence / pipeline parallelism, pinned-memory transfers, two-level all-reduce and a bucketed
gradient-sync hook.  Public names follow data_pipeline/trainer/kernels/distributed_kernels.py:42-1546.

On B200 the bandwidth-critical collectives of training do not go through this facade: they are fused into kernels
(`csrc/comm.cu`, `csrc/tp_gemm.cu`).  The facade is the plumbing API (NCCL on GPUs, gloo on CPU); every method degrades
to the identity when no process group is initialised.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass
from enum import Enum
from typing import Any, Sequence

import torch
import torch.distributed as dist

from ..utils.refargs import ANY, reference_kwargs

ReduceOp = dist.ReduceOp


class DistributedBackend(Enum):
    NCCL = "nccl"
    GLOO = "gloo"
    NONE = "none"

    def to_torch_backend(self) -> str | None:
        """Name for `torch.distributed.init_process_group` (None for NONE: no process group)."""
        return None if self is DistributedBackend.NONE else self.value


@dataclass
class DistributedConfig:
    bucket_size_mb: float = 25.0
    overlap_comm: bool = True
    num_comm_streams: int = 2
    compression: str = "none"            # none | bf16 | fp16 | powersgd | topk
    powersgd_rank: int = 4
    topk_ratio: float = 0.01
    average: bool = True
    tp_size: int = 1
    pp_size: int = 1
    dp_size: int = 1

    def validate_topology(self, world_size: int | None = None) -> None:
        """tp x pp x dp must equal the world size (the job's, when not given); ValueError otherwise."""
        w = world_size if world_size is not None else (dist.get_world_size() if _on() else 1)
        if min(self.tp_size, self.pp_size, self.dp_size) < 1:
            raise ValueError("parallel sizes must be >= 1")
        if self.tp_size * self.pp_size * self.dp_size != w:
            raise ValueError(f"tp ({self.tp_size}) x pp ({self.pp_size}) x dp ({self.dp_size}) != world size ({w})")


def _on() -> bool:
    return dist.is_available() and dist.is_initialized()


def get_distributed_backend() -> DistributedBackend:
    if not _on():
        return DistributedBackend.NONE
    return DistributedBackend.NCCL if dist.get_backend() == "nccl" else DistributedBackend.GLOO


def get_world_info() -> tuple[int, int, int, int]:
    """(rank, world_size, local_rank, local_world_size) from the process group or the launcher's environment."""
    import os
    rank = dist.get_rank() if _on() else int(os.environ.get("RANK", "0"))
    world = dist.get_world_size() if _on() else int(os.environ.get("WORLD_SIZE", "1"))
    return rank, world, int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("LOCAL_WORLD_SIZE", str(world)))


class CommStreamManager:
    """Round-robin pool of side streams for collectives that should overlap compute."""

    def __init__(self, num_streams: int = 2, device: torch.device | str | None = None):
        self.device = torch.device(device) if device is not None else \
            (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self._streams = [torch.cuda.Stream(self.device) for _ in range(num_streams)] \
            if self.device.type == "cuda" else []
        self._next = 0

    def get_stream(self):
        if not self._streams:
            return None
        s = self._streams[self._next % len(self._streams)]
        self._next += 1
        return s

    @contextlib.contextmanager
    def comm_stream(self):
        """Run the block on a side stream that first waits for the work already queued on the current stream."""
        s = self.get_stream()
        if s is None:
            yield None
            return
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            yield s

    def synchronize_all(self) -> None:
        for s in self._streams:
            torch.cuda.current_stream(self.device).wait_stream(s)

    # ---- event form of the same two edges, for code that picks its own stream
    def record_compute_event(self):
        """Mark "compute has produced its data" on the current stream; a side stream then waits for the returned event
        (`stream.wait_event(ev)`) instead of for the whole stream.  None without a GPU."""
        if not self._streams:
            return None
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        return ev

    def sync_back_to_compute(self, stream=None) -> None:
        """The current (compute) stream waits for what was queued on `stream` (default: every side stream)."""
        if not self._streams:
            return
        cur = torch.cuda.current_stream(self.device)
        for s in ([stream] if stream is not None else self._streams):
            cur.wait_stream(s)


_MANAGER: CommStreamManager | None = None


def get_comm_stream_manager(num_streams: int = 2) -> CommStreamManager:
    global _MANAGER
    if _MANAGER is None:
        _MANAGER = CommStreamManager(num_streams)
    return _MANAGER


class TensorBucket:
    """Tensors of one dtype that travel as one flat buffer."""

    def __init__(self, capacity_bytes: int, dtype: torch.dtype | None = None):
        self.capacity, self.dtype = capacity_bytes, dtype
        self.tensors: list[torch.Tensor] = []
        self.bytes = 0
        self._flat: torch.Tensor | None = None

    def add(self, tensor: torch.Tensor) -> bool:
        nb = tensor.numel() * tensor.element_size()
        if self.tensors and (self.bytes + nb > self.capacity or tensor.dtype != self.dtype):
            return False
        self.dtype = self.dtype or tensor.dtype
        self.tensors.append(tensor)
        self.bytes += nb
        return True

    def flatten(self) -> torch.Tensor:
        self._flat = torch.cat([t.reshape(-1) for t in self.tensors]) if len(self.tensors) > 1 \
            else self.tensors[0].reshape(-1).clone()
        return self._flat

    def unflatten(self) -> None:
        """Copy the (reduced) flat buffer back into the member tensors."""
        off = 0
        with torch.no_grad():
            for t in self.tensors:
                t.copy_(self._flat[off:off + t.numel()].view_as(t))
                off += t.numel()

    def clear(self) -> None:
        self.tensors, self.bytes, self._flat = [], 0, None


class BucketManager:
    def __init__(self, bucket_size_mb: float = 25.0):
        self.bucket_bytes = int(bucket_size_mb * 2 ** 20)

    def create_buckets(self, tensors: Sequence[torch.Tensor]) -> list[TensorBucket]:
        """Greedy fill in the given order, one dtype per bucket."""
        out: list[TensorBucket] = []
        open_by_dtype: dict[torch.dtype, TensorBucket] = {}
        for t in tensors:
            b = open_by_dtype.get(t.dtype)
            if b is None or not b.add(t):
                b = TensorBucket(self.bucket_bytes, t.dtype)
                b.add(t)
                out.append(b)
                open_by_dtype[t.dtype] = b
        return out


class GradientCompressor:
    """Lossy gradient encodings with error feedback (the part that was dropped is added to the next step's gradient).

    compress(t, key) -> (payload tensors, ctx) ;  decompress(payload, ctx) -> tensor of the original shape.
    PowerSGD payloads (P, Q) are each all-reducible; top-k payloads (values, indices) are all-gathered."""

    def __init__(self, use_fp16: bool = False, use_powersgd: bool = False, powersgd_rank: int = 4,
                 topk_ratio: float = 0.0, use_bf16: bool = False):
        self.use_fp16, self.use_bf16 = use_fp16, use_bf16
        self.use_powersgd, self.powersgd_rank, self.topk_ratio = use_powersgd, powersgd_rank, topk_ratio
        self._error_buffers: dict[Any, torch.Tensor] = {}
        self._q_buffers: dict[Any, torch.Tensor] = {}

    def _feedback(self, t: torch.Tensor, key) -> torch.Tensor:
        e = self._error_buffers.get(key)
        return t if e is None else t + e

    @reference_kwargs(tensor_id="key")
    def compress(self, tensor: torch.Tensor, key: Any = None) -> tuple[list[torch.Tensor], dict]:
        key = id(tensor) if key is None else key
        ctx = {"shape": tensor.shape, "dtype": tensor.dtype, "key": key}
        if self.use_powersgd and tensor.dim() >= 2 and min(tensor.shape[0], tensor[0].numel()) > self.powersgd_rank:
            m = self._feedback(tensor, key).reshape(tensor.shape[0], -1).float()
            q = self._q_buffers.get(key)
            if q is None:
                g = torch.Generator(device="cpu").manual_seed(hash(key) % (2 ** 31))
                q = torch.randn(m.shape[1], self.powersgd_rank, generator=g).to(m.device)
            p = m @ q
            p, _ = torch.linalg.qr(p)
            q = m.t() @ p
            self._q_buffers[key] = q
            self._error_buffers[key] = (m - p @ q.t()).view(tensor.shape).to(tensor.dtype)
            ctx["mode"] = "powersgd"
            return [p, q], ctx
        if self.topk_ratio > 0:
            flat = self._feedback(tensor, key).reshape(-1)
            k = max(1, int(flat.numel() * self.topk_ratio))
            _, idx = flat.abs().topk(k)
            vals = flat[idx]
            rest = flat.clone()
            rest[idx] = 0
            self._error_buffers[key] = rest.view(tensor.shape)
            ctx["mode"] = "topk"
            return [vals, idx], ctx
        if self.use_fp16 or self.use_bf16:
            ctx["mode"] = "cast"
            return [tensor.to(torch.float16 if self.use_fp16 else torch.bfloat16)], ctx
        ctx["mode"] = "none"
        return [tensor], ctx

    @reference_kwargs(tensor="payload", metadata="ctx")
    def decompress(self, payload: "Sequence[torch.Tensor] | torch.Tensor", ctx: dict) -> torch.Tensor:
        if torch.is_tensor(payload):
            payload = [payload]
        mode = ctx["mode"]
        if mode == "powersgd":
            p, q = payload
            return (p @ q.t()).view(ctx["shape"]).to(ctx["dtype"])
        if mode == "topk":
            vals, idx = payload
            n = 1
            for s in ctx["shape"]:
                n *= s
            out = torch.zeros(n, dtype=vals.dtype, device=vals.device)
            out.index_add_(0, idx, vals)
            return out.view(ctx["shape"]).to(ctx["dtype"])
        return payload[0].to(ctx["dtype"]).view(ctx["shape"])


class _Deferred:
    """A pending collective plus the host-side step that completes it (copy back, scaling) once it has finished."""

    def __init__(self, work, then):
        self.work, self.then = work, then

    def wait(self):
        self.work.wait()
        self.then()


class DistributedKernels:
    """One object for every collective the parallel layers use.  `async_op=True` returns at once and `wait_pending`
    settles everything issued so far."""

    def __init__(self, config: DistributedConfig | None = None):
        self.config = config or DistributedConfig()
        self._pending: list = []
        self._buckets = BucketManager(self.config.bucket_size_mb)

    @staticmethod
    def _n(group) -> int:
        return dist.get_world_size(group) if _on() else 1

    def _track(self, work, async_op: bool):
        if async_op and work is not None:
            self._pending.append(work)
        return work

    # ---------------------------------------------------------------- reductions
    def all_reduce(self, tensor: torch.Tensor, op=ReduceOp.SUM, group=None, async_op: bool = False,
                   average: bool = False) -> torch.Tensor:
        if self._n(group) > 1:
            w = dist.all_reduce(tensor, op=op, group=group, async_op=async_op)
            self._track(w, async_op)
            if average and not async_op:
                tensor.div_(self._n(group))
        return tensor

    def all_reduce_fused(self, tensors: Sequence[torch.Tensor], op=ReduceOp.SUM, group=None,
                         average: bool = False, async_op: bool = False) -> None:
        """Bucket by dtype / size, one all-reduce per flat bucket, results copied back in place.  With `async_op` the
        reductions are only issued; the copy back (and the averaging) happens in `wait_pending()`."""
        if self._n(group) == 1 or not tensors:
            return
        for b in self._buckets.create_buckets(list(tensors)):
            flat = b.flatten()
            w = dist.all_reduce(flat, op=op, group=group, async_op=async_op)
            if async_op:
                self._pending.append(_Deferred(w, (lambda f=flat, bb=b: (f.div_(self._n(group)) if average else f,
                                                                        bb.unflatten()))))
                continue
            if average:
                flat.div_(self._n(group))
            b.unflatten()

    def all_reduce_coalesced(self, tensors: Sequence[torch.Tensor], op=ReduceOp.SUM, group=None) -> None:
        self.all_reduce_fused(tensors, op, group)

    # ---------------------------------------------------------------- gathers / scatters
    def all_gather(self, tensor: torch.Tensor, group=None, dim: int = 0, async_op: bool = False) -> torch.Tensor:
        """Concatenation of every rank's tensor along `dim`.  `async_op` (dimension 0 only; other dimensions need the
        data for the concatenation and run synchronously): the result is complete after `wait_pending()`."""
        n = self._n(group)
        if n == 1:
            return tensor
        if async_op and dim == 0:
            return self.all_gather_into_tensor(None, tensor, group, async_op=True)
        parts = [torch.empty_like(tensor) for _ in range(n)]
        dist.all_gather(parts, tensor.contiguous(), group=group)
        return torch.cat(parts, dim=dim)

    @reference_kwargs(input_tensor="tensor")
    def all_gather_into_tensor(self, output: torch.Tensor | None, tensor: torch.Tensor, group=None,
                               async_op: bool = False) -> torch.Tensor:
        n = self._n(group)
        if n == 1:
            if output is None:
                return tensor
            output.copy_(tensor.view_as(output))
            return output
        if output is None:
            output = torch.empty((n * tensor.shape[0],) + tuple(tensor.shape[1:]), dtype=tensor.dtype,
                                 device=tensor.device)
        self._track(dist.all_gather_into_tensor(output, tensor.contiguous(), group=group, async_op=async_op), async_op)
        return output

    def reduce_scatter(self, tensor: torch.Tensor | None = None, op=ReduceOp.SUM, group=None, dim: int = 0, *,
                       output: torch.Tensor | None = None, input_tensors: Sequence[torch.Tensor] | None = None,
                       async_op: bool = False) -> torch.Tensor:
        """Sum over the group, keep this rank's slice along `dim`.  `reduce_scatter(output, input_tensors, op, group,
        async_op)` is the list form: rank r receives the reduction of every rank's `input_tensors[r]` in `output`."""
        if input_tensors is not None or isinstance(op, (list, tuple)):
            if isinstance(op, (list, tuple)):                            # positional (output, input_tensors, op, group)
                output, input_tensors, op, group = tensor, op, (group if group is not None else ReduceOp.SUM), \
                    (dim if not isinstance(dim, int) else None)
            output = output if output is not None else tensor
            if self._n(group) == 1:
                output.copy_(input_tensors[0])
                return output
            self._track(dist.reduce_scatter(output, [t.contiguous() for t in input_tensors], op=op, group=group,
                                            async_op=async_op), async_op)
            return output
        n = self._n(group)
        if n == 1:
            return tensor
        parts = [p.contiguous() for p in tensor.chunk(n, dim=dim)]
        out = torch.empty_like(parts[0])
        dist.reduce_scatter(out, parts, op=op, group=group)
        return out

    @reference_kwargs(input_tensor="tensor")
    def reduce_scatter_tensor(self, output: torch.Tensor | None, tensor: torch.Tensor, op=ReduceOp.SUM, group=None,
                              async_op: bool = False) -> torch.Tensor:
        n = self._n(group)
        if n == 1:
            if output is None:
                return tensor
            output.copy_(tensor.view_as(output))
            return output
        if output is None:
            output = torch.empty((tensor.shape[0] // n,) + tuple(tensor.shape[1:]), dtype=tensor.dtype,
                                 device=tensor.device)
        self._track(dist.reduce_scatter_tensor(output, tensor.contiguous(), op=op, group=group, async_op=async_op),
                    async_op)
        return output

    # ---------------------------------------------------------------- sequence / tensor parallel helpers
    @staticmethod
    def _dim_group(group, seq_dim):
        """`(x, dim, group)` is the reference's order, `(tensor, group, seq_dim)` ours: an int in the group's place is
        the dimension."""
        if isinstance(group, int) and not isinstance(group, bool):
            return (seq_dim if not isinstance(seq_dim, int) else None), group
        return group, seq_dim

    @reference_kwargs(x="tensor", dim="seq_dim")
    def sequence_parallel_all_gather(self, tensor: torch.Tensor, group=None, seq_dim: int = 1,
                                     async_op: bool = False) -> torch.Tensor:
        """[.., S/n, ..] -> [.., S, ..]: rank r holds the r-th slice of the sequence."""
        group, seq_dim = self._dim_group(group, seq_dim)
        if self._n(group) == 1:
            return tensor
        if seq_dim == 0:
            return self.all_gather_into_tensor(None, tensor, group, async_op=async_op)
        return self.all_gather(tensor, group, dim=seq_dim)

    @reference_kwargs(x="tensor", dim="seq_dim")
    def sequence_parallel_reduce_scatter(self, tensor: torch.Tensor, group=None, seq_dim: int = 1,
                                         async_op: bool = False) -> torch.Tensor:
        group, seq_dim = self._dim_group(group, seq_dim)
        if self._n(group) == 1:
            return tensor
        if seq_dim == 0:
            return self.reduce_scatter_tensor(None, tensor, group=group, async_op=async_op)
        return self.reduce_scatter(tensor, group=group, dim=seq_dim)

    def tensor_parallel_all_reduce(self, tensor: torch.Tensor, group=None, async_op: bool = False) -> torch.Tensor:
        return self.all_reduce(tensor, group=group, async_op=async_op)

    def tensor_parallel_all_gather(self, tensor: torch.Tensor, group=None, dim: int = -1) -> torch.Tensor:
        return self.all_gather(tensor, group, dim=dim)

    def tensor_parallel_reduce_scatter(self, tensor: torch.Tensor, group=None, dim: int = -1) -> torch.Tensor:
        return self.reduce_scatter(tensor, group=group, dim=dim)

    # ---------------------------------------------------------------- pipeline point-to-point
    @reference_kwargs(dst_rank="dst")
    def pipeline_send(self, tensor: torch.Tensor, dst: int, group=None, async_op: bool = True, tag: int = 0):
        w = dist.isend(tensor.contiguous(), dst, group=group, tag=tag)
        if async_op:
            self._pending.append(w)
        else:
            w.wait()
        return w

    @reference_kwargs(src_rank="src")
    def pipeline_recv(self, tensor: torch.Tensor, src: int, group=None, async_op: bool = False, tag: int = 0):
        w = dist.irecv(tensor, src, group=group, tag=tag)
        if async_op:
            self._pending.append(w)
        else:
            w.wait()
        return tensor

    def pipeline_send_recv(self, send_tensor: torch.Tensor | None, recv_tensor: torch.Tensor | None,
                           send_dst: int | None, recv_src: int | None, group=None, send_tag: int = 0,
                           recv_tag: int = 0) -> torch.Tensor | None:
        """Both directions in one batched call, so two neighbours exchanging at the same time cannot deadlock."""
        ops = []
        if send_tensor is not None and send_dst is not None:
            ops.append(dist.P2POp(dist.isend, send_tensor.contiguous(), send_dst, group, tag=send_tag))
        if recv_tensor is not None and recv_src is not None:
            ops.append(dist.P2POp(dist.irecv, recv_tensor, recv_src, group, tag=recv_tag))
        for w in (dist.batch_isend_irecv(ops) if ops else []):
            w.wait()
        return recv_tensor

    send_recv = pipeline_send_recv

    # ---------------------------------------------------------------- misc
    def broadcast(self, tensor: torch.Tensor, src: int = 0, group=None, async_op: bool = False) -> torch.Tensor:
        if self._n(group) > 1:
            self._track(dist.broadcast(tensor, src, group=group, async_op=async_op), async_op)
        return tensor

    @reference_kwargs(object_list="objects")
    def broadcast_object_list(self, objects: list, src: int = 0, group=None) -> list:
        if self._n(group) > 1:
            dist.broadcast_object_list(objects, src, group=group)
        return objects

    def wait_pending(self) -> None:
        for w in self._pending:
            w.wait()
        self._pending.clear()

    def barrier(self, group=None) -> None:
        if self._n(group) > 1:
            dist.barrier(group=group)


class ZeroCopyTransfer:
    """Host <-> device copies through a reusable pinned staging buffer, on their own stream."""

    def __init__(self, device: "torch.device | str | int | None" = None, staging_bytes: int = 64 * 2 ** 20, *,
                 pool_size_mb: int | None = None):
        """`pool_size_mb` (the reference's only argument, also taken positionally as an int): size of the pinned staging
        buffer."""
        if isinstance(device, int) and not isinstance(device, bool):
            pool_size_mb, device = device, None
        if pool_size_mb is not None:
            staging_bytes = int(pool_size_mb) * 2 ** 20
        self.device = torch.device(device) if device is not None else \
            (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self._cuda = self.device.type == "cuda"
        self._stream = torch.cuda.Stream(self.device) if self._cuda else None
        self._staging: dict[torch.dtype, torch.Tensor] = {}
        self.staging_bytes = staging_bytes

    def _pinned(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        buf = self._staging.get(dtype)
        if buf is None or buf.numel() < numel:
            buf = torch.empty(max(numel, self.staging_bytes // torch.empty((), dtype=dtype).element_size()),
                              dtype=dtype, pin_memory=self._cuda)
            self._staging[dtype] = buf
        return buf[:numel]

    @reference_kwargs(x="tensor")
    def host_to_device(self, tensor: torch.Tensor, non_blocking: bool = True, *, device=None,
                       use_pool: bool = True) -> torch.Tensor:
        """`device`: target (this object's device when None); `use_pool=False` pins a fresh buffer instead of the shared
        staging buffer (safe when several transfers are in flight)."""
        if device is not None and torch.device(device) != self.device:
            return ZeroCopyTransfer(device, self.staging_bytes).host_to_device(tensor, non_blocking, use_pool=use_pool)
        if not self._cuda:
            return tensor
        if tensor.is_pinned():
            src = tensor
        elif use_pool:
            src = self._pinned(tensor.numel(), tensor.dtype).copy_(tensor.reshape(-1))
        else:
            src = torch.empty(tensor.numel(), dtype=tensor.dtype, pin_memory=True).copy_(tensor.reshape(-1))
        with torch.cuda.stream(self._stream):
            out = src.to(self.device, non_blocking=non_blocking).view(tensor.shape)
        torch.cuda.current_stream(self.device).wait_stream(self._stream)
        return out

    @reference_kwargs(x="tensor")
    def device_to_host(self, tensor: torch.Tensor, non_blocking: bool = False, *, use_pool: bool = False) -> torch.Tensor:
        """`use_pool=True` lands in the shared staging buffer: the result is only valid until the next transfer."""
        if not tensor.is_cuda:
            return tensor
        host = self._pinned(tensor.numel(), tensor.dtype).view(tensor.shape) if use_pool else \
            torch.empty(tensor.shape, dtype=tensor.dtype, pin_memory=True)
        self._stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self._stream):
            host.copy_(tensor, non_blocking=True)
        if not non_blocking:
            self._stream.synchronize()
        return host


@reference_kwargs(x="tensor")
def pinned_memory_transfer(tensor: torch.Tensor, device: torch.device | str, non_blocking: bool = True) -> torch.Tensor:
    dev = torch.device(device)
    if dev.type != "cuda" or tensor.is_cuda:
        return tensor.to(dev)
    src = tensor if tensor.is_pinned() else tensor.pin_memory()
    return src.to(dev, non_blocking=non_blocking)


class HierarchicalCommunicator:
    """Two-level all-reduce: reduce-scatter inside the local (NVLink) group, all-reduce of the shard across the
    global (inter-node) group, all-gather inside the local group.  The slow network carries 1/local_size of the data."""

    def __init__(self, local_group=None, global_group=None):
        self.local_group, self.global_group = local_group, global_group
        self._kernels = DistributedKernels()

    def hierarchical_all_reduce(self, tensor: torch.Tensor, op=ReduceOp.SUM) -> torch.Tensor:
        nl = dist.get_world_size(self.local_group) if _on() and self.local_group is not None else 1
        ng = dist.get_world_size(self.global_group) if _on() and self.global_group is not None else 1
        if nl == 1:
            if ng > 1:
                dist.all_reduce(tensor, op=op, group=self.global_group)
            return tensor
        flat = tensor.reshape(-1)
        pad = (-flat.numel()) % nl
        work = torch.cat((flat, flat.new_zeros(pad))) if pad else flat.contiguous()
        shard = torch.empty(work.numel() // nl, dtype=work.dtype, device=work.device)
        dist.reduce_scatter_tensor(shard, work, op=op, group=self.local_group)
        if ng > 1:
            dist.all_reduce(shard, op=op, group=self.global_group)
        dist.all_gather_into_tensor(work, shard, group=self.local_group)
        with torch.no_grad():
            tensor.copy_(work[:flat.numel()].view_as(tensor))
        return tensor


class GradientSyncHook:
    """Data-parallel gradient averaging for a plain model: parameters are bucketed in reverse order, a bucket's
    all-reduce starts as soon as all of its gradients exist (inside backward), `synchronize()` waits and copies back."""

    def __init__(self, parameters, config: DistributedConfig | None = None, group=None):
        self.parameters = [p for p in parameters if p.requires_grad]
        self.config = config or DistributedConfig()
        self.group = group
        self._kernels = DistributedKernels(self.config)
        cap = int(self.config.bucket_size_mb * 2 ** 20)
        self._bucket_of: dict = {}
        self._buckets: list[list] = [[]]
        size = 0
        for p in reversed(self.parameters):
            nb = p.numel() * p.element_size()
            if self._buckets[-1] and size + nb > cap:
                self._buckets.append([])
                size = 0
            self._buckets[-1].append(p)
            self._bucket_of[p] = len(self._buckets) - 1
            size += nb
        self._ready = [0] * len(self._buckets)
        self._inflight: list = []
        self._handles = [p.register_post_accumulate_grad_hook(self._make_hook(p)) for p in self.parameters]
        self.enabled = True

    def _make_hook(self, p):
        def hook(*_):
            if not self.enabled:
                return
            b = self._bucket_of[p]
            self._ready[b] += 1
            if self._ready[b] == len(self._buckets[b]):
                self._launch(b)
        return hook

    def _launch(self, b: int) -> None:
        ps = [p for p in self._buckets[b] if p.grad is not None]
        n = dist.get_world_size(self.group) if _on() else 1
        if not ps or n == 1:
            return
        flat = torch.cat([p.grad.reshape(-1) for p in ps])
        if self.config.compression in ("bf16", "fp16"):
            flat = flat.to(torch.bfloat16 if self.config.compression == "bf16" else torch.float16)
        w = dist.all_reduce(flat, group=self.group, async_op=self.config.overlap_comm)
        self._inflight.append((w if self.config.overlap_comm else None, flat, ps, n))

    def synchronize(self) -> None:
        for w, flat, ps, n in self._inflight:
            if w is not None:
                w.wait()
            off = 0
            with torch.no_grad():
                for p in ps:
                    g = flat[off:off + p.numel()].view_as(p.grad).to(p.grad.dtype)
                    p.grad.copy_(g / n if self.config.average else g)
                    off += p.numel()
        self._inflight.clear()
        self._ready = [0] * len(self._buckets)

    @contextlib.contextmanager
    def no_sync(self):
        self.enabled = False
        try:
            yield
        finally:
            self.enabled = True

    def remove_hooks(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles = []


def create_process_groups(tensor_parallel_size: int = 1, pipeline_parallel_size: int = 1,
                          sequence_parallel_size: int = 1) -> dict[str, Any]:
    """Groups for a [data, pipeline, tensor] layout (tensor fastest).  Sequence parallelism shares the tensor group.
    Returns {"tensor", "pipeline", "data", "sequence"} (None where the degree is 1); {} without a process group."""
    if not _on():
        return {}
    world, rank = dist.get_world_size(), dist.get_rank()
    tp, pp = tensor_parallel_size, pipeline_parallel_size
    if world % (tp * pp):
        raise ValueError(f"world size {world} does not divide by tp*pp = {tp * pp}")
    dp = world // (tp * pp)
    out: dict[str, Any] = {"tensor": None, "pipeline": None, "data": None}

    def make(name, rank_lists):
        for ranks in rank_lists:
            g = dist.new_group(ranks) if len(ranks) > 1 else None
            if rank in ranks:
                out[name] = g

    make("tensor", [[(d * pp + p) * tp + t for t in range(tp)] for d in range(dp) for p in range(pp)])
    make("pipeline", [[(d * pp + p) * tp + t for p in range(pp)] for d in range(dp) for t in range(tp)])
    make("data", [[(d * pp + p) * tp + t for d in range(dp)] for p in range(pp) for t in range(tp)])
    out["sequence"] = out["tensor"] if sequence_parallel_size > 1 else None
    return out


def get_model_parallel_world_size(group=None) -> int:
    return dist.get_world_size(group) if _on() and group is not None else 1


def get_model_parallel_rank(group=None) -> int:
    return dist.get_rank(group) if _on() and group is not None else 0


_KERNELS: DistributedKernels | None = None


def get_distributed_kernels(config: DistributedConfig | None = None) -> DistributedKernels:
    global _KERNELS
    if _KERNELS is None or config is not None:
        _KERNELS = DistributedKernels(config)
    return _KERNELS
