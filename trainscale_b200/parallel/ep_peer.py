"""Expert-parallel dispatch and combine over NVLink peer memory (kernels: csrc/ep_comm.cu).

`PeerDispatcher` is the peer-memory counterpart of `ep.AllToAllDispatcher` (the `all_to_all_single` pair of
data_pipeline/trainer/distributed/expert_parallel.py:219-391).  What differs:

* nothing synchronises with the host: per-expert counts travel through a symmetric table, every offset is computed on
  the device, buffer sizes are static upper bounds;
* the permutation is part of the transfer: a token row is read once where the router left it and stored straight into
  the owner's receive buffer at the row the owner's grouped GEMM will read it from (segments per local expert, 128-row
  aligned), and on the way back a token's k expert outputs are pulled from their owners and summed with the routing
  weights in one kernel;
* the receive layout is the one `ops.moe.grouped_linear` wants, so the experts run as two grouped tcgen05 GEMM launches
  with no regrouping copy and no per-expert loop.

Step order on every rank (one stream; "barrier" is the flag barrier of csrc/comm.cu on the same stream):

  route     counts -> every peer's table | barrier | plan kernel
  dispatch  push rows -> owners' receive buffers | barrier | private copy with zeroed pad rows
  (experts) grouped GEMM, GLU, grouped GEMM
  combine   outputs -> symmetric buffer | barrier | pull + weighted sum

Backward runs the same two moves the other way round (the combine's backward is a scaled push, the dispatch's backward
an unweighted pull); it needs no new route.  The symmetric buffers are shared by all layers of a model: a buffer is
only overwritten after a barrier that every rank reaches after its last read of it, which holds because every rank
executes the same sequence of layer calls.

The low-level functions take explicit peer-address arrays, so the multi-rank data flow can also be exercised on ONE
GPU with several "ranks" whose buffers all live on that GPU (tests/test_moe_gpu.py).
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

import torch

from ..ops import _lib
from ..ops import moe as moe_ops
from . import fused_comm

_c = ctypes


def _arr(ptrs) -> ctypes.Array:
    return (_c.c_ulonglong * len(ptrs))(*[int(p) for p in ptrs])


def padded_rows(n_total: int, local_experts: int) -> int:
    r = int(_lib.load("ep_comm").ts_ep_padded_rows(_c.c_longlong(n_total), local_experts))
    if r < 0:
        raise ValueError("expert-parallel receive buffer would exceed 2^31 rows")
    return r


@dataclass
class Route:
    """Everything the two moves of one layer call need (device tensors, int32)."""
    ids: torch.Tensor            # [n] global expert of every routed slot
    rank_in_expert: torch.Tensor  # [n] stable position of the slot among this rank's slots for that expert
    send_base: torch.Tensor      # [E]
    dst_row: torch.Tensor        # [n] row in the owner's buffers (written by the first push)
    plan: moe_ops.MoEPlan        # this rank's receive layout, as `ops.moe.grouped_linear` reads it
    seg_real: torch.Tensor       # [El] received rows per local expert
    T: int
    k: int


# ------------------------------------------------------------------------------------------------ low-level launches
def counts_push(cnt_ptrs, counts: torch.Tensor, rank: int, world: int, E: int) -> None:
    rc = _lib.load("ep_comm").ts_ep_counts_push(cnt_ptrs, _lib.ptr(counts), rank, world, E, _lib.stream_ptr())
    _lib.check(rc, "ts_ep_counts_push")


def make_route(table: torch.Tensor, ids32: torch.Tensor, rank_in_expert: torch.Tensor, rank: int, world: int, E: int,
               cap_rows: int, T: int, k: int, overflow: torch.Tensor | None) -> Route:
    """Plan kernel on this rank's complete count table."""
    dev = table.device
    El = E // world
    i32 = dict(dtype=torch.int32, device=dev)
    send_base, seg_start, seg_real = torch.empty(E, **i32), torch.empty(El + 1, **i32), torch.empty(El, **i32)
    tile_expert = torch.empty(cap_rows // 128, **i32)
    rc = _lib.load("ep_comm").ts_ep_plan(_lib.ptr(table), rank, world, E, cap_rows, _lib.ptr(send_base),
                                         _lib.ptr(seg_start), _lib.ptr(seg_real), _lib.ptr(tile_expert),
                                         _lib.ptr(overflow), _lib.stream_ptr())
    _lib.check(rc, "ts_ep_plan")
    plan = moe_ops.MoEPlan(n=0, k=k, E=El, P=cap_rows, counts=seg_real, seg_start=seg_start, tile_expert=tile_expert,
                           dest=None, src_of_row=None)
    return Route(ids32, rank_in_expert, send_base, torch.empty(ids32.numel(), **i32), plan, seg_real, T, k)


def push_rows(xbuf_ptrs, x: torch.Tensor, rt: Route, world: int, scale: torch.Tensor | None = None,
              record_rows: bool = False) -> None:
    H = x.shape[1]
    rc = _lib.load("ep_comm").ts_ep_push_rows(xbuf_ptrs, _lib.ptr(x), _lib.ptr(rt.ids), _lib.ptr(rt.rank_in_expert),
                                              _lib.ptr(rt.send_base), _lib.ptr(scale),
                                              _lib.ptr(rt.dst_row if record_rows else None), rt.ids.numel(), H, rt.k,
                                              rt.plan.E, rt.plan.P, world, _lib.stream_ptr())
    _lib.check(rc, "ts_ep_push_rows")


def finalize(xbuf: torch.Tensor, rt: Route, H: int) -> torch.Tensor:
    priv = torch.empty(rt.plan.P, H, dtype=torch.bfloat16, device=xbuf.device)
    rc = _lib.load("ep_comm").ts_ep_finalize(_lib.ptr(xbuf), _lib.ptr(priv), _lib.ptr(rt.plan.seg_start),
                                             _lib.ptr(rt.seg_real), _lib.ptr(rt.plan.tile_expert), rt.plan.E,
                                             rt.plan.P, H, _lib.stream_ptr())
    _lib.check(rc, "ts_ep_finalize")
    return priv


def copy_used(src: torch.Tensor, dst: torch.Tensor, rt: Route, H: int) -> None:
    rc = _lib.load("ep_comm").ts_ep_copy_used(_lib.ptr(src), _lib.ptr(dst), _lib.ptr(rt.plan.seg_start[rt.plan.E:]),
                                              rt.plan.P, H, _lib.stream_ptr())
    _lib.check(rc, "ts_ep_copy_used")


def pull_combine(ybuf_ptrs, rt: Route, H: int, world: int, w: torch.Tensor | None, keep_rows: bool,
                 device) -> tuple[torch.Tensor, torch.Tensor | None]:
    out = torch.empty(rt.T, H, dtype=torch.bfloat16, device=device)
    ys = torch.empty(rt.T * rt.k, H, dtype=torch.bfloat16, device=device) if keep_rows else None
    rc = _lib.load("ep_comm").ts_ep_pull_combine(ybuf_ptrs, _lib.ptr(rt.ids), _lib.ptr(rt.dst_row), _lib.ptr(w),
                                                 _lib.ptr(out), _lib.ptr(ys), rt.T, H, rt.k, rt.plan.E, rt.plan.P,
                                                 world, _lib.stream_ptr())
    _lib.check(rc, "ts_ep_pull_combine")
    return out, ys


def local_ranks(ids: torch.Tensor, E: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(ids int32 [n], stable rank of every slot inside its expert [n], counts [E]) with the routing-plan kernel."""
    plan = moe_ops.make_plan(ids, E)
    ids32 = ids.reshape(-1).to(torch.int32).contiguous()
    rank_in = (plan.dest - plan.seg_start[:-1][ids32.long()]).contiguous()
    return ids32, rank_in, plan.counts


# ------------------------------------------------------------------------------------------------ dispatcher
class PeerDispatcher:
    """One per expert-parallel group, shared by all mixture-of-experts layers of a model."""

    def __init__(self, heap, num_experts: int, capacity_factor: float | None = None):
        """`capacity_factor`: None (default) sizes the receive buffers for the worst case - every slot of every rank
        routed to one rank - so nothing can overflow; a number f sizes them for f times the mean load (the buffers,
        and every intermediate of the experts, shrink by W / f), and a step that needs more sets the overflow flag
        (`check` raises; the rows that did not fit were dropped).  TS_EP_CAPACITY_FACTOR sets it from the
        environment."""
        import os
        self.heap = heap
        env = os.environ.get("TS_EP_CAPACITY_FACTOR")
        self.capacity_factor = float(env) if env else capacity_factor
        self.world, self.rank = heap.world, heap.rank
        if num_experts % self.world:
            raise ValueError("num_experts must divide by the expert-parallel size")
        self.num_experts, self.local_experts = num_experts, num_experts // self.world
        self.table = heap.alloc(self.world * num_experts, torch.int32)
        self._table_ptrs = heap.lookup(self.table)[0].peer_ptrs
        self.overflow = torch.zeros(1, dtype=torch.int32, device=heap.device)
        self.cap_rows = 0
        self.H = 0
        self.xbuf = self.ybuf = None
        self.calls = 0

    def _ensure(self, n: int, H: int) -> None:
        """(Re)allocate the two symmetric row buffers; collective, so every rank must see the same (n, H)."""
        total = self.world * n
        if self.capacity_factor is not None:
            total = min(total, int(math.ceil(self.capacity_factor * n)))
        cap = padded_rows(total, self.local_experts)
        if cap <= self.cap_rows and H == self.H:
            return
        self.cap_rows, self.H = max(cap, self.cap_rows), H
        self.xbuf = self.heap.alloc(self.cap_rows * H, torch.bfloat16)
        self.ybuf = self.heap.alloc(self.cap_rows * H, torch.bfloat16)
        self._x_ptrs = self.heap.lookup(self.xbuf)[0].peer_ptrs
        self._y_ptrs = self.heap.lookup(self.ybuf)[0].peer_ptrs

    def barrier(self) -> None:
        fused_comm.barrier(self.heap, self.table)

    def route(self, ids: torch.Tensor, H: int) -> Route:
        T, k = ids.shape
        self._ensure(T * k, H)
        ids32, rank_in, counts = local_ranks(ids, self.num_experts)
        counts_push(self._table_ptrs, counts, self.rank, self.world, self.num_experts)
        self.barrier()
        self.calls += 1
        return make_route(self.table, ids32, rank_in, self.rank, self.world, self.num_experts, self.cap_rows, T, k,
                          self.overflow)

    # the two moves; `first` marks the forward dispatch, which records the destination rows
    def send(self, x: torch.Tensor, rt: Route, scale: torch.Tensor | None = None, first: bool = False) -> torch.Tensor:
        push_rows(self._x_ptrs, x, rt, self.world, scale, record_rows=first)
        self.barrier()
        return finalize(self.xbuf, rt, x.shape[1])

    def fetch(self, y: torch.Tensor, rt: Route, w: torch.Tensor | None, keep_rows: bool):
        copy_used(y, self.ybuf, rt, y.shape[1])
        self.barrier()
        return pull_combine(self._y_ptrs, rt, y.shape[1], self.world, w, keep_rows, y.device)

    def check(self) -> None:
        """Host read (call where the loss is read): raises if a receive buffer was too small."""
        if int(self.overflow.item()) != 0:
            self.overflow.zero_()
            from ..core.errors import CommunicationError
            raise CommunicationError("an expert-parallel receive buffer overflowed (ranks routed different numbers of "
                                     "slots?)", rank=self.rank, world=self.world)


class _DispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, d: PeerDispatcher, rt: Route):
        ctx.d, ctx.rt = d, rt
        return d.send(x2.contiguous(), rt, first=True)

    @staticmethod
    def backward(ctx, dxr):
        dx2, _ = ctx.d.fetch(dxr.contiguous(), ctx.rt, None, False)
        return dx2, None, None


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, w, d: PeerDispatcher, rt: Route):
        wf = w.reshape(-1).float().contiguous()
        out, ys = d.fetch(y.contiguous(), rt, wf, keep_rows=True)
        ctx.save_for_backward(ys, wf)
        ctx.d, ctx.rt, ctx.w_dtype, ctx.w_shape = d, rt, w.dtype, w.shape
        return out

    @staticmethod
    def backward(ctx, dout):
        ys, wf = ctx.saved_tensors
        rt = ctx.rt
        dout = dout.contiguous()
        n, H = ys.shape
        lib = _lib.load("moe")
        dw = torch.empty(n, dtype=torch.float32, device=ys.device)
        ident = torch.arange(n, dtype=torch.int32, device=ys.device)
        rc = lib.ts_moe_combine_dw(_lib.ptr(dout), _lib.ptr(ys), _lib.ptr(ident), _lib.ptr(dw), n, H, rt.k,
                                   _lib.stream_ptr())
        _lib.check(rc, "ts_moe_combine_dw")
        dy = ctx.d.send(dout, rt, scale=wf)           # dy[row(t, j)] = w[t, j] * dout[t] on the owner; pad rows zero
        return dy, dw.view(ctx.w_shape).to(ctx.w_dtype), None, None


def expert_parallel_ffn(x2: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_gate_up: torch.Tensor,
                        w_down: torch.Tensor, d: PeerDispatcher, act: str = "silu") -> torch.Tensor:
    """out[t] = sum_j weights[t, j] * FFN_{ids[t, j]}(x2[t]) with the experts sharded over the dispatcher's group:
    w_gate_up [El, 2I, H], w_down [El, H, I] are this rank's experts.  Collective; differentiable."""
    from ..ops import activation
    rt = d.route(ids, x2.shape[1])
    xr = _DispatchFn.apply(x2, d, rt)
    h = moe_ops.grouped_linear(xr, w_gate_up, rt.plan)
    h = activation.glu(h, act)
    y = moe_ops.grouped_linear(h, w_down, rt.plan)
    return _CombineFn.apply(y, weights, d, rt)
