"""Python front-end of csrc/comm.cu (reduce-scatter+cast+norm, AdamW+all-gather, pull all-gather, barrier)."""
from __future__ import annotations

import ctypes

import torch

from ..ops import _lib
from .symm import SymmetricHeap

_ll, _f, _u = ctypes.c_longlong, ctypes.c_float, ctypes.c_uint
SLOT_RS, SLOT_AG, SLOT_BAR = 0, 16, 32


def reduce_scatter_fp32(heap: SymmetricHeap, flat_grad: torch.Tensor, out_shard: torch.Tensor, shard_start: int,
                        scale: float, sumsq: torch.Tensor | None, nonfinite: torch.Tensor | None,
                        max_blocks: int = 0) -> None:
    """out_shard[i] = scale * sum_r grad_r[shard_start + i]; sumsq += sum(out^2). Reads peers inside the kernel."""
    buf, off = heap.lookup(flat_grad)
    lib = _lib.load("comm")
    # what is left of the symmetric allocation behind `flat_grad`, in elements: the launcher refuses a shard that would
    # run past it on this rank or (same layout everywhere) on a peer
    room = (buf.tensor.numel() * buf.tensor.element_size() - off) // flat_grad.element_size()
    rc = lib.ts_symm_reduce_scatter(buf.peer_ptrs, buf.pad_ptrs, ctypes.c_ulonglong(buf.multicast_ptr), _ll(off),
                                    int(flat_grad.dtype == torch.bfloat16), heap.rank, heap.world, _ll(shard_start),
                                    _ll(out_shard.numel()), _lib.ptr(out_shard), _f(scale), _lib.ptr(sumsq),
                                    _lib.ptr(nonfinite), _u(SLOT_RS), _u(buf.next_epoch("rs")), _ll(heap.wait_cycles),
                                    _lib.ptr(heap.status), max_blocks, _ll(room), _lib.stream_ptr())
    _lib.check(rc, "ts_symm_reduce_scatter")


def adamw_bcast(heap: SymmetricHeap, flat_param: torch.Tensor, param_offset: int, master, m, v, grad, *, lr, beta1,
                beta2, eps, weight_decay, step, grad_mul=1.0, sumsq=None, max_norm=0.0, skip_flag=None) -> None:
    """AdamW on the fp32 shard; the bf16 result lands at flat_param[param_offset:...] on EVERY rank."""
    buf, off = heap.lookup(flat_param)
    lib = _lib.load("comm")
    rc = lib.ts_symm_adamw_bcast(_lib.ptr(master), _lib.ptr(m), _lib.ptr(v), _lib.ptr(grad), buf.peer_ptrs,
                                 ctypes.c_ulonglong(buf.multicast_ptr), _ll(off), heap.world, _ll(param_offset),
                                 _ll(master.numel()), _f(lr), _f(beta1), _f(beta2), _f(eps), _f(weight_decay), int(step),
                                 _f(grad_mul), _lib.ptr(sumsq), _f(max_norm), _lib.ptr(skip_flag), 0, _lib.stream_ptr())
    _lib.check(rc, "ts_symm_adamw_bcast")


def all_gather_inplace(heap: SymmetricHeap, flat: torch.Tensor, shard_start: int, shard_numel: int) -> None:
    buf, off = heap.lookup(flat)
    lib = _lib.load("comm")
    rc = lib.ts_symm_all_gather(buf.peer_ptrs, buf.pad_ptrs, _ll(off), heap.rank, heap.world,
                                _ll(shard_numel * flat.element_size()), _u(SLOT_AG), _u(buf.next_epoch("ag")),
                                _ll(heap.wait_cycles), _lib.ptr(heap.status), _lib.stream_ptr())
    _lib.check(rc, "ts_symm_all_gather")


def gather_pull(heap: SymmetricHeap, shard: torch.Tensor, out_full: torch.Tensor, max_blocks: int = 0,
                engine: str = "ce") -> None:
    """out_full = concatenation over ranks of `shard` (a view into symmetric memory, same offset on every rank).
    One-sided: reads the peers' shards and waits for nobody; the caller guarantees that no rank is writing its shard
    (shards change only inside the optimizer step, between the step's barriers).
    engine "ce": peer-to-peer copies on the copy engines (no SM is used); "sm": a small grid of load/store CTAs."""
    buf, off = heap.lookup(shard)
    nbytes = shard.numel() * shard.element_size()
    if out_full.numel() * out_full.element_size() != nbytes * heap.world:
        raise ValueError("gather_pull: output must hold world x shard")
    lib = _lib.load("comm")
    if engine == "ce":
        rc = lib.ts_symm_gather_ce(buf.peer_ptrs, _ll(off), _lib.ptr(out_full), heap.rank, heap.world, _ll(nbytes),
                                   _lib.stream_ptr())
        _lib.check(rc, "ts_symm_gather_ce")
        return
    rc = lib.ts_symm_gather_pull(buf.peer_ptrs, _ll(off), _lib.ptr(out_full), heap.rank, heap.world, _ll(nbytes),
                                 int(max_blocks), _lib.stream_ptr())
    _lib.check(rc, "ts_symm_gather_pull")


def barrier(heap: SymmetricHeap, anchor: torch.Tensor) -> None:
    """Device-side barrier of all ranks on the current stream (all earlier peer stores are visible after it)."""
    buf, _ = heap.lookup(anchor)
    lib = _lib.load("comm")
    rc = lib.ts_symm_barrier(buf.pad_ptrs, heap.rank, heap.world, _u(SLOT_BAR), _u(buf.next_epoch("bar")),
                             _ll(heap.wait_cycles), _lib.ptr(heap.status), _lib.stream_ptr())
    _lib.check(rc, "ts_symm_barrier")


def wait_selftest(limit_cycles: int = 2_000_000) -> tuple[int, tuple]:
    """Run the bounded wait on a flag nothing sets; returns (status, error word)."""
    lib = _lib.load("comm")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.clear_device_error("comm")
    rc = lib.ts_symm_wait_selftest(_lib.ptr(flag), _ll(limit_cycles), _lib.ptr(status), _lib.stream_ptr())
    _lib.check(rc, "ts_symm_wait_selftest")
    torch.cuda.synchronize()
    err = _lib.device_error("comm")
    _lib.clear_device_error("comm")
    return int(status.item()), err
