"""Symmetric (peer-mapped) device memory for the fused compute+collective kernels.

Every rank allocates the same sizes in the same order; each allocation is rendezvoused once and yields the peer
addresses of the buffer on all ranks, the addresses of its signal pad and, when the fabric supports it, an
NVSwitch multicast address.  Allocation and handle exchange go through `torch.distributed._symmetric_memory`
(CUDA VMM + fabric/posix handles over the process group's store); the kernels in csrc/comm.cu only ever see raw
addresses.  The reference has no counterpart (it issues every collective through torch.distributed -> NCCL,
data_pipeline/trainer/kernels/distributed_kernels.py:480-1072).
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class SymmBuffer:
    tensor: torch.Tensor
    handle: object
    peer_ptrs: ctypes.Array        # c_ulonglong[world]
    pad_ptrs: ctypes.Array
    multicast_ptr: int
    epochs: dict

    def next_epoch(self, key: str) -> int:
        e = self.epochs.get(key, 0) + 1
        self.epochs[key] = e
        return e


class SymmetricHeap:
    """Allocator + registry of symmetric buffers of one process group."""

    def __init__(self, group, device):
        self.group = group if group is not None else dist.group.WORLD
        self.device = torch.device(device)
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self._by_ptr: dict[int, SymmBuffer] = {}
        self.use_multicast = os.environ.get("TS_SYMM_MULTICAST", "1") != "0"
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        # A peer wait gives up after `wait_cycles` clock ticks and sets `status`.  Until `mark_warm()` the limit is
        # generous (lazy library loading and first-use allocations put ranks tens of seconds apart on the first step);
        # afterwards a rank that is this late is treated as lost.  TS_SYMM_WAIT_SECONDS overrides both (tests shorten it).
        env = os.environ.get("TS_SYMM_WAIT_SECONDS")
        self._cold_cycles = int(float(env if env else "60") * 1.9e9)
        self._warm_cycles = int(float(env if env else "10") * 1.9e9)
        self.wait_cycles = self._cold_cycles

    def mark_warm(self) -> None:
        """Call once every rank has completed a full step: later peer waits use the short limit."""
        self.wait_cycles = self._warm_cycles

    @classmethod
    def try_create(cls, group, device):
        if os.environ.get("TS_DISABLE_SYMM", "0") == "1":
            return None
        try:
            import torch.distributed._symmetric_memory as symm_mem  # noqa: F401
            heap = cls(group, device)
            probe = heap.alloc(1024, torch.float32)   # fails here if peer access / VMM sharing is unavailable
            del probe
            return heap
        except Exception as e:   # noqa: BLE001 - any failure means "use the NCCL path"
            if os.environ.get("TS_SYMM_DEBUG"):
                import traceback
                traceback.print_exc()
            if dist.get_rank() == 0:
                print(f"[trainscale_b200] symmetric memory unavailable ({type(e).__name__}: {e}); using NCCL path")
            return None

    GUARD_BYTES = 256
    CANARY = 0xC5

    def alloc(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        import torch.distributed._symmetric_memory as symm_mem
        if os.environ.get("TS_DEBUG", "0") == "1":
            return self._alloc_guarded(numel, dtype)
        t = symm_mem.empty(numel, dtype=dtype, device=self.device)
        h = symm_mem.rendezvous(t, self.group)
        t.zero_()
        arr = ctypes.c_ulonglong * self.world
        mc = int(getattr(h, "multicast_ptr", 0) or 0) if self.use_multicast else 0
        buf = SymmBuffer(t, h, arr(*[int(p) for p in h.buffer_ptrs]), arr(*[int(p) for p in h.signal_pad_ptrs]), mc, {})
        self._by_ptr[t.data_ptr()] = buf
        self.bytes_allocated = getattr(self, "bytes_allocated", 0) + numel * t.element_size()
        return t

    def _alloc_guarded(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """Debug build: the buffer sits between two 256-byte guard zones filled with a canary byte.  The kernels get
        the addresses of the inner part, so a store that runs past either end of a (local or peer) buffer lands in a
        guard zone, where `check_canaries` finds it."""
        import torch.distributed._symmetric_memory as symm_mem
        esz = torch.empty(0, dtype=dtype).element_size()
        g = self.GUARD_BYTES
        nbytes = numel * esz
        raw = symm_mem.empty(nbytes + 2 * g, dtype=torch.uint8, device=self.device)
        h = symm_mem.rendezvous(raw, self.group)
        raw.zero_()
        raw[:g].fill_(self.CANARY)
        raw[g + nbytes:].fill_(self.CANARY)
        t = raw[g:g + nbytes].view(dtype)
        arr = ctypes.c_ulonglong * self.world
        mc = int(getattr(h, "multicast_ptr", 0) or 0) if self.use_multicast else 0
        buf = SymmBuffer(t, h, arr(*[int(p) + g for p in h.buffer_ptrs]), arr(*[int(p) for p in h.signal_pad_ptrs]),
                         mc + g if mc else 0, {})
        buf.raw = raw
        self._by_ptr[t.data_ptr()] = buf
        self.bytes_allocated = getattr(self, "bytes_allocated", 0) + nbytes + 2 * g
        return t

    def check_canaries(self) -> None:
        """Debug build: raises when any guard zone around a symmetric buffer of this rank was written."""
        bad = []
        for buf in self._by_ptr.values():
            raw = getattr(buf, "raw", None)
            if raw is None:
                continue
            g = self.GUARD_BYTES
            if not (bool((raw[:g] == self.CANARY).all()) and bool((raw[-g:] == self.CANARY).all())):
                bad.append(hex(buf.tensor.data_ptr()))
        if bad:
            from ..core.errors import CommunicationError
            raise CommunicationError(f"guard zone of symmetric buffer(s) {bad} was overwritten", rank=self.rank,
                                     world=self.world)

    def lookup(self, t: torch.Tensor) -> tuple[SymmBuffer, int]:
        """(buffer, byte offset) of a tensor that is a view into a symmetric allocation."""
        p = t.data_ptr()
        b = self._by_ptr.get(p)
        if b is not None:
            return b, 0
        for base, buf in self._by_ptr.items():
            size = buf.tensor.numel() * buf.tensor.element_size()
            if base <= p < base + size:
                return buf, p - base
        raise KeyError("tensor is not backed by symmetric memory")

    def status_flag(self) -> torch.Tensor:
        """1.0 on the device when a fused collective of this heap gave up waiting for a peer (no host sync)."""
        return self.status.ne(0).to(torch.float32)

    def check_status(self) -> None:
        """Host read of the status word; raises CommunicationError when a peer wait ran out."""
        if int(self.status.item()) != 0:
            self.status.zero_()
            from ..core.errors import CommunicationError
            raise CommunicationError("a peer did not arrive within the wait limit of a fused collective",
                                     rank=self.rank, world=self.world)
