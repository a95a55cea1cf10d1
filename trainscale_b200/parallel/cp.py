"""Context parallelism: causal-balanced sequence sharding and ring attention with a full backward pass.

Feature set after data_pipeline/trainer/distributed/context_parallel.py:1016-2231 (HEAD_TAIL / ZIGZAG balancers,
position ids per shard, ring order send to (r+1) % N / receive from (r-1) % N, LSE-weighted merge of partial
results `O = (e^{l1-m} O1 + e^{l2-m} O2) / (e^{l1-m} + e^{l2-m})`, output gather) and
hybrid_cp_scheduler.py:93-621 (per-sequence CP degree).  The reference's ring is forward-only placeholder math;
here forward and backward are exact:

  forward   each rank keeps its two query chunks (head-tail layout: chunks r and 2cp-1-r) and walks the ring of
            K/V shards; per step only the (query chunk, key chunk) pairs that the causal mask leaves non-empty are
            computed - two full pairs per step on every rank, so the work is balanced - with the flash kernel
            returning (O, LSE) per pair, merged in fp32;
  backward  the same walk with the merged LSE: dQ accumulates locally, each step's dK/dV travels on around the ring
            and arrives at its owner after cp steps.
K/V (and dK/dV) transfers are posted one step ahead on a side stream so they overlap the current step's kernels.
GQA-aware: only the Hkv key/value heads travel.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

from enum import IntEnum

import contextlib

import torch
import torch.distributed as dist
import torch.nn as nn

from ..utils.refargs import ANY, reference_kwargs

from ..ops.attention import attention_reference


# ------------------------------------------------------------------------------------------------ sharding layouts
class HeadTailBalancer:
    """2*cp chunks; rank r owns chunks r and 2cp-1-r (equal causal work per rank)."""

    def __init__(self, cp: int, rank: int):
        self.cp, self.rank = cp, rank

    def chunk_ids(self, rank: int | None = None) -> tuple[int, int]:
        r = self.rank if rank is None else rank
        return r, 2 * self.cp - 1 - r

    def indices(self, seq_len: int, rank: int | None = None) -> torch.Tensor:
        assert seq_len % (2 * self.cp) == 0, "sequence length must divide by 2*cp"
        c = seq_len // (2 * self.cp)
        a, b = self.chunk_ids(rank)
        return torch.cat((torch.arange(a * c, (a + 1) * c), torch.arange(b * c, (b + 1) * c)))

    def shard(self, x: torch.Tensor, dim: int = 1) -> torch.Tensor:
        return x.index_select(dim, self.indices(x.shape[dim]).to(x.device))

    def unshard(self, parts: list[torch.Tensor], dim: int = 1) -> torch.Tensor:
        """parts[r] = rank r's shard -> original order."""
        full_len = sum(p.shape[dim] for p in parts)
        order = torch.cat([self.indices(full_len, r) for r in range(self.cp)])
        inv = torch.empty_like(order)
        inv[order] = torch.arange(full_len)
        return torch.cat(parts, dim=dim).index_select(dim, inv.to(parts[0].device))

    # ---- stateless forms with the rank and the degree as arguments
    # (data_pipeline/trainer/distributed/context_parallel.py:980-1010); every balancer of this module inherits them
    def partition(self, tensor: torch.Tensor, cp_rank: int, cp_world_size: int, seq_dim: int = 1) -> torch.Tensor:
        return type(self)(cp_world_size, cp_rank).shard(tensor, seq_dim)

    def gather(self, shards: list[torch.Tensor], cp_world_size: int | None = None, seq_dim: int = 1) -> torch.Tensor:
        return type(self)(cp_world_size or len(shards), 0).unshard(list(shards), seq_dim)

    def compute_global_positions(self, local_len: int, cp_rank: int, cp_world_size: int,
                                 total_len: int | None = None) -> torch.Tensor:
        """Position in the full sequence of each of the rank's `local_len` tokens (what RoPE and the causal mask need)."""
        total = total_len if total_len is not None else local_len * cp_world_size
        idx = type(self)(cp_world_size, cp_rank).indices(total)
        if idx.numel() != local_len:
            raise ValueError(f"rank {cp_rank} of {cp_world_size} owns {idx.numel()} of {total} tokens, not {local_len}")
        return idx


class ZigZagBalancer(HeadTailBalancer):
    """Token-level boustrophedon: waves of cp tokens, odd waves reversed."""

    def indices(self, seq_len: int, rank: int | None = None) -> torch.Tensor:
        r = self.rank if rank is None else rank
        pos = torch.arange(seq_len)
        wave, off = pos // self.cp, pos % self.cp
        owner = torch.where(wave % 2 == 0, off, self.cp - 1 - off)
        return pos[owner == r]


class PTRRBalancer(HeadTailBalancer):
    """4*cp chunks walked forward, reverse, reverse, forward: rank r owns chunks r, 2cp-1-r, 3cp-1-r, 3cp+r
    (data_pipeline/trainer/distributed/context_parallel.py:1224).  Falls back to plain contiguous chunks when the
    sequence is shorter than 4*cp tokens."""

    def indices(self, seq_len: int, rank: int | None = None) -> torch.Tensor:
        r = self.rank if rank is None else rank
        n = 4 * self.cp
        c = seq_len // n
        if c < 1 or seq_len % n != 0:
            per = seq_len // self.cp
            return torch.arange(r * per, (r + 1) * per if r < self.cp - 1 else seq_len)
        ids = [r, 2 * self.cp - 1 - r, 3 * self.cp - 1 - r, 3 * self.cp + r]
        return torch.cat([torch.arange(i * c, (i + 1) * c) for i in ids])


class ContiguousBalancer(HeadTailBalancer):
    """Rank r owns tokens [r S/cp, (r+1) S/cp): the layout of all-to-all (Ulysses) sequence parallelism, where every
    rank ends up attending over the whole sequence and causal balance is not a concern."""

    def indices(self, seq_len: int, rank: int | None = None) -> torch.Tensor:
        assert seq_len % self.cp == 0, "sequence length must divide by cp"
        r = self.rank if rank is None else rank
        c = seq_len // self.cp
        return torch.arange(r * c, (r + 1) * c)


def create_balancer(name: str, cp: int, rank: int):
    name = (name or "head_tail").lower()
    if name in ("contiguous", "ulysses"):
        return ContiguousBalancer(cp, rank)
    if name in ("head_tail", "headtail"):
        return HeadTailBalancer(cp, rank)
    if name in ("zigzag", "zig_zag"):
        return ZigZagBalancer(cp, rank)
    if name == "ptrr":
        return PTRRBalancer(cp, rank)
    raise ValueError(f"unknown context-parallel balancer {name!r}")


def shard_inputs(batch: dict, cp: int, rank: int, balancer: str = "head_tail") -> dict:
    """Shard input_ids / labels / attention_mask / document_ids along the sequence and attach global position_ids.
    Labels are shifted BEFORE sharding (the next token of a chunk's last position lives on another rank)."""
    bal = create_balancer(balancer, cp, rank)
    ids = batch["input_ids"]
    S = ids.shape[1]
    out = {}
    labels = batch.get("labels", ids)
    shifted = torch.full_like(labels, -100)
    shifted[:, :-1] = labels[:, 1:]
    if "attention_mask" in batch:
        shifted = shifted.masked_fill(torch.cat((batch["attention_mask"][:, 1:], batch["attention_mask"][:, :1] * 0), 1) == 0, -100)
    out["input_ids"] = bal.shard(ids)
    out["labels"] = bal.shard(shifted)
    out["labels_shifted"] = True
    pos = batch.get("position_ids")
    if pos is None:
        pos = torch.arange(S, device=ids.device).unsqueeze(0).expand_as(ids)
    out["position_ids"] = bal.shard(pos)
    for k in ("attention_mask", "document_ids"):
        if k in batch:
            out[k] = bal.shard(batch[k])
    return out


def merge_partials(o1, lse1, o2, lse2):
    """Exact merge of two attention partials. o [.., D] fp32/bf16, lse [..] fp32 (rows broadcast over D)."""
    m = torch.maximum(lse1, lse2)
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w1, w2 = torch.exp(lse1 - m_safe), torch.exp(lse2 - m_safe)
    den = (w1 + w2).clamp(min=1e-38)
    o = (o1.float() * w1.unsqueeze(-1) + o2.float() * w2.unsqueeze(-1)) / den.unsqueeze(-1)
    return o, m_safe + torch.log(den)


# ------------------------------------------------------------------------------------------------ pair kernels
def _pair_forward(q, k, v, causal: bool, scale: float):
    """q [C, Hq, D], k/v [C, Hkv, D] -> (o [C, Hq, D] fp32-able, lse [Hq, C])."""
    C, Hq, D = q.shape
    Hkv = k.shape[1]
    if q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128):
        from ..ops import flash
        packed = torch.cat((q.reshape(C, -1), k.reshape(C, -1), v.reshape(C, -1)), dim=-1).unsqueeze(0)
        o, lse = flash.flash_forward_only(packed, Hq, Hkv, D, causal, scale)
        return o.view(C, Hq, D), lse
    g = Hq // Hkv
    qf = q.float().permute(1, 0, 2)
    kf = k.float().permute(1, 0, 2).repeat_interleave(g, 0)
    vf = v.float().permute(1, 0, 2).repeat_interleave(g, 0)
    s = qf @ kf.transpose(-1, -2) * scale
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(C, C, dtype=torch.bool, device=q.device), 1), float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.softmax(s, -1) @ vf
    return o.permute(1, 0, 2), lse


def _pair_backward(q, k, v, o_final, lse_final, do, causal: bool, scale: float):
    """Gradients of one (q chunk, kv chunk) pair given the merged LSE and final output: (dq, dk, dv)."""
    C, Hq, D = q.shape
    Hkv = k.shape[1]
    if q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128):
        from ..ops import flash
        packed = torch.cat((q.reshape(C, -1), k.reshape(C, -1), v.reshape(C, -1)), dim=-1).contiguous()
        d = flash._bwd(packed, o_final.reshape(C, -1).to(q.dtype).contiguous(), lse_final.contiguous(),
                       do.reshape(C, -1).to(q.dtype).contiguous(), Hq, Hkv, D, 1, C, None, C, causal, scale)
        dq, dk, dv = d.split((Hq * D, Hkv * D, Hkv * D), dim=-1)
        return dq.view(C, Hq, D).float(), dk.view(C, Hkv, D).float(), dv.view(C, Hkv, D).float()
    g = Hq // Hkv
    qf, dof = q.float().permute(1, 0, 2), do.float().permute(1, 0, 2)
    kf = k.float().permute(1, 0, 2).repeat_interleave(g, 0)
    vf = v.float().permute(1, 0, 2).repeat_interleave(g, 0)
    s = qf @ kf.transpose(-1, -2) * scale
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(C, C, dtype=torch.bool, device=q.device), 1), float("-inf"))
    p = torch.exp(s - lse_final.unsqueeze(-1))
    delta = (dof * o_final.float().permute(1, 0, 2)).sum(-1, keepdim=True)
    dv = p.transpose(-1, -2) @ dof
    ds = p * (dof @ vf.transpose(-1, -2) - delta) * scale
    dq = ds @ kf
    dk = ds.transpose(-1, -2) @ qf
    dk = dk.view(Hkv, g, C, D).sum(1)
    dv = dv.view(Hkv, g, C, D).sum(1)
    return dq.permute(1, 0, 2), dk.permute(1, 0, 2), dv.permute(1, 0, 2)


def _pairs_for_step(r: int, j: int, cp: int):
    """(query slot, key slot, causal) pairs that are non-empty when rank r holds the K/V of rank j.
    Slot 0 is the early chunk (index rank), slot 1 the late chunk (index 2cp-1-rank)."""
    if j == r:
        return [(0, 0, True), (1, 0, False), (1, 1, True)]
    if j < r:
        return [(0, 0, False), (1, 0, False)]
    return [(1, 0, False), (1, 1, False)]


class _RingExchange:
    """Double-buffered ring send/recv on a side stream (send to rank+1, receive from rank-1)."""

    def __init__(self, group, rank: int, cp: int, device):
        self.group, self.rank, self.cp = group, rank, cp
        self.ranks = dist.get_process_group_ranks(group) if group is not None else list(range(cp))
        self.cuda = torch.device(device).type == "cuda"
        self.stream = torch.cuda.Stream(device=device) if self.cuda else None

    def start(self, send: torch.Tensor):
        recv = torch.empty_like(send)
        dst, src = self.ranks[(self.rank + 1) % self.cp], self.ranks[(self.rank - 1) % self.cp]
        if self.cuda:
            self.stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.stream):
                works = dist.batch_isend_irecv([dist.P2POp(dist.isend, send, dst, self.group),
                                                dist.P2POp(dist.irecv, recv, src, self.group)])
        else:
            works = dist.batch_isend_irecv([dist.P2POp(dist.isend, send, dst, self.group),
                                            dist.P2POp(dist.irecv, recv, src, self.group)])
        return recv, works, send

    def finish(self, handle):
        recv, works, _send = handle
        for w in works:
            w.wait()
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.stream)
        return recv


class _PeerKV:
    """K/V exchange of context parallelism over NVLink peer memory instead of NCCL send/recv.

    On an NVSwitch node every rank reaches every peer at full bandwidth, so there is no reason to pass K/V around a ring
    hop by hop: each rank publishes its K/V chunk in a symmetric buffer and PULLS all other chunks with one kernel
    (`csrc/comm.cu` pull all-gather, plain peer loads) on a side stream while the attention of its own chunk runs.
    In backward every rank writes its partial dK/dV for all chunks into a symmetric fp32 buffer and the owners sum
    their slot across ranks with the peer-memory reduce-scatter kernel.  Buffers are allocated once per
    (group, size) - symmetric allocation is a collective - and reused by every layer; a device-side barrier before
    each reuse keeps a fast rank from overwriting a slot that a slow rank is still reading."""

    _heaps: dict = {}
    _bufs: dict = {}

    @classmethod
    def get(cls, group, device, numel: int, dtype):
        from .symm import SymmetricHeap
        hk = (id(group), str(device))
        if hk not in cls._heaps:
            cls._heaps[hk] = SymmetricHeap.try_create(group, device)
        heap = cls._heaps[hk]
        if heap is None:
            return None
        bk = hk + (numel, dtype)
        if bk not in cls._bufs:
            cp = heap.world
            cls._bufs[bk] = cls(heap, heap.alloc(cp * numel, dtype), heap.alloc(cp * numel, torch.float32), numel,
                                torch.cuda.Stream(device=device))
        return cls._bufs[bk]

    def __init__(self, heap, kv_all, dkv_all, numel, stream):
        self.heap, self.kv_all, self.dkv_all, self.numel, self.stream = heap, kv_all, dkv_all, numel, stream

    def publish_and_gather(self, kv: torch.Tensor):
        """Start pulling everybody's K/V; returns the [cp, ...] view that is complete after `wait()`."""
        from . import fused_comm
        heap, r, n = self.heap, self.heap.rank, self.numel
        fused_comm.barrier(heap, self.kv_all)
        self.kv_all[r * n:(r + 1) * n].copy_(kv.reshape(-1))
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            fused_comm.all_gather_inplace(heap, self.kv_all, r * n, n)
        return self.kv_all.view((heap.world,) + tuple(kv.shape))

    def wait(self) -> None:
        torch.cuda.current_stream().wait_stream(self.stream)

    def grad_slots(self, shape) -> torch.Tensor:
        """Zeroed [cp, *shape] fp32 partial-gradient slots (slot j = my contribution to rank j's dK/dV)."""
        from . import fused_comm
        fused_comm.barrier(self.heap, self.dkv_all)
        self.dkv_all.zero_()
        return self.dkv_all.view((self.heap.world,) + tuple(shape))

    def reduce_grads(self, out: torch.Tensor) -> torch.Tensor:
        """out (fp32, one slot) = sum over ranks of their slot for me."""
        from . import fused_comm
        fused_comm.reduce_scatter_fp32(self.heap, self.dkv_all, out.reshape(-1), self.heap.rank * self.numel, 1.0,
                                       None, None)
        return out


def _use_peer(q: torch.Tensor, comm: str) -> bool:
    return comm in ("auto", "peer", "fused") and q.is_cuda


class _PeerAttention(torch.autograd.Function):
    """Same maths as `_RingAttention`; K/V and dK/dV travel through `_PeerKV`."""

    @staticmethod
    def forward(ctx, q, k, v, group, scale, pk):
        cp, r = dist.get_world_size(group), dist.get_rank(group)
        C = q.shape[0] // 2
        kv = torch.stack((k, v)).contiguous()
        kv_all = pk.publish_and_gather(kv)
        o = [None, None]
        lse = [None, None]
        for step in range(cp):
            j = (r - step) % cp
            if step == 1:
                pk.wait()                                   # the pull ran under the attention of the local chunk
            cur = kv if step == 0 else kv_all[j]
            for qs, ks, causal in _pairs_for_step(r, j, cp):
                po, pl = _pair_forward(q[qs * C:(qs + 1) * C], cur[0, ks * C:(ks + 1) * C], cur[1, ks * C:(ks + 1) * C],
                                       causal, scale)
                if o[qs] is None:
                    o[qs], lse[qs] = po.float(), pl
                else:
                    o[qs], lse[qs] = merge_partials(o[qs], lse[qs].transpose(0, 1), po, pl.transpose(0, 1))
                    lse[qs] = lse[qs].transpose(0, 1)
        if cp == 1:
            pk.wait()
        out = torch.cat((o[0], o[1])).to(q.dtype)
        lse_all = torch.cat((lse[0], lse[1]), dim=1).contiguous()
        ctx.save_for_backward(q, k, v, out, lse_all)
        ctx.group, ctx.scale, ctx.pk = group, scale, pk
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse_all = ctx.saved_tensors
        group, scale, pk = ctx.group, ctx.scale, ctx.pk
        cp, r = dist.get_world_size(group), dist.get_rank(group)
        C = q.shape[0] // 2
        kv = torch.stack((k, v)).contiguous()
        kv_all = pk.publish_and_gather(kv)
        slots = pk.grad_slots(kv.shape)                     # [cp, 2, 2C, Hkv, D] fp32
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        for step in range(cp):
            j = (r - step) % cp
            if step == 1:
                pk.wait()
            cur = kv if step == 0 else kv_all[j]
            for qs, ks, causal in _pairs_for_step(r, j, cp):
                sl_q, sl_k = slice(qs * C, (qs + 1) * C), slice(ks * C, (ks + 1) * C)
                a, b, c = _pair_backward(q[sl_q], cur[0, sl_k], cur[1, sl_k], out[sl_q], lse_all[:, sl_q], do[sl_q],
                                         causal, scale)
                dq[sl_q] += a
                slots[j, 0, sl_k] += b
                slots[j, 1, sl_k] += c
        if cp == 1:
            pk.wait()
        dkv = pk.reduce_grads(torch.empty(kv.shape, dtype=torch.float32, device=q.device))
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None, None


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, group, scale):
        # q [2C, Hq, D] (slot 0 rows then slot 1 rows), k/v [2C, Hkv, D]
        cp = dist.get_world_size(group)
        r = dist.get_rank(group)
        C = q.shape[0] // 2
        ex = _RingExchange(group, r, cp, q.device)
        kv = torch.stack((k, v)).contiguous()           # [2, 2C, Hkv, D]
        o = [None, None]
        lse = [None, None]
        for step in range(cp):
            j = (r - step) % cp
            nxt = ex.start(kv) if step + 1 < cp else None
            for qs, ks, causal in _pairs_for_step(r, j, cp):
                po, pl = _pair_forward(q[qs * C:(qs + 1) * C], kv[0, ks * C:(ks + 1) * C], kv[1, ks * C:(ks + 1) * C],
                                       causal, scale)
                if o[qs] is None:
                    o[qs], lse[qs] = po.float(), pl
                else:
                    o[qs], lse[qs] = merge_partials(o[qs], lse[qs].transpose(0, 1), po, pl.transpose(0, 1))
                    lse[qs] = lse[qs].transpose(0, 1)
            if nxt is not None:
                kv = ex.finish(nxt)
        out = torch.cat((o[0], o[1])).to(q.dtype)
        lse_all = torch.cat((lse[0], lse[1]), dim=1).contiguous()   # [Hq, 2C]
        ctx.save_for_backward(q, k, v, out, lse_all)
        ctx.group, ctx.scale = group, scale
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse_all = ctx.saved_tensors
        group, scale = ctx.group, ctx.scale
        cp = dist.get_world_size(group)
        r = dist.get_rank(group)
        C = q.shape[0] // 2
        ex_kv = _RingExchange(group, r, cp, q.device)
        ex_g = _RingExchange(group, r, cp, q.device)
        kv = torch.stack((k, v)).contiguous()
        dkv = torch.zeros(2, 2 * C, k.shape[1], k.shape[2], dtype=torch.float32, device=q.device)
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        for step in range(cp):
            j = (r - step) % cp
            nxt = ex_kv.start(kv) if step + 1 < cp else None
            for qs, ks, causal in _pairs_for_step(r, j, cp):
                sl_q, sl_k = slice(qs * C, (qs + 1) * C), slice(ks * C, (ks + 1) * C)
                a, b, c = _pair_backward(q[sl_q], kv[0, sl_k], kv[1, sl_k], out[sl_q], lse_all[:, sl_q], do[sl_q],
                                         causal, scale)
                dq[sl_q] += a
                dkv[0, sl_k] += b
                dkv[1, sl_k] += c
            # the gradient buffer belongs to rank j's K/V: pass it on so that it is home after cp hops
            h = ex_g.start(dkv)
            if nxt is not None:
                kv = ex_kv.finish(nxt)
            dkv = ex_g.finish(h)
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group, scale: float | None = None,
                   comm: str | None = None) -> torch.Tensor:
    """Causal attention over a sequence sharded with the head-tail layout. q [B=1, S_local, Hq, D]; returns the same
    shape. Local rows are (chunk rank | chunk 2cp-1-rank).
    `comm`: "nccl" = K/V passed around the ring with batched send/recv; "peer" = pulled over NVLink peer memory by the
    framework's own kernels (`_PeerKV`); "auto" (default, or env TS_CP_COMM) = peer on CUDA when symmetric memory is
    available, else nccl."""
    import os
    B, S, Hq, D = q.shape
    assert B == 1, "ring attention handles one (packed) sequence per step"
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    comm = comm or os.environ.get("TS_CP_COMM", "auto")
    if _use_peer(q, comm):
        kv_numel = 2 * k[0].numel()
        pk = _PeerKV.get(group, q.device, kv_numel, k.dtype) if (kv_numel * k.element_size()) % 16 == 0 else None
        if pk is not None:
            return _PeerAttention.apply(q[0], k[0], v[0], group, scale, pk).unsqueeze(0)
        if comm == "peer":
            raise RuntimeError("peer-memory context parallelism was requested but symmetric memory is unavailable")
    o = _RingAttention.apply(q[0], k[0], v[0], group, scale)
    return o.unsqueeze(0)


def attention_qkv_cp(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, group) -> torch.Tensor:
    """Drop-in for ops.attention.attention_qkv under context parallelism (qkv already rotated with global positions)."""
    B, S, _ = qkv.shape
    q, k, v = qkv.split((n_heads * head_dim, n_kv_heads * head_dim, n_kv_heads * head_dim), dim=-1)
    o = ring_attention(q.reshape(B, S, n_heads, head_dim), k.reshape(B, S, n_kv_heads, head_dim),
                       v.reshape(B, S, n_kv_heads, head_dim), group)
    return o.reshape(B, S, n_heads * head_dim)


def gather_output(x_local: torch.Tensor, group, balancer: str = "head_tail", dim: int = 1) -> torch.Tensor:
    cp, r = dist.get_world_size(group), dist.get_rank(group)
    parts = [torch.empty_like(x_local) for _ in range(cp)]
    dist.all_gather(parts, x_local.contiguous(), group=group)
    return create_balancer(balancer, cp, r).unshard(parts, dim)


def estimate_memory_per_gpu(seq_len: int = None, cp: int = None, hidden: int = None, n_layers: int = 1,
                            n_kv_heads: int = None, head_dim: int = None, bytes_per_el: int = 2,
                            checkpointing: bool = True, *, batch_size: int | None = None, hidden_dim: int | None = None,
                            num_heads: int | None = None, cp_degree: int | None = None, precision: str | None = None):
    """Per-GPU activation and ring-buffer sizes of a context-parallel layer stack (a dict, in GiB).  The reference's
    keyword form (`batch_size, seq_len, hidden_dim, num_heads, cp_degree, precision`) describes ONE layer without
    recomputation and returns its bytes as an int (data_pipeline/trainer/distributed/context_parallel.py:2107)."""
    if head_dim is None and n_kv_heads is not None and cp_degree is None and hidden_dim is None:
        # five positional sizes and no head dimension: (batch_size, seq_len, hidden_dim, num_heads, cp_degree)
        batch_size, seq_len, hidden_dim, num_heads, cp_degree = seq_len, cp, hidden, n_layers, n_kv_heads
    if cp_degree is not None or hidden_dim is not None:
        eb = {"fp32": 4, "fp16": 2, "bf16": 2, "fp8": 1}[precision or "bf16"]
        d = estimate_memory_per_gpu(seq_len, cp_degree or 1, hidden_dim, 1, num_heads, hidden_dim // num_heads, eb, False)
        return int((d["activations_gb"] + d["ring_buffers_gb"]) * 2 ** 30) * int(batch_size or 1)
    s = seq_len // cp
    act = s * hidden * bytes_per_el * (2 if checkpointing else 34) * n_layers
    kv_ring = 2 * 2 * s * n_kv_heads * head_dim * bytes_per_el   # double-buffered K and V
    return {"tokens_per_gpu": s, "activations_gb": act / 2 ** 30, "ring_buffers_gb": kv_ring / 2 ** 30}


# ------------------------------------------------------------------------------------------------ hybrid DP x CP
@dataclass
class HybridCPConfig:
    max_tokens_per_rank: int = 8192
    world_size: int = 8


class BalancedCPScheduler:
    """Per-sequence CP degree = next power of two of len / max_tokens_per_rank; greedy balance of the quadratic
    workload L^2 / cp over GPUs (data_pipeline/trainer/distributed/hybrid_cp_scheduler.py:149-621)."""

    def __init__(self, cfg: "HybridCPConfig | int | None" = None, dp_cp_group=None, *, max_seq_len_per_rank: int | None = None):
        """`BalancedCPScheduler(HybridCPConfig(...))`, or the reference's `(max_seq_len_per_rank, dp_cp_group)`: the world
        is then the size of that group (of the default group, or 1, when it is None)."""
        if max_seq_len_per_rank is not None or isinstance(cfg, int):
            per_rank = int(max_seq_len_per_rank if max_seq_len_per_rank is not None else cfg)
            if dp_cp_group is not None and hasattr(dp_cp_group, "size"):
                world = int(dp_cp_group.size())
            else:
                world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
            cfg = HybridCPConfig(max_tokens_per_rank=per_rank, world_size=world)
        self.cfg = cfg if cfg is not None else HybridCPConfig()

    max_seq_len_per_rank = property(lambda self: self.cfg.max_tokens_per_rank)
    total_hdp_gpus = property(lambda self: self.cfg.world_size)

    @reference_kwargs(seq_len="length")
    def gpus_needed(self, length: int) -> int:
        n = max(1, math.ceil(length / self.cfg.max_tokens_per_rank))
        return min(self.cfg.world_size, 1 << (n - 1).bit_length())

    @staticmethod
    def workload(length: int, cp: int) -> float:
        return length * length / cp

    def schedule(self, lengths: list[int]) -> list[list[tuple[int, int]]]:
        """Returns per-GPU lists of (sequence index, cp degree); sequences needing cp GPUs occupy cp aligned slots."""
        W = self.cfg.world_size
        load = [0.0] * W
        plan: list[list[tuple[int, int]]] = [[] for _ in range(W)]
        for i in sorted(range(len(lengths)), key=lambda k: -lengths[k]):
            cp = self.gpus_needed(lengths[i])
            best, best_load = 0, float("inf")
            for start in range(0, W, cp):
                l = max(load[start:start + cp])
                if l < best_load:
                    best, best_load = start, l
            w = self.workload(lengths[i], cp)
            for g in range(best, best + cp):
                load[g] = best_load + w
                plan[g].append((i, cp))
        return plan

    # -- the reference scheduler's finer-grained steps (hybrid_cp_scheduler.py:149-621), on the same cost model
    @reference_kwargs(seq_length="length", cp_size="cp")
    def get_total_workload(self, length: int, cp: int | None = None) -> float:
        """Attention work one GPU does for a sequence of `length` split over `cp` GPUs: L^2 / cp."""
        return self.workload(length, cp or self.gpus_needed(length))

    def _buckets_in_order(self, samples: list, estimator) -> list:
        """(sample id, length) pairs cut, in the given order, into k consecutive runs of near-equal work, k = number of
        distinct CP degrees among them (data_pipeline/trainer/distributed/hybrid_cp_scheduler.py:197)."""
        from collections import deque
        if not samples:
            return []
        k = len({self.gpus_needed(l) for _, l in samples})
        work = [float(estimator(l, self.gpus_needed(l))) for _, l in samples]
        target, out, cur, acc = sum(work) / k, [], [], 0.0
        for i, s in enumerate(samples):
            must_close = len(samples) - i <= k - len(out) - 1          # keep one sample for each bucket still to open
            if cur and len(out) < k - 1 and (acc + work[i] > 1.1 * target or must_close):
                out.append(deque(cur))
                cur, acc = [], 0.0
            cur.append(s)
            acc += work[i]
        out.append(deque(cur))
        return out

    def make_buckets_equal(self, lengths: list | None = None, num_buckets=None, *, sample_seqlens=None,
                           compute_estimator=None):
        """Longest-processing-time split of sequence indices into `num_buckets` buckets of near-equal total work.
        `make_buckets_equal(sample_seqlens, compute_estimator)` is the reference's form: (id, length) pairs kept in
        order, one deque per distinct CP degree."""
        if sample_seqlens is not None or compute_estimator is not None or callable(num_buckets):
            return self._buckets_in_order(list(sample_seqlens if sample_seqlens is not None else lengths),
                                          compute_estimator or num_buckets)
        buckets: list[list[int]] = [[] for _ in range(num_buckets)]
        load = [0.0] * num_buckets
        for i in sorted(range(len(lengths)), key=lambda k: -self.get_total_workload(lengths[k])):
            b = min(range(num_buckets), key=load.__getitem__)
            buckets[b].append(i)
            load[b] += self.get_total_workload(lengths[i])
        return buckets

    def _next_group_reference(self, samples: list, estimator, total_gpus: int, delta: float, strategy: str):
        """(micro_batches, leftovers, exec_times, sample_ids_per_gpu) for the samples that fit `total_gpus` once: every
        GPU of a sample's group lists the sample's full length and is charged estimator(length, cp)
        (data_pipeline/trainer/distributed/hybrid_cp_scheduler.py:264)."""
        if strategy not in ("dp", "pp"):
            raise ValueError(f"strategy must be 'dp' or 'pp', got {strategy!r}")
        W = int(total_gpus)
        sched = self if W == self.cfg.world_size else BalancedCPScheduler(HybridCPConfig(self.cfg.max_tokens_per_rank, W))
        samples = list(samples)
        lengths = [l for _, l in samples]
        chosen, nxt = sched.next_hdp_group(lengths, 0) if samples else ([], 0)
        # more single-GPU samples may ride along while the spread of the per-GPU times stays within delta
        idx = [i for i, _ in chosen]
        plan = sched.balanced_schedule([lengths[i] for i in idx]) if idx else [[] for _ in range(W)]
        times = [sum(float(estimator(lengths[idx[j]], cp)) for j, cp in gpu) for gpu in plan]
        while nxt < len(samples) and sched.gpus_needed(lengths[nxt]) == 1 and times:
            lo = min(range(W), key=times.__getitem__)
            cost = float(estimator(lengths[nxt], 1))
            if times[lo] + cost > (1.0 + delta) * max(times):
                break
            idx.append(nxt)
            plan[lo].append((len(idx) - 1, 1))
            times[lo] += cost
            nxt += 1
        micro = [[lengths[idx[j]] for j, _ in gpu] for gpu in plan]
        ids = [[samples[idx[j]][0] for j, _ in gpu] for gpu in plan]
        return micro, samples[nxt:], times, ids

    def next_hdp_group(self, lengths: list | None = None, start=0, total_gpus: int | None = None, delta: float = 0.05,
                       strategy: str = "dp", *, sample_seqlens=None, compute_estimator=None):
        """Takes sequences from `start` on until their GPU demand fills the world: returns [(index, cp)], next start.
        `next_hdp_group(sample_seqlens, compute_estimator, total_gpus, delta, strategy)` is the reference's form."""
        if sample_seqlens is not None or compute_estimator is not None or callable(start):
            return self._next_group_reference(sample_seqlens if sample_seqlens is not None else lengths,
                                              compute_estimator or start, total_gpus or self.cfg.world_size, delta, strategy)
        used, out, i = 0, [], start
        while i < len(lengths):
            cp = self.gpus_needed(lengths[i])
            if used + cp > self.cfg.world_size:
                break
            out.append((i, cp))
            used += cp
            i += 1
        if not out and i < len(lengths):          # a single sequence that wants the whole world
            out.append((i, self.cfg.world_size))
            i += 1
        return out, i

    def get_groups_and_subsamples(self, sample_id_seqlens: list[tuple[int, int]], config: "HybridCPConfig | None" = None):
        """Cut a batch of (sample id, length) into successive groups that each fill the world once; inside a group
        the samples are balanced over the GPUs by `schedule`.  Returns (groups, sample_id_groups): groups[g][gpu] is
        that GPU's list of (sample id, cp degree) in group g, sample_id_groups[g][gpu] the sample ids alone
        (data_pipeline/trainer/distributed/hybrid_cp_scheduler.py:580-621)."""
        sched = self if config is None else BalancedCPScheduler(config)
        items = sorted(sample_id_seqlens, key=lambda t: -t[1])              # longest first packs best
        lengths = [l for _, l in items]
        groups, id_groups, start = [], [], 0
        while start < len(items):
            chosen, nxt = sched.next_hdp_group(lengths, start)
            idx = [i for i, _ in chosen]
            plan = sched.schedule([lengths[i] for i in idx])
            groups.append([[(items[idx[j]][0], cp) for j, cp in gpu] for gpu in plan])
            id_groups.append([[sid for sid, _ in gpu] for gpu in groups[-1]])
            start = nxt
        return groups, id_groups

    def _trim_overloaded(self, plan: list[list[tuple[int, int]]], lengths: list[int], tolerance: float = 1.25):
        """Moves single-GPU sequences off GPUs whose load exceeds tolerance x mean onto the least loaded GPU."""
        def load(g):
            return sum(self.workload(lengths[i], cp) for i, cp in plan[g])
        W = len(plan)
        for _ in range(4 * W):
            loads = [load(g) for g in range(W)]
            mean = sum(loads) / W
            hi = max(range(W), key=loads.__getitem__)
            lo = min(range(W), key=loads.__getitem__)
            movable = [(i, cp) for i, cp in plan[hi] if cp == 1]
            if loads[hi] <= tolerance * mean or not movable:
                break
            item = min(movable, key=lambda t: lengths[t[0]])
            if loads[lo] + self.workload(lengths[item[0]], 1) >= loads[hi]:
                break
            plan[hi].remove(item)
            plan[lo].append(item)
        return plan

    def _fill_empty_gpus(self, plan: list[list[tuple[int, int]]], lengths: list[int]):
        """No GPU may idle while another holds several single-GPU sequences."""
        for g in range(len(plan)):
            if plan[g]:
                continue
            donors = [d for d in range(len(plan)) if sum(1 for _, cp in plan[d] if cp == 1) >= 2 or
                      (len(plan[d]) >= 2 and any(cp == 1 for _, cp in plan[d]))]
            if not donors:
                continue
            d = max(donors, key=lambda k: sum(self.workload(lengths[i], cp) for i, cp in plan[k]))
            item = max((t for t in plan[d] if t[1] == 1), key=lambda t: lengths[t[0]])
            plan[d].remove(item)
            plan[g].append(item)
        return plan

    def balanced_schedule(self, lengths: list[int]) -> list[list[tuple[int, int]]]:
        return self._fill_empty_gpus(self._trim_overloaded(self.schedule(lengths), lengths), lengths)


def hybrid_context_parallel_forward_backward(model_step=None, batches: list[dict] | None = None,
                                             scheduler: "BalancedCPScheduler | None" = None, rank: int = 0,
                                             lengths: list[int] | None = None, *, forward_step_func=None,
                                             data_iterator=None, model=None, num_microbatches: int = 1,
                                             forward_data_store: list | None = None, config=None,
                                             collect_non_loss_data: bool = False, first_val_step=None,
                                             forward_only: bool = False, no_sync_func=None, total_num_tokens=0,
                                             model_type=None, get_data_parallel_rank=None,
                                             get_tensor_model_parallel_rank=None, get_tensor_model_parallel_src_rank=None,
                                             get_tensor_model_parallel_group=None, get_data_parallel_group=None):
    """Runs `model_step(batch, cp_degree, cp_slot)` for every sequence this rank takes part in, in schedule order.
    `batches[i]` is sequence i (dict with input_ids [1, L]); `cp_slot` is this rank's position inside the sequence's
    group of `cp_degree` consecutive ranks.  Returns the per-sequence results of this rank.

    With `forward_step_func=` (the reference's keywords, data_pipeline/trainer/distributed/hybrid_cp_scheduler.py:627,
    where the body is left unimplemented) the Megatron-style loop runs instead: for each of `num_microbatches`,
    `forward_step_func(data_iterator, model)` returns (output, loss_func); `loss_func(output)` returns (loss, stats) or
    (loss, num_tokens, stats); the loss is back-propagated unless `forward_only`, gradient synchronisation is held
    back by `no_sync_func()` on all but the last micro-batch; returns (forward_data_store, total_num_tokens)."""
    if forward_step_func is not None:
        import contextlib
        store = forward_data_store if forward_data_store is not None else []
        for i in range(int(num_microbatches)):
            last = i == num_microbatches - 1
            hold = no_sync_func() if (no_sync_func is not None and not last and not forward_only) else contextlib.nullcontext()
            with hold:
                output, loss_func = forward_step_func(data_iterator, model)
                if collect_non_loss_data:
                    store.append(loss_func(output, non_loss_data=True))
                    continue
                res = loss_func(output)
                loss, stats = res[0], res[-1]
                if len(res) == 3:
                    total_num_tokens = total_num_tokens + res[1]
                if not forward_only:
                    (loss / num_microbatches).backward()
                store.append(stats)
        return store, total_num_tokens
    lengths = lengths or [int(b["input_ids"].shape[1]) for b in batches]
    plan = scheduler.balanced_schedule(lengths)
    out = []
    for i, cp in plan[rank]:
        out.append(model_step(batches[i], cp, rank % cp))
    return out


# ------------------------------------------------------------------------------------------------ engine-level API
class LoadBalancer(IntEnum):
    NONE = 0
    HEAD_TAIL = 1
    ZIGZAG = 2
    PTRR = 3


class CommBackend(IntEnum):
    NCCL = 0
    GLOO = 1


class AttentionPattern(IntEnum):
    CAUSAL = 0
    FULL = 1
    SLIDING_WINDOW = 2


def get_load_balancer(strategy: "LoadBalancer | str", cp: int = 1, rank: int = 0):
    name = strategy.name.lower() if isinstance(strategy, LoadBalancer) else str(strategy).lower()
    if name == "none":
        raise ValueError("contiguous (unbalanced) sharding is not provided: causal work would be rank-skewed")
    return create_balancer(name, cp, rank)


class TensorArena:
    """Bump allocator over one pre-allocated byte buffer: per-step scratch without touching the caching allocator.
    `allocate` returns Err when the arena is exhausted; `reset` makes the whole arena available again."""

    ALIGN = 256

    @reference_kwargs(capacity_bytes="size_bytes")
    def __init__(self, size_bytes: int, device: torch.device | str = "cpu", dtype: torch.dtype | None = None):
        """`dtype`: the element type most allocations will have (recorded as `default_dtype`; the arena itself is bytes)."""
        self.default_dtype = dtype
        self.size = int(size_bytes)
        self.buf = torch.empty(self.size, dtype=torch.uint8, device=device)
        self.offset = 0
        self.peak = 0

    def allocate(self, shape: tuple, dtype: torch.dtype):
        from ..core.types import Err, Ok
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        start = (self.offset + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        if start + nbytes > self.size:
            return Err(MemoryError(f"arena exhausted: need {nbytes} bytes, {self.size - start} left"))
        self.offset = start + nbytes
        self.peak = max(self.peak, self.offset)
        return Ok(self.buf[start:start + nbytes].view(dtype).view(shape))

    def reset(self) -> None:
        self.offset = 0

    @property
    def utilization(self) -> float:
        return self.offset / self.size if self.size else 0.0

    @property
    def available_bytes(self) -> int:
        return self.size - self.offset


class RingBufferPool:
    """K/V staging buffers of the ring: while one is computed on, one is being sent and one received."""

    FREE, COMPUTE, SENDING, RECEIVING = range(4)

    def __init__(self, *args, count: int | None = None, shape=None, dtype: torch.dtype | None = None,
                 device: torch.device | str | None = None, num_buffers: int | None = None, pin_memory: bool = False):
        """`RingBufferPool(count, shape, dtype, device)`, or the reference's `(shape, dtype, device, num_buffers=3,
        pin_memory=False)` (data_pipeline/trainer/distributed/context_parallel.py RingBufferPool); `pin_memory` pins
        host-side buffers when a CUDA device is present."""
        names = ("shape", "dtype", "device", "num_buffers", "pin_memory") if args and not isinstance(args[0], int) \
            else ("count", "shape", "dtype", "device")
        if len(args) > len(names):
            raise TypeError(f"at most {names} positionally")
        given = dict(zip(names, args))
        shape, dtype = given.get("shape", shape), given.get("dtype", dtype)
        device = given.get("device", device) or "cpu"
        pin_memory = given.get("pin_memory", pin_memory)
        count = given.get("count", count)
        count = int(count if count is not None else given.get("num_buffers", num_buffers if num_buffers is not None else 3))
        if shape is None or dtype is None:
            raise TypeError("shape and dtype are required")
        if count < 2:
            raise ValueError("a ring needs at least two buffers")
        pin = bool(pin_memory) and torch.device(device).type == "cpu" and torch.cuda.is_available()
        self.buffers = [torch.empty(tuple(shape), dtype=dtype, device=device, pin_memory=pin) for _ in range(count)]
        self.state = [self.FREE] * count

    def _take(self, new_state: int) -> int:
        for i, s in enumerate(self.state):
            if s == self.FREE:
                self.state[i] = new_state
                return i
        raise RuntimeError("no free ring buffer (a transfer was not marked free)")

    def get_compute_buffer(self) -> tuple[torch.Tensor, int]:
        i = self._take(self.COMPUTE)
        return self.buffers[i], i

    def get_recv_buffer(self) -> tuple[torch.Tensor, int]:
        i = self._take(self.RECEIVING)
        return self.buffers[i], i

    def mark_sending(self, idx: int) -> None:
        self.state[idx] = self.SENDING

    def mark_receiving(self, idx: int) -> None:
        self.state[idx] = self.RECEIVING

    def mark_free(self, idx: int) -> None:
        self.state[idx] = self.FREE

    def get_buffer(self, idx: int) -> torch.Tensor:
        return self.buffers[idx]


@dataclass
class ContextParallelMetrics:
    steps: int = 0
    bytes_sent: int = 0
    comm_ms: float = 0.0
    compute_ms: float = 0.0
    flops: float = 0.0

    def compute_bandwidth_gbps(self) -> float:
        return self.bytes_sent / (self.comm_ms * 1e6) if self.comm_ms > 0 else 0.0

    def compute_tflops(self) -> float:
        return self.flops / (self.compute_ms * 1e9) if self.compute_ms > 0 else 0.0

    def to_dict(self) -> dict:
        return dict(self.__dict__, bandwidth_gbps=self.compute_bandwidth_gbps(), tflops=self.compute_tflops())


@dataclass
class ContextParallelConfig:
    cp_degree: int = 1
    load_balancer: LoadBalancer = LoadBalancer.HEAD_TAIL
    attention_pattern: AttentionPattern = AttentionPattern.CAUSAL
    sliding_window_size: int = 0
    use_ring_attention: bool = True
    ring_buffer_count: int = 3
    overlap_comm_compute: bool = True
    use_arena_allocator: bool = False
    arena_size_gb: float = 2.0
    use_activation_checkpointing: bool = False
    use_triton_kernels: bool = False          # the sm_100a flash kernels are used on CUDA
    comm_backend: CommBackend = CommBackend.NCCL

    def __post_init__(self):
        if isinstance(self.load_balancer, str):
            self.load_balancer = LoadBalancer[self.load_balancer.upper()]
        if self.cp_degree < 1:
            raise ValueError("cp_degree must be >= 1")
        if self.attention_pattern is not AttentionPattern.CAUSAL and self.cp_degree > 1:
            raise ValueError("the ring implementation covers causal attention")
        if self.load_balancer is not LoadBalancer.HEAD_TAIL and self.use_ring_attention and self.cp_degree > 1:
            raise ValueError("ring attention pairs the head-tail layout; zigzag / ptrr serve the all-gather path")

    @classmethod
    def from_dict(cls, config_dict: dict):
        from ..core.types import Err, Ok
        try:
            known = {k: v for k, v in config_dict.items() if k in cls.__dataclass_fields__}
            return Ok(cls(**known))
        except (ValueError, KeyError, TypeError) as e:
            return Err(ValueError(str(e)))

    def compute_memory_requirement(self, *args, **kwargs):
        """`(seq_len, hidden, n_layers, n_kv_heads, head_dim, bytes_per_el=2)` -> dict in GiB for a layer stack; the
        reference's `(batch_size, seq_len, hidden_dim, num_heads)` -> bytes of ONE layer's q / k / v, ring buffers,
        output and log-sum-exp at 2 bytes per element (data_pipeline/trainer/distributed/context_parallel.py:615)."""
        if {"batch_size", "hidden_dim", "num_heads"} & set(kwargs) or (len(args) == 4 and not kwargs):
            names = ("batch_size", "seq_len", "hidden_dim", "num_heads")
            a = dict(zip(names, args), **kwargs)
            b, s, h, nh = (int(a[n]) for n in names)
            local = s // self.cp_degree
            per_tensor = b * local * h * 2
            return 3 * per_tensor + self.ring_buffer_count * 2 * per_tensor + per_tensor + b * nh * local * 4
        return self._memory_of_stack(*args, **kwargs)

    def _memory_of_stack(self, seq_len: int, hidden: int, n_layers: int, n_kv_heads: int, head_dim: int,
                         bytes_per_el: int = 2) -> dict:
        return estimate_memory_per_gpu(seq_len, self.cp_degree, hidden, n_layers, n_kv_heads, head_dim, bytes_per_el,
                                       self.use_activation_checkpointing)


class RingCommunicator:
    """Neighbour exchange of the ring: send to rank+1, receive from rank-1, as one batched call."""

    def __init__(self, group=None, *, cp_rank: int | None = None, cp_world_size: int | None = None, process_group=None,
                 device=None, k_shape=None, v_shape=None, dtype: torch.dtype | None = None):
        """`RingCommunicator(group)`; the reference's keyword form names the rank and size itself and the shapes of
        the k / v blocks (receive buffers are then allocated once and reused by `start_send_recv(k_local=, v_local=)`)
        (data_pipeline/trainer/distributed/context_parallel.py RingCommunicator)."""
        group = process_group if process_group is not None else group
        self.group = group
        on = dist.is_available() and dist.is_initialized()
        self.world = int(cp_world_size) if cp_world_size is not None else (dist.get_world_size(group) if on else 1)
        self.rank = int(cp_rank) if cp_rank is not None else (dist.get_rank(group) if on else 0)
        if self.world > 1 and not on:
            raise RuntimeError("a ring of more than one rank needs an initialised process group")
        self.bytes_sent = 0
        self._recv_kv = None
        if k_shape is not None and v_shape is not None:
            if tuple(k_shape) != tuple(v_shape):
                raise ValueError("k and v travel as one message: their shapes must match")
            self._recv_kv = [torch.empty((2, *k_shape), dtype=dtype or torch.float32, device=device or "cpu") for _ in range(2)]
            self._turn = 0

    def _global(self, r: int) -> int:
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    def start_send_recv(self, send: torch.Tensor | None = None, recv: torch.Tensor | None = None, *, k_local=None,
                        v_local=None):
        """`start_send_recv(send, recv)` -> handles.  `start_send_recv(k_local=, v_local=)` -> (k_recv, v_recv, handles):
        the blocks of the previous rank, valid once `wait_recv(handles)` returned; two receive buffers alternate, so
        the blocks of one step stay readable while the next step's transfer runs."""
        if k_local is not None or v_local is not None:
            send = torch.stack((k_local, v_local))
            if self._recv_kv is not None and self._recv_kv[0].shape == send.shape and self._recv_kv[0].dtype == send.dtype:
                recv = self._recv_kv[self._turn]
                self._turn ^= 1
            else:
                recv = torch.empty_like(send)
            return recv[0], recv[1], self.start_send_recv(send, recv)
        if self.world == 1:
            recv.copy_(send)
            return []
        nxt, prv = self._global((self.rank + 1) % self.world), self._global((self.rank - 1) % self.world)
        ops = [dist.P2POp(dist.isend, send.contiguous(), nxt, self.group), dist.P2POp(dist.irecv, recv, prv, self.group)]
        self.bytes_sent += send.numel() * send.element_size()
        return dist.batch_isend_irecv(ops)

    @staticmethod
    @reference_kwargs(event="handles")
    def wait_recv(handles) -> None:
        for h in handles:
            h.wait()

    @contextlib.contextmanager
    def ring_step_context(self, k_local: torch.Tensor, v_local: torch.Tensor):
        """`with ring.ring_step_context(k, v) as (k_next, v_next):` - the exchange with the neighbours runs while the
        body computes on the CURRENT k / v; on exit the received blocks are complete.  k and v travel as one message."""
        send = torch.stack((k_local, v_local))
        recv = torch.empty_like(send)
        handles = self.start_send_recv(send, recv)
        try:
            yield recv[0], recv[1]
        finally:
            self.wait_recv(handles)


class ContextParallelEngine:
    """Shards a batch over the context-parallel group, runs exact causal ring attention on the shards (forward and
    backward through autograd), gathers outputs back into sequence order."""

    def __init__(self, config: ContextParallelConfig | None = None, group=None):
        self._config = config or ContextParallelConfig()
        self.group = group
        self._metrics = ContextParallelMetrics()
        self._initialized = False
        self._rank, self._world = 0, 1
        self.arena: TensorArena | None = None

    def initialize(self, group=None, device: torch.device | str = "cpu", *, cp_mesh=None):
        """`cp_mesh`: a one-dimensional DeviceMesh whose group is the context-parallel group."""
        from ..core.types import Err, Ok
        group = cp_mesh if cp_mesh is not None else group
        if group is not None and hasattr(group, "get_group"):
            group = group.get_group()
        self.group = group if group is not None else self.group
        on = dist.is_available() and dist.is_initialized()
        self._world = dist.get_world_size(self.group) if on else 1
        self._rank = dist.get_rank(self.group) if on else 0
        if self._world != self._config.cp_degree:
            return Err(ValueError(f"cp_degree {self._config.cp_degree} != group size {self._world}"))
        if self._config.use_arena_allocator:
            self.arena = TensorArena(int(self._config.arena_size_gb * 2 ** 30), device)
        self._initialized = True
        return Ok(self)

    config = property(lambda self: self._config)
    cp_rank = property(lambda self: self._rank)
    cp_world_size = property(lambda self: self._world)

    def _balancer(self) -> str:
        # without ring attention the engine exchanges token shards for head shards (Ulysses): contiguous token layout
        return self._config.load_balancer.name.lower() if self._config.use_ring_attention else "contiguous"

    def shard_inputs(self, input_ids: torch.Tensor, labels: torch.Tensor | None = None,
                     attention_mask: torch.Tensor | None = None, position_ids: torch.Tensor | None = None,
                     seq_dim: int = 1):
        """-> (input_ids, labels (already shifted), attention_mask, position_ids) of this rank."""
        assert seq_dim == 1, "sequences are dimension 1"
        batch = {"input_ids": input_ids}
        if labels is not None:
            batch["labels"] = labels
        if attention_mask is not None:
            batch["attention_mask"] = attention_mask
        if position_ids is not None:
            batch["position_ids"] = position_ids
        out = shard_inputs(batch, self._world, self._rank, self._balancer()) if self._world > 1 else \
            dict(batch, position_ids=position_ids if position_ids is not None else
                 torch.arange(input_ids.shape[1], device=input_ids.device).unsqueeze(0).expand_as(input_ids))
        return out["input_ids"], out.get("labels"), out.get("attention_mask"), out["position_ids"]

    def ring_attention_forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                               attention_mask: torch.Tensor | None = None) -> torch.Tensor:
        """q [1, S_local, Hq, D], k / v [1, S_local, Hkv, D] (rotary already applied with global positions)."""
        if attention_mask is not None:
            raise ValueError("padding masks are not supported by the ring path: pack the sequences instead")
        self._metrics.steps += 1
        if self._world == 1:
            from ..ops.attention import attention_reference
            return attention_reference(q, k, v, causal=True).to(q.dtype)
        S, Hq, D = q.shape[1], q.shape[2], q.shape[3]
        self._metrics.flops += 4.0 * (S * self._world) * (S * self._world) * Hq * D / 2 / self._world
        if not self._config.use_ring_attention:
            self._metrics.bytes_sent += (2 * q.numel() + 2 * k.numel()) * q.element_size() * (self._world - 1) // self._world
            return ulysses_attention(q, k, v, self.group)
        self._metrics.bytes_sent += 2 * k.numel() * k.element_size() * (self._world - 1)
        return ring_attention(q, k, v, self.group)

    @reference_kwargs(sharded_output="x_local")
    def gather_output(self, x_local: torch.Tensor, seq_dim: int = 1) -> torch.Tensor:
        if self._world == 1:
            return x_local
        return gather_output(x_local, self.group, self._balancer(), seq_dim)

    def get_metrics(self) -> ContextParallelMetrics:
        return self._metrics

    def reset_metrics(self) -> None:
        self._metrics = ContextParallelMetrics()


class ContextParallelAttention(nn.Module):
    """Attention core for modules that produce q / k / v themselves: ring attention when the engine spans more than one
    rank, plain causal attention otherwise."""

    def __init__(self, engine: "ContextParallelEngine | ContextParallelConfig | None" = None, *rest, config=None,
                 hidden_dim: int | None = None, num_heads: int | None = None, head_dim: int | None = None):
        """`ContextParallelAttention(engine)`: q / k / v arrive as [B, S_local, heads, D].  The reference's
        `(config, engine, hidden_dim, num_heads, head_dim=None)` names the head split, and q / k / v then arrive as
        [B, S_local, hidden] or [B, heads, S_local, D] and the output has the input's shape
        (data_pipeline/trainer/distributed/context_parallel.py:1965)."""
        super().__init__()
        if isinstance(engine, ContextParallelConfig) or (engine is None and rest):
            config, engine, rest = engine, (rest[0] if rest else None), rest[1:]
        if rest:
            given = dict(zip(("hidden_dim", "num_heads", "head_dim"), rest))
            hidden_dim, num_heads = given.get("hidden_dim", hidden_dim), given.get("num_heads", num_heads)
            head_dim = given.get("head_dim", head_dim)
        if engine is None:
            raise TypeError("an initialised ContextParallelEngine is required")
        self.engine = engine
        self.config = config if config is not None else engine.config
        self.hidden_dim, self.num_heads = hidden_dim, num_heads
        self.head_dim = head_dim or (hidden_dim // num_heads if hidden_dim and num_heads else None)
        self.scale = 1.0 / math.sqrt(self.head_dim) if self.head_dim else None

    def forward(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                attention_mask: torch.Tensor | None = None, position_ids: torch.Tensor | None = None) -> torch.Tensor:
        if self.num_heads is None:
            return self.engine.ring_attention_forward(query, key, value, attention_mask)
        if query.dim() == 3:                                # [B, S, hidden] -> [B, S, heads, D] and back
            B, S, _ = query.shape
            split = lambda t: t.view(B, S, -1, self.head_dim)            # noqa: E731
            out = self.engine.ring_attention_forward(split(query), split(key), split(value), attention_mask)
            return out.reshape(B, S, -1)
        out = self.engine.ring_attention_forward(query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2),
                                                 attention_mask)
        return out.transpose(1, 2)


def create_context_parallel_engine(cp_degree: int = 1, load_balancer: str = "head_tail", use_ring_attention: bool = True,
                                   use_triton: bool = False, group=None, **kwargs):
    """-> Result[ContextParallelEngine]: configuration errors and a group of the wrong size come back as Err."""
    from ..core.types import Err
    r = ContextParallelConfig.from_dict(dict(kwargs, cp_degree=cp_degree, load_balancer=load_balancer,
                                             use_ring_attention=use_ring_attention))
    if r.is_err():
        return r
    return ContextParallelEngine(r.unwrap(), group).initialize(group)


class ContextParallel:
    """Two-call convenience wrapper: `shard_inputs(batch)` before the model, `restore_sequence(x)` after it."""

    def __init__(self, group=None, load_balancer: str = "head_tail", *, config=None):
        """`ContextParallel(group, load_balancer)`, or the reference's `ContextParallel(config)` with a
        `ContextParallelConfig` or a dict of its fields: the wrapper then drives a `ContextParallelEngine`, initialised
        by the first `shard_inputs` (data_pipeline/trainer/distributed/context_parallel.py:2147)."""
        if isinstance(group, (ContextParallelConfig, dict)):
            config, group = group, None
        self._engine = None
        if config is not None:
            config = ContextParallelConfig(**config) if isinstance(config, dict) else config
            self._config, self._engine, self._initialized = config, ContextParallelEngine(config), False
            load_balancer = config.load_balancer.name.lower()
        self.group, self.load_balancer = group, load_balancer
        on = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if on else 1
        self.rank = dist.get_rank(group) if on else 0

    def shard_inputs(self, batch: "dict | torch.Tensor | None" = None, labels=None, attention_mask=None, position_ids=None,
                     cp_mesh=None, seq_dim: int = 1, *, input_ids=None):
        """`shard_inputs(batch dict)` -> dict; `shard_inputs(input_ids, labels, attention_mask, position_ids, cp_mesh,
        seq_dim)` -> the tuple of this rank's shards."""
        if isinstance(batch, dict):
            return shard_inputs(batch, self.world, self.rank, self.load_balancer) if self.world > 1 else batch
        input_ids = input_ids if input_ids is not None else batch
        eng = self._engine
        if eng is None:
            eng = self._engine = ContextParallelEngine(ContextParallelConfig(cp_degree=self.world,
                                                                             load_balancer=self.load_balancer), self.group)
            self._initialized = False
        if not self._initialized:
            r = eng.initialize(cp_mesh if cp_mesh is not None else self.group, input_ids.device)
            r.unwrap()                                       # raises the engine's error (group of the wrong size, ...)
            self._initialized = True
            self.group, self.world, self.rank = eng.group, eng.cp_world_size, eng.cp_rank
        return eng.shard_inputs(input_ids, labels, attention_mask, position_ids, seq_dim)

    @reference_kwargs(sharded_output="x_local", seq_dim="dim")
    def restore_sequence(self, x_local: torch.Tensor, dim: int = 1) -> torch.Tensor:
        return gather_output(x_local, self.group, self.load_balancer, dim) if self.world > 1 else x_local


# ------------------------------------------------------------------------------------------------ Ulysses (head <-> sequence all-to-all)
def _seq_to_heads(x: torch.Tensor, group, P: int) -> torch.Tensor:
    """[B, S/P, H, D] on every rank -> [B, S, H/P, D]: rank r ends with head group r of the whole sequence."""
    from .ep import _AllToAll
    B, Sl, H, D = x.shape
    send = x.view(B, Sl, P, H // P, D).permute(2, 0, 1, 3, 4).contiguous().view(P * B * Sl, (H // P) * D)
    recv = _AllToAll.apply(send, [B * Sl] * P, [B * Sl] * P, group)            # leading index = source rank = chunk
    return recv.view(P, B, Sl, H // P, D).permute(1, 0, 2, 3, 4).reshape(B, P * Sl, H // P, D)


def _heads_to_seq(x: torch.Tensor, group, P: int) -> torch.Tensor:
    """Inverse of `_seq_to_heads`: [B, S, H/P, D] -> [B, S/P, H, D]."""
    from .ep import _AllToAll
    B, S, Hl, D = x.shape
    Sl = S // P
    send = x.view(B, P, Sl, Hl, D).permute(1, 0, 2, 3, 4).contiguous().view(P * B * Sl, Hl * D)
    recv = _AllToAll.apply(send, [B * Sl] * P, [B * Sl] * P, group)            # leading index = source rank = head group
    return recv.view(P, B, Sl, Hl, D).permute(1, 2, 0, 3, 4).reshape(B, Sl, P * Hl, D)


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group, causal: bool = True,
                      scale: float | None = None, window: int | None = None, softcap: float = 0.0) -> torch.Tensor:
    """Sequence parallelism by all-to-all (DeepSpeed-Ulysses): the sequence is sharded CONTIGUOUSLY over the group
    (rank r holds tokens [r S/P, (r+1) S/P)), one all-to-all turns the token shards into head shards, every rank runs
    ordinary (flash) attention over the whole sequence for Hq/P query and Hkv/P key/value heads, a second all-to-all
    turns the result back.  Needs Hq and Hkv divisible by P; no causal load balancing is needed because every rank sees
    all tokens.  q [B, S/P, Hq, D], k / v [B, S/P, Hkv, D] -> [B, S/P, Hq, D].  The reference has no such path."""
    from ..ops import attention as A
    P = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    if P == 1:
        B, S, Hq, D = q.shape
        qkv = torch.cat((q.reshape(B, S, -1), k.reshape(B, S, -1), v.reshape(B, S, -1)), -1)
        return A.attention_qkv(qkv, Hq, k.shape[2], D, causal, scale, window, softcap).view(B, S, Hq, D)
    Hq, Hkv, D = q.shape[2], k.shape[2], q.shape[3]
    if Hq % P or Hkv % P:
        raise ValueError(f"Ulysses needs the head counts ({Hq}, {Hkv}) to divide by the group size {P}")
    qh, kh, vh = _seq_to_heads(q, group, P), _seq_to_heads(k, group, P), _seq_to_heads(v, group, P)
    B, S = qh.shape[0], qh.shape[1]
    qkv = torch.cat((qh.reshape(B, S, -1), kh.reshape(B, S, -1), vh.reshape(B, S, -1)), -1)
    o = A.attention_qkv(qkv, Hq // P, Hkv // P, D, causal, scale, window, softcap).view(B, S, Hq // P, D)
    return _heads_to_seq(o, group, P)


class LoadBalancerStrategy:
    """Interface of a sequence partitioner for context parallelism (data_pipeline/trainer/distributed/
    context_parallel.py:980): `partition(tensor, cp_rank, cp_world_size, seq_dim)` returns the rank's part and
    `unpartition(parts, seq_dim)` restores the order.  `BalancerStrategy(name)` adapts the balancers of this module."""

    def partition(self, tensor: torch.Tensor, cp_rank: int, cp_world_size: int, seq_dim: int) -> torch.Tensor:
        raise NotImplementedError

    def unpartition(self, parts: list[torch.Tensor], seq_dim: int) -> torch.Tensor:
        raise NotImplementedError

    def gather(self, shards: list[torch.Tensor], cp_world_size: int | None = None, seq_dim: int = 1) -> torch.Tensor:
        return self.unpartition(list(shards), seq_dim)

    def compute_global_positions(self, local_len: int, cp_rank: int, cp_world_size: int,
                                 total_len: int | None = None) -> torch.Tensor:
        """Derived from `partition` applied to the positions 0 .. total-1 themselves."""
        total = total_len if total_len is not None else local_len * cp_world_size
        return self.partition(torch.arange(total).unsqueeze(0), cp_rank, cp_world_size, 1).squeeze(0)


class BalancerStrategy(LoadBalancerStrategy):
    def __init__(self, name: str = "head_tail"):
        self.name = name

    def partition(self, tensor, cp_rank, cp_world_size, seq_dim):
        return create_balancer(self.name, cp_world_size, cp_rank).shard(tensor, seq_dim)

    def unpartition(self, parts, seq_dim):
        return create_balancer(self.name, len(parts), 0).unshard(parts, seq_dim)


# ---- type aliases of data_pipeline/trainer/distributed/hybrid_cp_scheduler.py
SampleSeqLen = tuple[int, int]             # (sample id, sequence length)
MicroBatch = list[int]                     # sequence lengths one GPU processes
SampleIdList = list[int]
