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

import torch
import torch.distributed as dist

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


def create_balancer(name: str, cp: int, rank: int):
    name = (name or "head_tail").lower()
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


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group, scale: float | None = None) -> torch.Tensor:
    """Causal attention over a sequence sharded with the head-tail layout. q [B=1, S_local, Hq, D]; returns the same
    shape. Local rows are (chunk rank | chunk 2cp-1-rank)."""
    B, S, Hq, D = q.shape
    assert B == 1, "ring attention handles one (packed) sequence per step"
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
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


def estimate_memory_per_gpu(seq_len: int, cp: int, hidden: int, n_layers: int, n_kv_heads: int, head_dim: int,
                            bytes_per_el: int = 2, checkpointing: bool = True) -> dict:
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

    def __init__(self, cfg: HybridCPConfig):
        self.cfg = cfg

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
