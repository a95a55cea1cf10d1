"""Mixture-of-experts layers and expert parallelism.

Feature set after data_pipeline/trainer/distributed/expert_parallel.py:83-1976 (TopK / ExpertChoice / SoftMoE
routers, ExpertFFN, GroupedExperts, SharedExpert, MoELayer, all-to-all dispatcher, ExpertParallelMoE, HierarchicalMoE;
capacity = max(min_cap, cf * T * k / E), aux losses E * sum f_i P_i, z-loss, importance CV^2) and the MoE kernels of
data_pipeline/trainer/kernels/moe_kernels.py:219-785 (token permute / un-permute, grouped GEMM, router top-k softmax).
The distributed combine here returns the expert outputs to their source ranks (the reference's returns zeros).

Token movement: tokens are sorted by expert once (permute), each expert's contiguous slice runs the tcgen05 GEMMs
(one launch per expert per projection), and the un-permute applies the routing weights.  Across ranks the sorted
slices are exchanged with `all_to_all_single` using exact (not capacity-padded) split sizes.
"""
from __future__ import annotations

import contextlib

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..ops import activation, gemm
from ..utils.refargs import reference_kwargs


@dataclass
class ExpertParallelConfig:
    num_experts: int = 8
    top_k: int = 2
    hidden_size: int = 256
    intermediate_size: int = 512
    capacity_factor: float = 1.25
    min_capacity: int = 4
    drop_tokens: bool = False
    router: str = "top_k"              # top_k | expert_choice | soft
    aux_loss_weight: float = 1e-2
    z_loss_weight: float = 1e-3
    num_shared_experts: int = 0
    normalize_topk: bool = True
    jitter: float = 0.0
    expert_parallel_group: object = None   # process group the experts are spread over (None: the default group)
    use_fp32_router: bool = True

    @property
    def num_local_experts(self) -> int:
        """Experts held by each rank of the expert-parallel group."""
        w = get_expert_parallel_world_size(self.expert_parallel_group)
        if self.num_experts % w:
            raise ValueError(f"num_experts ({self.num_experts}) must be divisible by the group size ({w})")
        return self.num_experts // w

    @property
    def local_expert_offset(self) -> int:
        """Global index of this rank's first expert."""
        return get_expert_parallel_rank(self.expert_parallel_group) * self.num_local_experts


def moe_capacity(tokens: int, num_experts: int, top_k: int, capacity_factor: float, min_capacity: int = 4) -> int:
    return max(min_capacity, int(math.ceil(capacity_factor * tokens * top_k / num_experts)))


# ------------------------------------------------------------------------------------------------ routers
def _dense_routing(cfg, logits, w, idx, aux_loss, padding_mask=None, meta=None):
    """A top-k decision (weights / experts [T, k], logits [T, E]) as the dense capacity-slotted `RoutingOutput`: slot of
    a (token, choice) inside its expert = number of earlier slots routed to the same expert; slots past the capacity
    are dropped; padded tokens (`padding_mask` True) are routed nowhere."""
    T, E = logits.shape
    k = idx.shape[1]
    C = moe_capacity(T, E, k, cfg.capacity_factor, cfg.min_capacity)
    live = torch.ones(T, dtype=torch.bool, device=logits.device) if padding_mask is None \
        else ~padding_mask.reshape(-1).to(torch.bool)
    hot = F.one_hot(idx.reshape(-1), E) * live.repeat_interleave(k)[:, None]        # [T*k, E]
    slot = (hot.cumsum(0) - hot).gather(1, idx.reshape(-1, 1)).reshape(T, k)
    keep = (slot < C) & live[:, None]
    w = w * live[:, None].to(w.dtype)
    dispatch = torch.zeros(T, E, C, dtype=torch.bool, device=logits.device)
    combine = torch.zeros(T, E, C, dtype=w.dtype, device=logits.device)
    t = torch.arange(T, device=logits.device)[:, None].expand_as(idx)
    dispatch[t[keep], idx[keep], slot[keep]] = True
    combine[t[keep], idx[keep], slot[keep]] = w[keep]
    info = {"capacity": C, "dropped": int((~keep & live[:, None]).sum()), "tokens_per_expert": hot.sum(0)}
    info.update(meta or {})
    return RoutingOutput(dispatch, combine, idx, w, logits, aux_loss, info)


def _aux_total(cfg, aux: dict):
    total = 0.0
    if "load_balance" in aux:
        total = total + cfg.aux_loss_weight * aux["load_balance"]
    if "z_loss" in aux:
        total = total + cfg.z_loss_weight * aux["z_loss"]
    return total if torch.is_tensor(total) else torch.zeros(())


class TopKRouter(nn.Module):
    """`router(x [T, H])` -> (weights, experts, aux dict); `router(hidden_states=[B, S, H], padding_mask=[B, S])` ->
    the dense `RoutingOutput` (data_pipeline/trainer/distributed/expert_parallel.py:653)."""

    @reference_kwargs(config="cfg")
    def __init__(self, cfg: ExpertParallelConfig, dtype=None, device=None):
        super().__init__()
        self.cfg = cfg
        self.weight = nn.Parameter(torch.empty(cfg.num_experts, cfg.hidden_size, dtype=dtype, device=device))
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, x: torch.Tensor | None = None, *, hidden_states=None, padding_mask=None):
        """x [T, H] -> (weights [T, k], experts [T, k], aux dict)."""
        if hidden_states is not None:
            flat = hidden_states.reshape(-1, hidden_states.shape[-1])
            w, idx, aux = self.forward(flat)
            logits = F.linear(flat.float(), self.weight.float())
            return _dense_routing(self.cfg, logits, w, idx, _aux_total(self.cfg, aux), padding_mask,
                                  {"importance_cv2": aux["importance_cv2"]})
        cfg = self.cfg
        logits = F.linear(x.float(), self.weight.float())
        if self.training and cfg.jitter > 0:
            logits = logits * torch.empty_like(logits).uniform_(1 - cfg.jitter, 1 + cfg.jitter)
        from ..ops import moe as moe_ops
        w, idx, probs = moe_ops.topk_softmax(logits, cfg.top_k, cfg.normalize_topk)   # device kernel on CUDA
        f = F.one_hot(idx, cfg.num_experts).float().sum(1).mean(0) / cfg.top_k
        P = probs.mean(0)
        aux = {"load_balance": cfg.num_experts * (f * P).sum(), "z_loss": (torch.logsumexp(logits, -1) ** 2).mean(),
               "importance_cv2": probs.sum(0).var() / probs.sum(0).mean().clamp(min=1e-9) ** 2,
               "tokens_per_expert": F.one_hot(idx, cfg.num_experts).sum((0, 1))}
        return w.to(x.dtype), idx, aux


class ExpertChoiceRouter(nn.Module):
    """Each expert picks its top-`capacity` tokens (perfect balance, tokens may get 0..E experts)."""

    @reference_kwargs(config="cfg")
    def __init__(self, cfg: ExpertParallelConfig, dtype=None, device=None):
        super().__init__()
        self.cfg = cfg
        self.weight = nn.Parameter(torch.empty(cfg.num_experts, cfg.hidden_size, dtype=dtype, device=device))
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, x=None, *, hidden_states=None, padding_mask=None):
        """x [T, H] -> (weights [E, cap], tokens [E, cap], aux).  `forward(hidden_states=, padding_mask=)` gives the
        dense `RoutingOutput` instead: slot c of expert e holds its c-th chosen token
        (data_pipeline/trainer/distributed/expert_parallel.py:903)."""
        if hidden_states is not None:
            flat = hidden_states.reshape(-1, hidden_states.shape[-1])
            logits = F.linear(flat.float(), self.weight.float())
            if padding_mask is not None:
                logits = logits.masked_fill(padding_mask.reshape(-1, 1).to(torch.bool), float("-inf"))
            probs = torch.softmax(logits, dim=-1).nan_to_num(0.0)
            T, E = probs.shape
            cap = min(T, moe_capacity(T, E, self.cfg.top_k, self.cfg.capacity_factor, self.cfg.min_capacity))
            w, tok = probs.t().topk(cap, dim=-1)                                      # [E, cap]
            dispatch = torch.zeros(T, E, cap, dtype=torch.bool, device=flat.device)
            combine = torch.zeros(T, E, cap, dtype=w.dtype, device=flat.device)
            e = torch.arange(E, device=flat.device)[:, None].expand_as(tok)
            c = torch.arange(cap, device=flat.device)[None, :].expand_as(tok)
            live = w > 0
            dispatch[tok[live], e[live], c[live]] = True
            combine[tok[live], e[live], c[live]] = w[live]
            k = min(self.cfg.top_k, E)
            tw, ti = combine.sum(-1).topk(k, dim=-1)
            return RoutingOutput(dispatch, combine, ti, tw.to(hidden_states.dtype), logits, logits.new_zeros(()),
                                 {"capacity": cap, "tokens_per_expert": dispatch.sum((0, 2))})
        cfg = self.cfg
        T = x.shape[0]
        probs = torch.softmax(F.linear(x.float(), self.weight.float()), dim=-1)     # [T, E]
        cap = min(T, moe_capacity(T, cfg.num_experts, cfg.top_k, cfg.capacity_factor, cfg.min_capacity))
        w, tok = probs.t().topk(cap, dim=-1)                                          # [E, cap]
        return w.to(x.dtype), tok, {"capacity": cap}


class SoftMoERouter(nn.Module):
    """Soft MoE: every slot is a convex combination of all tokens (fully differentiable, no dropping)."""

    @reference_kwargs(config="cfg")
    def __init__(self, cfg: ExpertParallelConfig, slots_per_expert: int = 1, dtype=None, device=None):
        super().__init__()
        self.cfg, self.slots = cfg, slots_per_expert
        self.phi = nn.Parameter(torch.empty(cfg.hidden_size, cfg.num_experts * slots_per_expert, dtype=dtype, device=device))
        nn.init.normal_(self.phi, std=0.02)

    def forward(self, x=None, *, hidden_states=None, padding_mask=None):
        """x [T, H] -> (dispatch [T, E*slots], combine [T, E*slots], {}).  `forward(hidden_states=, padding_mask=)`
        returns them as a `RoutingOutput` whose masks are the soft weights [T, E, slots]: padded tokens get no share of
        a slot (data_pipeline/trainer/distributed/expert_parallel.py:1046)."""
        if hidden_states is not None:
            flat = hidden_states.reshape(-1, hidden_states.shape[-1])
            logits = flat.float() @ self.phi.float()
            T, E = flat.shape[0], self.cfg.num_experts
            dl = logits if padding_mask is None else logits.masked_fill(padding_mask.reshape(-1, 1).to(torch.bool), float("-inf"))
            dispatch = torch.softmax(dl, dim=0).nan_to_num(0.0).view(T, E, self.slots)
            combine = torch.softmax(logits, dim=1).view(T, E, self.slots)
            if padding_mask is not None:
                combine = combine * (~padding_mask.reshape(-1).to(torch.bool))[:, None, None]
            per_expert = combine.sum(-1)
            k = min(self.cfg.top_k, E)
            tw, ti = per_expert.topk(k, dim=-1)
            return RoutingOutput(dispatch, combine, ti, tw, logits.view(T, E, self.slots).mean(-1), logits.new_zeros(()),
                                 {"slots_per_expert": self.slots})
        logits = x.float() @ self.phi.float()                  # [T, E*slots]
        dispatch = torch.softmax(logits, dim=0)                # over tokens
        combine = torch.softmax(logits, dim=1)                 # over slots
        return dispatch.to(x.dtype), combine.to(x.dtype), {}


# ------------------------------------------------------------------------------------------------ experts
_PLAIN_ACT = {"silu": F.silu, "swish": F.silu, "gelu": F.gelu, "relu": F.relu,
              "gelu_tanh": lambda v: F.gelu(v, approximate="tanh"), "gelu_new": lambda v: F.gelu(v, approximate="tanh")}
_GLU_ACT = {"silu": "silu", "swish": "silu", "gelu": "gelu", "gelu_tanh": "gelu_tanh", "gelu_new": "gelu_tanh"}


def _ffn(x, w_up, w_down, act: str, gated: bool):
    """One feed-forward block: act(gate) * up (gated; gate | up stacked in `w_up`) or act(up), then the down projection.
    The gated silu / gelu forms run the fused GLU kernel; relu and the ungated forms are plain PyTorch."""
    h = gemm.linear(x, w_up)
    if gated and act in _GLU_ACT:
        h = activation.glu(h, _GLU_ACT[act])
    elif gated:
        g, u = h.chunk(2, dim=-1)
        h = _PLAIN_ACT[act](g) * u
    else:
        h = _PLAIN_ACT[act](h)
    return gemm.linear(h, w_down)


def _expert_options(rest, activation, dropout, use_gated, dtype, device):
    """The positional tail of an expert's constructor: `(dtype, device)`, or the reference's `(activation, dropout,
    use_gated)` when it starts with the activation's name."""
    if rest and isinstance(rest[0], str):
        if len(rest) > 3:
            raise TypeError("at most (activation, dropout, use_gated) after the sizes")
        activation = rest[0]
        dropout = float(rest[1]) if len(rest) > 1 else dropout
        use_gated = bool(rest[2]) if len(rest) > 2 else use_gated
    elif rest:
        if len(rest) > 2:
            raise TypeError("at most (dtype, device) after the sizes")
        dtype = rest[0]
        device = rest[1] if len(rest) > 1 else device
    return activation, dropout, use_gated, dtype, device


class ExpertFFN(nn.Module):
    """One expert: `down(act(gate(x)) * up(x))`, or `down(act(up(x)))` with `use_gated=False`
    (data_pipeline/trainer/distributed/expert_parallel.py:1126)."""

    @reference_kwargs(hidden_size="hidden", intermediate_size="inter")
    def __init__(self, hidden: int, inter: int, *rest, dtype=None, device=None, activation: str = "silu",
                 dropout: float = 0.0, use_gated: bool = True):
        super().__init__()
        activation, dropout, use_gated, dtype, device = _expert_options(rest, activation, dropout, use_gated, dtype, device)
        if activation not in _PLAIN_ACT:
            raise ValueError(f"unknown activation {activation!r}; one of {sorted(_PLAIN_ACT)}")
        self.act, self.use_gated = activation, bool(use_gated)
        self.w_gate_up = nn.Parameter(torch.empty((2 if use_gated else 1) * inter, hidden, dtype=dtype, device=device))
        self.w_down = nn.Parameter(torch.empty(hidden, inter, dtype=dtype, device=device))
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()
        nn.init.normal_(self.w_gate_up, std=0.02)
        nn.init.normal_(self.w_down, std=0.02)

    def forward(self, x):
        return self.dropout(_ffn(x, self.w_gate_up, self.w_down, self.act, self.use_gated))


class GroupedExperts(nn.Module):
    """E experts stored as stacked weights; `forward(x_sorted, counts)` runs each expert on its contiguous slice."""

    @reference_kwargs(hidden_size="hidden", intermediate_size="inter")
    def __init__(self, num_experts: int, hidden: int, inter: int, *rest, dtype=None, device=None,
                 activation: str = "silu", dropout: float = 0.0, use_gated: bool = True):
        super().__init__()
        activation, dropout, use_gated, dtype, device = _expert_options(rest, activation, dropout, use_gated, dtype, device)
        if activation not in _PLAIN_ACT:
            raise ValueError(f"unknown activation {activation!r}; one of {sorted(_PLAIN_ACT)}")
        self.num_experts, self.act, self.use_gated = num_experts, activation, bool(use_gated)
        self.w_gate_up = nn.Parameter(torch.empty(num_experts, (2 if use_gated else 1) * inter, hidden, dtype=dtype, device=device))
        self.w_down = nn.Parameter(torch.empty(num_experts, hidden, inter, dtype=dtype, device=device))
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()
        nn.init.normal_(self.w_gate_up, std=0.02)
        nn.init.normal_(self.w_down, std=0.02)

    def forward(self, x_sorted: torch.Tensor | None = None, counts: "list[int] | None" = None, expert_weights=None, *,
                tokens=None, expert_indices=None) -> torch.Tensor:
        """`forward(x_sorted, counts)`: rows already grouped by expert.  `forward(tokens, expert_indices, expert_weights)`
        (tokens [T, H], choices and weights [T, k]) groups them, runs the experts and returns the weighted sum per token
        (data_pipeline/trainer/distributed/expert_parallel.py:1267)."""
        if tokens is not None or torch.is_tensor(counts) or expert_indices is not None:
            x = tokens if tokens is not None else x_sorted
            idx = expert_indices if expert_indices is not None else counts
            if expert_weights is None:
                raise TypeError("forward(tokens, expert_indices, expert_weights) needs the routing weights")
            xs, order, cnt = permute_tokens(x, idx, self.num_experts)
            return unpermute_tokens(self.forward(xs, cnt.tolist()), order, expert_weights.to(x.dtype), x.shape[0])
        outs, off = [], 0
        for e, n in enumerate(counts):
            if n == 0:
                continue
            xe = x_sorted[off:off + n]
            outs.append(self.dropout(_ffn(xe, self.w_gate_up[e], self.w_down[e], self.act, self.use_gated)))
            off += n
        if not outs:
            return x_sorted.new_zeros(0, x_sorted.shape[-1])
        return torch.cat(outs)


class SharedExpert(ExpertFFN):
    """Expert every token passes through, next to the routed ones."""

    @property
    def ffn(self) -> "SharedExpert":
        return self


def permute_tokens(x: torch.Tensor, experts: torch.Tensor, num_experts: int):
    """x [T, H], experts [T, k] -> (x_sorted [T*k, H], order [T*k], counts [E]); row i of x_sorted is token order[i] // k."""
    flat = experts.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts)
    return x[order // experts.shape[1]], order, counts


def unpermute_tokens(y_sorted: torch.Tensor, order: torch.Tensor, weights: torch.Tensor, T: int) -> torch.Tensor:
    """Weighted scatter-add of expert outputs back to token order."""
    k = weights.shape[1]
    w = weights.reshape(-1)[order].unsqueeze(-1)
    out = y_sorted.new_zeros(T, y_sorted.shape[-1], dtype=torch.float32)
    out.index_add_(0, order // k, (y_sorted * w).float())
    return out.to(y_sorted.dtype)


class MoELayer(nn.Module):
    """Single-process MoE block (all experts local)."""

    @reference_kwargs(config="cfg")
    def __init__(self, cfg: ExpertParallelConfig, dtype=None, device=None):
        super().__init__()
        self.cfg = cfg
        self.router = {"top_k": TopKRouter, "expert_choice": ExpertChoiceRouter}.get(cfg.router, TopKRouter)(cfg, dtype, device) \
            if cfg.router != "soft" else SoftMoERouter(cfg, 1, dtype, device)
        self.experts = GroupedExperts(cfg.num_experts, cfg.hidden_size, cfg.intermediate_size, dtype, device)
        self.shared = nn.ModuleList(SharedExpert(cfg.hidden_size, cfg.intermediate_size, dtype, device)
                                    for _ in range(cfg.num_shared_experts))
        self.aux_loss = torch.zeros(())

    def _aux(self, aux: dict) -> torch.Tensor:
        cfg = self.cfg
        loss = 0.0
        if "load_balance" in aux:
            loss = loss + cfg.aux_loss_weight * aux["load_balance"]
        if "z_loss" in aux:
            loss = loss + cfg.z_loss_weight * aux["z_loss"]
        return loss

    def route_and_run(self, x2: torch.Tensor, run_experts) -> torch.Tensor:
        cfg = self.cfg
        T = x2.shape[0]
        if cfg.router == "soft":
            dispatch, combine, aux = self.router(x2)
            slots = dispatch.t() @ x2                                        # [E, H] (one slot per expert)
            y = run_experts(slots, torch.arange(cfg.num_experts, device=x2.device).unsqueeze(1),
                            torch.ones(cfg.num_experts, 1, device=x2.device, dtype=x2.dtype))
            self.aux_loss = x2.new_zeros(())
            return combine @ y
        if cfg.router == "expert_choice":
            w, tok, aux = self.router(x2)                                    # [E, cap]
            E, cap = tok.shape
            xs = x2[tok.reshape(-1)]
            ys = self.experts(xs, [cap] * E)
            out = x2.new_zeros(T, x2.shape[-1], dtype=torch.float32)
            out.index_add_(0, tok.reshape(-1), (ys * w.reshape(-1, 1)).float())
            self.aux_loss = x2.new_zeros(())
            return out.to(x2.dtype)
        w, idx, aux = self.router(x2)
        if cfg.drop_tokens:
            cap = moe_capacity(T, cfg.num_experts, cfg.top_k, cfg.capacity_factor, cfg.min_capacity)
            pos = torch.zeros_like(idx)
            flat = idx.reshape(-1)
            onehot = F.one_hot(flat, cfg.num_experts)
            rank_in_expert = (onehot.cumsum(0) - 1).gather(1, flat.unsqueeze(1)).squeeze(1)
            keep = (rank_in_expert < cap).view_as(idx)
            w = w * keep
        self.aux_loss = self._aux(aux)
        return run_experts(x2, idx, w)

    def _local(self, x2, idx, w):
        from ..ops import moe as moe_ops
        if moe_ops.available(x2) and isinstance(self.experts, GroupedExperts) \
                and self.experts.use_gated and self.experts.act == "silu" and isinstance(self.experts.dropout, nn.Identity) \
                and self.experts.w_gate_up.dtype == torch.bfloat16 and self.experts.w_down.shape[-1] % 64 == 0 \
                and x2.shape[-1] % 64 == 0:
            # device-side plan + one grouped tcgen05 GEMM per projection: no host sync on the expert counts
            return moe_ops.moe_ffn(x2, idx, w, self.experts.w_gate_up, self.experts.w_down)
        xs, order, counts = permute_tokens(x2, idx, self.cfg.num_experts)
        ys = self.experts(xs, counts.tolist())
        return unpermute_tokens(ys, order, w, x2.shape[0])

    def _masked(self, run, x2, attention_mask):
        """`run` on the valid rows only (`attention_mask` 1 = valid); padded rows come out as zeros and take no part in
        the routing statistics."""
        if attention_mask is None:
            return self.route_and_run(x2, run)
        valid = attention_mask.reshape(-1).to(torch.bool)
        out = torch.zeros_like(x2)
        if valid.any():
            out[valid] = self.route_and_run(x2[valid], run)
        return out

    def _reference_forward(self, run, hidden_states, attention_mask, output_router_logits):
        shp = hidden_states.shape
        x2 = hidden_states.reshape(-1, shp[-1])
        y = self._masked(run, x2, attention_mask)
        for s in self.shared:
            y = y + s(x2)
        logits = None
        if output_router_logits:
            w = getattr(self.router, "weight", None)
            logits = F.linear(x2.float(), w.float()) if w is not None else x2.float() @ self.router.phi.float()
        aux = self.aux_loss if torch.is_tensor(self.aux_loss) else x2.new_zeros(())
        return y.view(shp), aux, logits

    def forward(self, x: torch.Tensor | None = None, *, hidden_states=None, attention_mask=None,
                output_router_logits: bool = False):
        """`layer(x)` -> output (the auxiliary loss is left in `aux_loss`).  `layer(hidden_states=, attention_mask=,
        output_router_logits=)` -> (output, auxiliary loss, router logits or None)
        (data_pipeline/trainer/distributed/expert_parallel.py:1480)."""
        if hidden_states is not None:
            return self._reference_forward(self._local, hidden_states, attention_mask, output_router_logits)
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        y = self.route_and_run(x2, self._local)
        for s in self.shared:
            y = y + s(x2)
        return y.view(shp)


# ------------------------------------------------------------------------------------------------ expert parallelism
class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, in_splits, out_splits, group):
        ctx.in_splits, ctx.out_splits, ctx.group = in_splits, out_splits, group
        out = x.new_empty(sum(out_splits), *x.shape[1:])
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty(sum(ctx.in_splits), *g.shape[1:])
        dist.all_to_all_single(out, g.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.group)
        return out, None, None, None


class AllToAllDispatcher:
    """Moves expert-sorted token rows to the ranks that own the experts, and back."""

    def __init__(self, *args, group=None, num_experts: int | None = None, num_local_experts: int | None = None,
                 capacity: int | None = None):
        """`AllToAllDispatcher(group, num_experts)`, or the reference's `(num_experts, num_local_experts, capacity,
        group)` (data_pipeline/trainer/distributed/expert_parallel.py:232); the capacity is only used by the
        mask form of `dispatch`."""
        if args and isinstance(args[0], int):                       # (num_experts, num_local_experts, capacity, group)
            names = ("num_experts", "num_local_experts", "capacity", "group")
        else:
            names = ("group", "num_experts")
        if len(args) > len(names):
            raise TypeError(f"at most {names} positionally")
        given = dict(zip(names, args))
        group = given.get("group", group)
        num_experts = given.get("num_experts", num_experts)
        num_local_experts = given.get("num_local_experts", num_local_experts)
        capacity = given.get("capacity", capacity)
        if num_experts is None:
            raise TypeError("num_experts is required")
        self.group = group
        self.world = get_expert_parallel_world_size(group)
        self.rank = get_expert_parallel_rank(group)
        assert num_experts % self.world == 0, "num_experts must divide by the expert-parallel size"
        self.num_experts, self.local_experts = num_experts, num_experts // self.world
        if num_local_experts is not None and int(num_local_experts) != self.local_experts:
            raise ValueError(f"num_local_experts={num_local_experts} but {num_experts} experts over {self.world} ranks "
                             f"give {self.local_experts}")
        self.capacity = capacity
        self._slots = None

    num_local_experts = property(lambda self: self.local_experts)
    world_size = property(lambda self: self.world)

    # ---- capacity-slotted form: dispatch(tokens, dispatch_mask [T, E]) / combine(expert_outputs, combine_weights, ...)
    def _dispatch_mask(self, tokens: torch.Tensor, mask: torch.Tensor):
        T, H = tokens.shape
        E, W, El = self.num_experts, self.world, self.local_experts
        mask = mask.to(torch.bool)
        C = int(self.capacity) if self.capacity is not None else max(int(mask.sum(0).max()), 1)
        slot = mask.long().cumsum(0) - 1                                   # [T, E] position of a token inside its expert
        keep = mask & (slot < C)
        t, e = keep.nonzero(as_tuple=True)
        send = tokens.new_zeros(E, C, H).index_put((e, slot[t, e]), tokens[t])
        counts = keep.sum(0)
        self._slots = (t, e, slot[t, e], C)
        if W == 1:
            self._order = None
            return send, counts
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts.contiguous(), group=self.group)       # [W, El] by source rank
        n = El * C
        recv = _AllToAll.apply(send.view(E * C, H), [n] * W, [n] * W, self.group).view(W, El, C, H)
        # per local expert: the valid rows of every source rank, in rank order, then the empty slots
        valid = torch.arange(C, device=tokens.device)[None, None, :] < recv_counts.view(W, El, 1)
        valid = valid.permute(1, 0, 2).reshape(El, W * C)
        order = torch.argsort((~valid).to(torch.uint8), dim=1, stable=True)
        rows = recv.permute(1, 0, 2, 3).reshape(El, W * C, H)
        self._order = order
        return rows.gather(1, order[..., None].expand(-1, -1, H)), recv_counts.view(W, El).sum(0)

    def _combine_mask(self, expert_outputs, combine_weights, original_positions=None, num_tokens=None):
        if self._slots is None:
            raise RuntimeError("combine(expert_outputs, combine_weights, ...) follows dispatch(tokens, dispatch_mask)")
        t, e, s, C = self._slots
        W, El, H = self.world, self.local_experts, expert_outputs.shape[-1]
        if W > 1:
            rows = torch.zeros_like(expert_outputs).scatter(1, self._order[..., None].expand(-1, -1, H), expert_outputs)
            rows = rows.view(El, W, C, H).permute(1, 0, 2, 3).reshape(W * El * C, H)
            n = El * C
            expert_outputs = _AllToAll.apply(rows, [n] * W, [n] * W, self.group).view(self.num_experts, C, H)
        if combine_weights.dim() == 3:                                      # [T, E, C] -> weight of the slot used
            wt = combine_weights[t, e, s]
        else:
            wt = combine_weights[t, e]
        T = int(num_tokens) if num_tokens is not None else combine_weights.shape[0]
        pos = t if original_positions is None else original_positions.to(t.device)[t]
        out = expert_outputs.new_zeros(T, H, dtype=torch.float32)
        out = out.index_add(0, pos, (expert_outputs[e, s] * wt[:, None].to(expert_outputs.dtype)).float())
        return out.to(expert_outputs.dtype)

    def dispatch(self, x_sorted: torch.Tensor | None = None, counts: torch.Tensor | None = None, *, tokens=None,
                 dispatch_mask=None):
        """counts [E] (tokens this rank routes to each global expert). Returns (rows for my experts ordered by
        (source rank, local expert), recv_counts [W, E_local], bookkeeping).

        `dispatch(tokens [T, H], dispatch_mask [T, E])` is the capacity-slotted form: returns (rows
        [E_local, W * capacity, H], valid rows per local expert); the rows of one expert are those of rank 0, rank 1, ...
        followed by zero rows."""
        if tokens is not None or dispatch_mask is not None or (counts is not None and counts.dim() == 2):
            return self._dispatch_mask(tokens if tokens is not None else x_sorted,
                                       dispatch_mask if dispatch_mask is not None else counts)
        W, El = self.world, self.local_experts
        send_counts = counts.view(W, El)
        if W == 1:                                       # every expert is local: nothing moves
            return x_sorted, send_counts, None
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts.contiguous(), group=self.group)
        in_splits = send_counts.sum(1).tolist()
        out_splits = recv_counts.sum(1).tolist()
        recv = _AllToAll.apply(x_sorted, in_splits, out_splits, self.group)
        return recv, recv_counts, (in_splits, out_splits)

    def combine(self, y: torch.Tensor | None = None, book=None, original_positions=None, num_tokens=None, *,
                expert_outputs=None, combine_weights=None) -> torch.Tensor:
        """`combine(y, book)` undoes `dispatch(x_sorted, counts)`.  `combine(expert_outputs, combine_weights [T, E] or
        [T, E, C], original_positions, num_tokens)` undoes the mask form and returns the weighted sum per token."""
        if expert_outputs is not None or combine_weights is not None or torch.is_tensor(book):
            return self._combine_mask(expert_outputs if expert_outputs is not None else y,
                                      combine_weights if combine_weights is not None else book,
                                      original_positions, num_tokens)
        if book is None:
            return y
        in_splits, out_splits = book
        return _AllToAll.apply(y, out_splits, in_splits, self.group)


class ExpertParallelMoE(MoELayer):
    """MoE block whose experts are sharded over an expert-parallel group (E / W local experts per rank)."""

    @reference_kwargs(config="cfg")
    def __init__(self, cfg: ExpertParallelConfig, group=None, dtype=None, device=None):
        nn.Module.__init__(self)
        self.cfg = cfg
        group = group if group is not None else getattr(cfg, "expert_parallel_group", None)
        self.router = TopKRouter(cfg, dtype, device)
        self.dispatcher = AllToAllDispatcher(group, cfg.num_experts)
        self.experts = GroupedExperts(self.dispatcher.local_experts, cfg.hidden_size, cfg.intermediate_size, dtype, device)
        self.shared = nn.ModuleList(SharedExpert(cfg.hidden_size, cfg.intermediate_size, dtype, device)
                                    for _ in range(cfg.num_shared_experts))
        self.aux_loss = torch.zeros(())

    def _distributed(self, x2, idx, w):
        d = self.dispatcher
        xs, order, counts = permute_tokens(x2, idx, self.cfg.num_experts)
        recv, recv_counts, book = d.dispatch(xs, counts)
        # received rows are ordered (source rank, local expert): regroup them by local expert
        W, El = d.world, d.local_experts
        rc = recv_counts.tolist()
        offs, o = [[0] * El for _ in range(W)], 0
        for r in range(W):
            for e in range(El):
                offs[r][e] = o
                o += rc[r][e]
        gather_idx = torch.cat([torch.arange(offs[r][e], offs[r][e] + rc[r][e], device=x2.device)
                                for e in range(El) for r in range(W)]) if o > 0 else torch.zeros(0, dtype=torch.long, device=x2.device)
        per_expert = [sum(rc[r][e] for r in range(W)) for e in range(El)]
        ye = self.experts(recv[gather_idx], per_expert)
        back = torch.empty_like(ye)
        back[gather_idx] = ye
        ys = d.combine(back, book)
        return unpermute_tokens(ys, order, w, x2.shape[0])

    moe_layer = property(lambda self: self)

    def forward(self, x=None, *, hidden_states=None, attention_mask=None, output_router_logits: bool = False):
        self.__dict__["_forward_count"] = self.__dict__.get("_forward_count", 0) + 1
        if hidden_states is not None:
            if attention_mask is not None and self.dispatcher.world > 1:
                # every rank must enter the all-to-all: route all rows, zero the padded ones afterwards
                out, aux, logits = self._reference_forward(self._distributed, hidden_states, None, output_router_logits)
                return out * attention_mask.reshape(*out.shape[:-1], 1).to(out.dtype), aux, logits
            return self._reference_forward(self._distributed, hidden_states, attention_mask, output_router_logits)
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        y = self.route_and_run(x2, self._distributed)
        for s in self.shared:
            y = y + s(x2)
        return y.view(shp)

    def get_routing_statistics(self) -> dict:
        return {"forward_count": self.__dict__.get("_forward_count", 0), "num_experts": self.cfg.num_experts,
                "num_local_experts": self.dispatcher.local_experts, "top_k": self.cfg.top_k,
                "aux_loss": float(self.aux_loss.detach()) if torch.is_tensor(self.aux_loss) else float(self.aux_loss)}


class HierarchicalMoE(nn.Module):
    """Two-level routing: a coarse router picks a group, the group's MoE picks experts."""

    @reference_kwargs(config="cfg")
    def __init__(self, cfg: ExpertParallelConfig, num_groups: int = 2, dtype=None, device=None):
        super().__init__()
        assert cfg.num_experts % num_groups == 0
        import dataclasses
        sub = dataclasses.replace(cfg, num_experts=cfg.num_experts // num_groups)
        self.groups = nn.ModuleList(MoELayer(sub, dtype, device) for _ in range(num_groups))
        self.coarse = nn.Linear(cfg.hidden_size, num_groups, bias=False, dtype=dtype, device=device)

    def forward(self, x=None, *, hidden_states=None, attention_mask=None):
        """`layer(x)` -> output; `layer(hidden_states=, attention_mask=)` -> (output, auxiliary loss): padded rows
        (mask 0) are routed nowhere and come out as zeros."""
        reference_form = hidden_states is not None
        x = hidden_states if reference_form else x
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        g = torch.softmax(self.coarse(x2).float(), -1)
        top = g.argmax(-1)
        if attention_mask is not None:
            top = top.masked_fill(~attention_mask.reshape(-1).to(torch.bool), -1)
        out = torch.zeros_like(x2)
        for gi, layer in enumerate(self.groups):
            m = top == gi
            if m.any():
                out[m] = layer(x2[m]) * g[m, gi].unsqueeze(-1).to(x2.dtype)
        if reference_form:
            aux = self.aux_loss
            return out.view(shp), aux if torch.is_tensor(aux) else x2.new_zeros(())
        return out.view(shp)

    @property
    def aux_loss(self):
        return sum(l.aux_loss for l in self.groups)


# ------------------------------------------------------------------------------------------------ decoder integration
class ExpertParallelDecoderMoE(nn.Module):
    """The decoder's mixture-of-experts MLP (`models.llama.LlamaMoEMLP`) with its experts sharded over an
    expert-parallel group: rank r keeps experts [r E/W, (r+1) E/W); the router is replicated.  Tokens are sorted by
    expert, sent to the owners with one all-to-all, run through the local experts, sent back and combined with the
    routing weights.  Gradients of the local experts are complete on their owner (every token that chose them was
    there); the router's gradient is a data-parallel gradient like any replicated parameter."""

    def __init__(self, mlp, group, peer=None):
        super().__init__()
        E = mlp.router.shape[0]
        self.dispatcher = AllToAllDispatcher(group, E)
        # `ep_peer.PeerDispatcher` of the group (shared by all layers) or None: tokens then travel through the
        # library all-to-all above
        self.peer = peer
        El, r = self.dispatcher.local_experts, self.dispatcher.rank
        self.act, self.top_k, self.norm_topk, self.aux_coef = mlp.act, mlp.top_k, mlp.norm_topk, mlp.aux_coef
        self.num_experts = E
        self.router = nn.Parameter(mlp.router.detach().clone())
        self.w_gate_up = nn.Parameter(mlp.w_gate_up.detach()[r * El:(r + 1) * El].clone())
        self.w_down = nn.Parameter(mlp.w_down.detach()[r * El:(r + 1) * El].clone())
        for p in (self.w_gate_up, self.w_down):
            p.expert_parallel = True          # not replicated over the ep group: no gradient averaging across it
        self.lora = None
        self.aux_loss = None

    def _local_experts(self, rows: torch.Tensor, per_expert: list[int]) -> torch.Tensor:
        outs, off = [], 0
        for e, n in enumerate(per_expert):
            if n:
                xe = rows[off:off + n]
                outs.append(gemm.linear(activation.glu(gemm.linear(xe, self.w_gate_up[e]), self.act), self.w_down[e]))
                off += n
        return torch.cat(outs) if outs else rows.new_zeros(0, rows.shape[-1])

    def forward(self, x):
        from ..ops import moe as moe_ops
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        logits = F.linear(x2, self.router)
        w, ids, probs = moe_ops.topk_softmax(logits, self.top_k, self.norm_topk)
        if self.peer is not None and moe_ops.available(x2):
            # peer-memory path: no host synchronisation, permutation fused into the transfers, grouped GEMMs
            from .ep_peer import expert_parallel_ffn
            y = expert_parallel_ffn(x2.contiguous(), ids, w.to(x2.dtype), self.w_gate_up, self.w_down, self.peer, self.act)
            self._aux(ids, probs, x)
            return y.view(shape)
        d = self.dispatcher
        xs, order, counts = permute_tokens(x2, ids, self.num_experts)
        recv, recv_counts, book = d.dispatch(xs, counts)
        W, El = d.world, d.local_experts
        rc = recv_counts.tolist()
        offs, o = [[0] * El for _ in range(W)], 0
        for r in range(W):
            for e in range(El):
                offs[r][e] = o
                o += rc[r][e]
        gather_idx = torch.cat([torch.arange(offs[r][e], offs[r][e] + rc[r][e], device=x2.device)
                                for e in range(El) for r in range(W)]) if o > 0 else \
            torch.zeros(0, dtype=torch.long, device=x2.device)
        ye = self._local_experts(recv[gather_idx], [sum(rc[r][e] for r in range(W)) for e in range(El)])
        back = torch.zeros_like(recv)
        back = back.index_copy(0, gather_idx, ye.to(back.dtype)) if o > 0 else back
        ys = d.combine(back, book)
        y = unpermute_tokens(ys, order, w.to(ys.dtype), x2.shape[0])
        self._aux(ids, probs, x)
        return y.view(shape)

    def _aux(self, ids, probs, x) -> None:
        if self.aux_coef > 0 and self.training:
            frac = torch.zeros(self.num_experts, device=x.device).index_add_(
                0, ids.reshape(-1).long(), torch.ones(ids.numel(), device=x.device)) / ids.numel()
            self.aux_loss = self.num_experts * (frac * probs.mean(0)).sum()

    def full_expert_weights(self):
        """(w_gate_up [E, 2I, H], w_down [E, H, I]) gathered over the group (collective)."""
        out = []
        for t in (self.w_gate_up, self.w_down):
            parts = [torch.empty_like(t) for _ in range(self.dispatcher.world)]
            dist.all_gather(parts, t.detach().contiguous(), group=self.dispatcher.group)
            out.append(torch.cat(parts))
        return tuple(out)


def make_peer_dispatcher(group, num_experts: int, device):
    """`ep_peer.PeerDispatcher` over a symmetric-memory heap of `group`, or None where peer memory is not available
    (CPU, no peer access, TS_DISABLE_SYMM=1).  Collective over the group."""
    device = torch.device(device)
    if device.type != "cuda":
        return None
    from .ep_peer import PeerDispatcher
    from .symm import SymmetricHeap
    heap = SymmetricHeap.try_create(group, device)
    return None if heap is None else PeerDispatcher(heap, num_experts)


def shard_model_for_expert_parallel(model, group, comm: str = "nccl", device=None) -> int:
    """Replace every mixture-of-experts MLP of a framework decoder by its expert-parallel form.  Returns the number of
    layers converted.  Call before the data-parallel engine is built (parameters are re-created).
    `comm`: "nccl" moves tokens with the library all-to-all; "auto" / "fused" with the peer-memory kernels of
    `ep_peer` when the group has symmetric memory ("fused" raises when it has not)."""
    from ..models.llama import LlamaMoEMLP
    moe_layers = [layer for layer in model.model.layers if isinstance(layer.mlp, LlamaMoEMLP)]
    peer = None
    if moe_layers and comm in ("auto", "fused"):
        device = device if device is not None else next(model.parameters()).device
        peer = make_peer_dispatcher(group, moe_layers[0].mlp.router.shape[0], device)
        if peer is None and comm == "fused":
            raise RuntimeError("distributed.comm: fused needs symmetric memory over the expert-parallel group")
    for layer in moe_layers:
        layer.mlp = ExpertParallelDecoderMoE(layer.mlp, group, peer)
    model.ep_peer = peer
    return len(moe_layers)


# ------------------------------------------------------------------------------------------------ trainer engine
class ExpertParallelEngine:
    """Data parallelism with the decoder's experts sharded over expert-parallel groups, behind the engine surface
    SOTATrainer drives (`backward`, `step`, `zero_grad`, `param_groups`, `state_dict`, ...).

    `distributed.parallel.ep = k` cuts the W data-parallel ranks into W / k groups of k consecutive ranks; inside a
    group every rank keeps E / k experts of every mixture-of-experts layer and tokens travel to their experts and
    back (data_pipeline/trainer/distributed/expert_parallel.py:219-454,1693; mesh keys :1049-1057 of parallel_dims.py).
    Two flat engines share the model and its autograd graph:
      dense   every parameter that is replicated on all W ranks (attention, norms, routers, embeddings): reduced over W
      expert  the expert weights: the W / k ranks that hold the same experts reduce among themselves; a gradient
              already holds the contributions of the k ranks whose tokens visited the expert, so it is scaled by 1 / k
              to make the update the gradient of the global mean loss
    and they clip with ONE norm: dense norm^2 + expert norm^2 summed over the k different expert shards."""

    def __init__(self, model, cfg, ep_size: int, device, sharding: str = "SHARD_GRAD_OP"):
        import copy as _copy

        from .flat_engine import FlatShardedEngine
        W, rank = dist.get_world_size(), dist.get_rank()
        if W % ep_size:
            raise ValueError(f"expert-parallel size {ep_size} must divide the data-parallel size {W}")
        self.ep_size = ep_size
        self.ep_group = self.edp_group = None
        for g in range(W // ep_size):            # every rank creates every group, in the same order
            grp = dist.new_group(list(range(g * ep_size, (g + 1) * ep_size)))
            if rank // ep_size == g:
                self.ep_group = grp
        for j in range(ep_size):
            grp = dist.new_group(list(range(j, W, ep_size)))
            if rank % ep_size == j:
                self.edp_group = grp
        self.converted = shard_model_for_expert_parallel(model, self.ep_group, getattr(cfg, "comm", "nccl"), device)
        self.peer = getattr(model, "ep_peer", None)
        if self.converted == 0:
            raise ValueError("distributed.parallel.ep > 1 but the model has no mixture-of-experts layer")
        expert_ids = {id(p) for p in model.parameters() if getattr(p, "expert_parallel", False)}
        dense_cfg = _copy.copy(cfg)
        dense_cfg.sharding_strategy = sharding if sharding != "FULL_SHARD" else "SHARD_GRAD_OP"
        self.dense = FlatShardedEngine(model, dense_cfg, device=device, param_filter=lambda p: id(p) not in expert_ids)
        exp_cfg = _copy.copy(cfg)
        exp_cfg.sharding_strategy, exp_cfg.comm, exp_cfg.grad_mul = dense_cfg.sharding_strategy, "nccl", 1.0 / ep_size
        self.expert = FlatShardedEngine(model, exp_cfg, process_group=self.edp_group, device=device,
                                        solo=W // ep_size == 1, param_filter=lambda p: id(p) in expert_ids)
        self.param_groups = self.dense.param_groups
        self.cfg = dense_cfg
        self.model = model

    @property
    def micro_step(self):
        return self.dense.micro_step

    @micro_step.setter
    def micro_step(self, v):
        self.dense.micro_step = self.expert.micro_step = v

    @property
    def units(self):
        return self.dense.units + self.expert.units

    @property
    def last_grad_norm(self):
        return self.dense.last_grad_norm

    def backward(self, loss):
        sync = self.dense.backward(loss)       # one backward over the shared graph; both engines' hooks fire in it
        self.expert.after_backward()
        return sync

    def step(self, lr=None):
        d, e = self.dense, self.expert
        e.param_groups[0].update(d.param_groups[0])
        d.reduce_and_norm()
        e.reduce_and_norm()
        ex = e.norm_sq.clone()
        nf = e.nonfinite.clone()
        dist.all_reduce(ex, group=self.ep_group)                     # the k ranks of a group hold different experts
        dist.all_reduce(nf, op=dist.ReduceOp.MAX, group=self.ep_group)
        total = d.norm_sq + ex
        flag = torch.maximum(d.nonfinite, nf)
        for eng in (d, e):
            eng.norm_sq.copy_(total)
            eng.nonfinite.copy_(flag)
        gn = d.apply_update(lr)
        e.apply_update(lr)
        return gn

    def zero_grad(self):
        self.dense.zero_grad()
        self.expert.zero_grad()

    def check_comm_status(self):
        self.dense.check_comm_status()
        self.expert.check_comm_status()
        if self.peer is not None:
            self.peer.heap.check_status()
            self.peer.check()

    @contextlib.contextmanager
    def summon_full_params(self):
        with self.dense.summon_full_params(), self.expert.summon_full_params():
            yield

    def state_dict(self):
        return {"dense": self.dense.state_dict(), "expert": self.expert.state_dict(), "ep_size": self.ep_size}

    def load_state_dict(self, sd):
        self.dense.load_state_dict(sd["dense"])
        self.expert.load_state_dict(sd["expert"])

    def memory_summary(self):
        return f"ep={self.ep_size} | dense: {self.dense.memory_summary()} | experts: {self.expert.memory_summary()}"


# ------------------------------------------------------------------------------------------------ reference surface
from enum import Enum  # noqa: E402
from typing import NamedTuple  # noqa: E402


class RoutingStrategy(Enum):
    TOP_K = "top_k"
    EXPERT_CHOICE = "expert_choice"
    SOFT_MOE = "soft"
    HASH_ROUTING = "hash"


class LoadBalanceLossType(Enum):
    SWITCH = "switch"        # E * sum_e f_e P_e
    GSHARD = "gshard"        # the same on the top-1 assignment only
    STMOE = "stmoe"          # Switch term + z-loss
    VMOE = "vmoe"            # squared coefficient of variation of importance and of load


class RoutingOutput(NamedTuple):
    """Dense (capacity-slotted) view of a routing decision (data_pipeline/trainer/distributed/expert_parallel.py:67)."""
    dispatch_mask: torch.Tensor       # [T, E, C] bool
    combine_weights: torch.Tensor     # [T, E, C]
    expert_indices: torch.Tensor      # [T, k]
    expert_weights: torch.Tensor      # [T, k]
    router_logits: torch.Tensor       # [T, E]
    auxiliary_loss: torch.Tensor
    metadata: dict


def get_expert_parallel_rank(group=None) -> int:
    return dist.get_rank(group=group) if dist.is_available() and dist.is_initialized() else 0


def get_expert_parallel_world_size(group=None) -> int:
    return dist.get_world_size(group=group) if dist.is_available() and dist.is_initialized() else 1


def load_balance_loss(kind: LoadBalanceLossType, probs: torch.Tensor, expert_indices: torch.Tensor,
                      logits: torch.Tensor | None = None, z_weight: float = 1e-3) -> torch.Tensor:
    """Auxiliary loss of the chosen flavour from router probabilities [T, E] and chosen experts [T, k]."""
    E = probs.shape[1]
    hot = F.one_hot(expert_indices, E).float()
    if kind is LoadBalanceLossType.GSHARD:
        hot = hot[:, :1]
    f = hot.sum(1).mean(0) / hot.shape[1]
    P = probs.mean(0)
    if kind is LoadBalanceLossType.VMOE:
        cv2 = lambda v: v.var() / v.mean().clamp(min=1e-9) ** 2      # noqa: E731
        return cv2(probs.sum(0)) + cv2(hot.sum((0, 1)))
    loss = E * (f * P).sum()
    if kind is LoadBalanceLossType.STMOE and logits is not None:
        loss = loss + z_weight * torch.logsumexp(logits.float(), -1).pow(2).mean()
    return loss


class RouterBase(nn.Module):
    """Common part of a router: the projection hidden -> experts (small initial weights), the auxiliary loss, and the
    conversion of a top-k decision into the dense capacity-slotted `RoutingOutput`.  Subclasses implement `route`."""

    def __init__(self, config: ExpertParallelConfig, loss_type: LoadBalanceLossType = LoadBalanceLossType.SWITCH):
        super().__init__()
        self.config, self.loss_type = config, loss_type
        self.router = nn.Linear(config.hidden_size, config.num_experts, bias=False)
        nn.init.normal_(self.router.weight, std=0.01)

    def route(self, logits: torch.Tensor):
        """logits [T, E] -> (weights [T, k], experts [T, k], probs [T, E]); top-k soft-max by default."""
        from ..ops import moe as moe_ops
        return moe_ops.topk_softmax(logits, self.config.top_k, self.config.normalize_topk)

    def compute_router_logits(self, hidden_states: torch.Tensor) -> torch.Tensor:
        """[..., H] -> [..., E]; in fp32 (input and weight upcast) when `use_fp32_router`: the soft-max over experts is
        sensitive to bf16 rounding of near-tied logits."""
        if getattr(self.config, "use_fp32_router", True) and hidden_states.dtype != torch.float32:
            return F.linear(hidden_states.float(), self.router.weight.float())
        return self.router(hidden_states)

    def compute_auxiliary_loss(self, router_logits: torch.Tensor, expert_mask: torch.Tensor, num_experts: int | None = None):
        """(weighted total, {name: unweighted term}) from raw logits [T, E] and the 0/1 mask of chosen experts [T, E]:
        `load_balance` = E sum_e f_e P_e always; `router_z_loss` = mean logsumexp^2 for ST-MoE and GShard;
        `importance_loss` = CV^2 of the per-expert probability mass for GShard and V-MoE
        (data_pipeline/trainer/distributed/expert_parallel.py:548-610)."""
        cfg, kind = self.config, self.loss_type
        E = num_experts or router_logits.shape[-1]
        logits = router_logits.float().reshape(-1, router_logits.shape[-1])
        probs = logits.softmax(-1)
        f = expert_mask.float().reshape(-1, expert_mask.shape[-1]).sum(0) / max(logits.shape[0], 1)
        terms = {"load_balance": E * (f * probs.mean(0)).sum()}
        if kind in (LoadBalanceLossType.STMOE, LoadBalanceLossType.GSHARD):
            terms["router_z_loss"] = torch.logsumexp(logits, -1).pow(2).mean()
        if kind in (LoadBalanceLossType.GSHARD, LoadBalanceLossType.VMOE):
            imp = probs.sum(0)
            terms["importance_loss"] = (imp.std() / (imp.mean() + 1e-9)) ** 2
        total = cfg.aux_loss_weight * terms["load_balance"]
        if "router_z_loss" in terms:
            total = total + cfg.z_loss_weight * terms["router_z_loss"]
        if "importance_loss" in terms:
            total = total + cfg.aux_loss_weight * terms["importance_loss"]
        return total, terms

    def forward(self, x: torch.Tensor | None = None, padding_mask=None, *, hidden_states=None) -> RoutingOutput:
        """[..., H] (and the padding mask [...], True = padded token) -> the dense `RoutingOutput`."""
        cfg = self.config
        x = hidden_states if hidden_states is not None else x
        flat = x.reshape(-1, x.shape[-1])
        logits = self.router(flat).float()
        w, idx, probs = self.route(logits)
        aux = cfg.aux_loss_weight * load_balance_loss(self.loss_type, probs, idx, logits, cfg.z_loss_weight)
        return _dense_routing(cfg, logits, w, idx, aux, padding_mask)


CACHE_LINE_SIZE, WARP_SIZE, EPS = 64, 32, 1e-6      # names of data_pipeline/trainer/distributed/expert_parallel.py
