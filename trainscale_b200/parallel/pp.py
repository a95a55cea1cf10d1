"""Pipeline parallelism: stage partitioning, schedules (GPipe, 1F1B, interleaved 1F1B, zero-bubble with the
B / W split), a schedule simulator, and a runtime that executes a schedule with NCCL / gloo point-to-point.

Feature set after data_pipeline/trainer/distributed/pipeline_parallel.py:1267-2619 (schedules, stage split by layer
count or by cost, micro-batch split) and data_pipeline/trainer/distributed/zbpp.py + ZBPP.md:716-960 (F / B_input /
B_params ops, weight-gradient work deferred into bubbles, bubble fraction = (makespan*P - sum compute) /
(makespan*P)).  Unlike the reference's single-process schedules, every stage here is a rank: activations and their
gradients move with `batch_isend_irecv` on the pipeline group, posted ahead of the compute that needs them.
The zero-bubble split uses the deferred weight-gradient queue of ops/gemm.py: B runs only input-gradient GEMMs,
W later runs the parked weight-gradient GEMMs.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops.gemm import WgradQueue

F_OP, B_OP, W_OP = "F", "B", "W"


@dataclass(frozen=True)
class Action:
    op: str          # F | B | W
    mb: int          # micro-batch index
    chunk: int = 0   # virtual stage (model chunk) index on this rank, for interleaved schedules


# ------------------------------------------------------------------------------------------------ schedules
def gpipe_schedule(stage: int, P: int, M: int) -> list[Action]:
    return [Action(F_OP, m) for m in range(M)] + [Action(B_OP, m) for m in reversed(range(M))]


def one_f_one_b_schedule(stage: int, P: int, M: int) -> list[Action]:
    warm = min(P - stage - 1, M)
    acts = [Action(F_OP, m) for m in range(warm)]
    f, b = warm, 0
    while f < M:
        acts.append(Action(F_OP, f))
        f += 1
        acts.append(Action(B_OP, b))
        b += 1
    while b < M:
        acts.append(Action(B_OP, b))
        b += 1
    return acts


def interleaved_1f1b_schedule(stage: int, P: int, M: int, V: int) -> list[Action]:
    """V model chunks per rank (virtual stage = chunk * P + stage); micro-batches advance in groups of P."""
    if M % P != 0:
        raise ValueError("interleaved 1F1B needs num_microbatches divisible by the pipeline size")
    total = M * V

    def fwd_id(k):   # k-th forward executed on this rank -> (chunk, micro-batch)
        group, within = divmod(k, P * V)
        chunk, j = divmod(within, P)
        return chunk, group * P + j

    def bwd_id(k):
        group, within = divmod(k, P * V)
        chunk, j = divmod(within, P)
        return V - 1 - chunk, group * P + j

    warm = min((P - stage - 1) * 2 + (V - 1) * P, total)
    acts = []
    for k in range(warm):
        c, m = fwd_id(k)
        acts.append(Action(F_OP, m, c))
    f, b = warm, 0
    while f < total:
        c, m = fwd_id(f)
        acts.append(Action(F_OP, m, c))
        f += 1
        c, m = bwd_id(b)
        acts.append(Action(B_OP, m, c))
        b += 1
    while b < total:
        c, m = bwd_id(b)
        acts.append(Action(B_OP, m, c))
        b += 1
    return acts


def zero_bubble_schedule(stage: int, P: int, M: int) -> list[Action]:
    """ZB-H1: 1F1B order for F and B (input gradients only); each W (weight gradients) is deferred and issued where
    1F1B would idle - during cool-down, and in steady state one W after each B once the warm-up debt is paid."""
    warm = min(P - stage - 1, M)
    acts = [Action(F_OP, m) for m in range(warm)]
    f, b, w = warm, 0, 0
    while f < M:
        acts.append(Action(F_OP, f))
        f += 1
        acts.append(Action(B_OP, b))
        b += 1
        if b - w > stage:   # later stages wait less during cool-down, so they can retire W work earlier
            acts.append(Action(W_OP, w))
            w += 1
    while b < M:
        acts.append(Action(B_OP, b))
        b += 1
        if w < b:
            acts.append(Action(W_OP, w))
            w += 1
    while w < M:
        acts.append(Action(W_OP, w))
        w += 1
    return acts


def create_schedule(name: str, stage: int, P: int, M: int, V: int = 1) -> list[Action]:
    name = name.lower()
    if name in ("gpipe", "fill_drain"):
        return gpipe_schedule(stage, P, M)
    if name in ("1f1b", "one_f_one_b"):
        return one_f_one_b_schedule(stage, P, M)
    if name in ("interleaved", "interleaved_1f1b"):
        return interleaved_1f1b_schedule(stage, P, M, V)
    if name in ("zero_bubble", "zb", "zbh1", "zbpp"):
        return zero_bubble_schedule(stage, P, M)
    raise ValueError(f"unknown pipeline schedule {name!r}")


def simulate(schedules: Sequence[Sequence[Action]], cost: dict[str, float] | None = None, comm: float = 0.0) -> dict:
    """Event simulation of per-stage action lists (single chunk per stage). Returns makespan, per-stage busy time and
    the bubble fraction. Dependencies: F(s,m) after F(s-1,m); B(s,m) after B(s+1,m) and F(s,m); W(s,m) after B(s,m)."""
    cost = cost or {F_OP: 1.0, B_OP: 2.0, W_OP: 0.0}
    P = len(schedules)
    has_w = any(a.op == W_OP for s in schedules for a in s)
    if has_w and cost.get(W_OP, 0.0) == 0.0:
        cost = {F_OP: cost[F_OP], B_OP: cost[B_OP] / 2, W_OP: cost[B_OP] / 2}
    done: dict[tuple, float] = {}
    t = [0.0] * P
    idx = [0] * P
    busy = [0.0] * P
    progressed = True
    while progressed:
        progressed = False
        for s in range(P):
            while idx[s] < len(schedules[s]):
                a = schedules[s][idx[s]]
                deps = []
                if a.op == F_OP and s > 0:
                    deps.append((F_OP, s - 1, a.mb))
                if a.op == B_OP:
                    deps.append((F_OP, s, a.mb))
                    if s < P - 1:
                        deps.append((B_OP, s + 1, a.mb))
                if a.op == W_OP:
                    deps.append((B_OP, s, a.mb))
                if any(d not in done for d in deps):
                    break
                ready = max([t[s]] + [done[d] + (comm if d[1] != s else 0.0) for d in deps])
                end = ready + cost[a.op]
                done[(a.op, s, a.mb)] = end
                t[s] = end
                busy[s] += cost[a.op]
                idx[s] += 1
                progressed = True
    if any(idx[s] < len(schedules[s]) for s in range(P)):
        raise RuntimeError("schedule deadlocks: unmet dependencies")
    makespan = max(t)
    return {"makespan": makespan, "busy": busy, "bubble_fraction": (makespan * P - sum(busy)) / (makespan * P)}


# ------------------------------------------------------------------------------------------------ partitioning
def split_layers(num_layers: int, num_stages: int, costs: Sequence[float] | None = None) -> list[range]:
    """Contiguous layer ranges per stage: equal counts, or minimal maximum stage cost (binary search) when per-layer
    costs are given (data_pipeline/trainer/distributed/zbpp.py:3119-3163)."""
    if costs is None:
        base, extra = divmod(num_layers, num_stages)
        out, s = [], 0
        for i in range(num_stages):
            n = base + (1 if i < extra else 0)
            out.append(range(s, s + n))
            s += n
        return out
    lo, hi = max(costs), sum(costs)

    def fits(cap):
        n, cur = 1, 0.0
        for c in costs:
            if cur + c > cap:
                n, cur = n + 1, 0.0
            cur += c
        return n <= num_stages

    for _ in range(50):
        mid = (lo + hi) / 2
        if fits(mid):
            hi = mid
        else:
            lo = mid
    out, s, cur = [], 0, 0.0
    for i, c in enumerate(costs):
        remaining_stages = num_stages - len(out) - 1
        if (cur + c > hi * (1 + 1e-9) and i > s) or (num_layers - i) <= remaining_stages and i > s:
            out.append(range(s, i))
            s, cur = i, 0.0
        cur += c
    out.append(range(s, num_layers))
    while len(out) < num_stages:
        out.append(range(num_layers, num_layers))
    return out


class LlamaStage(nn.Module):
    """One pipeline stage of the framework decoder: [embedding] + layers[a:b] + [final norm + loss head]."""

    def __init__(self, model, layers: range, first: bool, last: bool):
        super().__init__()
        self.first, self.last = first, last
        self.config = model.config
        self.embed_tokens = model.model.embed_tokens if first else None
        self.layers = nn.ModuleList(model.model.layers[i] for i in layers)
        self.norm = model.model.norm if last else None
        self.lm_head = model.lm_head if (last and model.lm_head is not None) else None
        self._tied = last and model.lm_head is None
        if self._tied:
            self.tied_embedding = model.model.embed_tokens   # last stage keeps its own copy; grads are all-reduced
        # rotary tables come from the whole decoder; kept out of the module tree so that a stage's parameters are
        # exactly what it trains (the optimizer of stage k must not hold another stage's embedding or norm)
        object.__setattr__(self, "_rope", model.model)

    def forward(self, x, labels=None, loss_scale: float = 1.0):
        """First stage: x = token ids [B, S]. Other stages: x = packed (hidden | residual) [B, S, 2H].
        Last stage with labels returns the loss; otherwise the packed activations."""
        from ..ops import cross_entropy
        if self.first:
            h, res = self.embed_tokens(x), None
            if getattr(self.config, "scale_embeddings", False):
                h = h * torch.tensor(self.config.hidden_size ** 0.5, dtype=h.dtype)
        else:
            H = x.shape[-1] // 2
            h, res = x[..., :H], x[..., H:]
        sp = getattr(self, "sp_ctx", None)
        S_full = h.shape[1] * (sp.size if (sp is not None and not self.first) else 1)
        cos, sin = self._rope.rope_tables(h.device, S_full)
        if sp is not None and self.first:
            # sequence parallelism: from here on (and between stages) every tensor-parallel rank holds S / tp tokens
            from . import tp as TP
            if h.shape[0] != 1:
                raise ValueError("sequence-parallel pipeline stages take one sequence per micro-batch")
            h = TP.scatter_to_sequence_parallel_region(h.view(S_full, -1), sp).view(1, S_full // sp.size, -1)
        ckpt = self._rope.gradient_checkpointing and self.training and torch.is_grad_enabled()
        every = max(1, getattr(self._rope, "checkpoint_every", 1))
        for i, layer in enumerate(self.layers):
            if ckpt and i % every == 0:
                from torch.utils.checkpoint import checkpoint
                h, res = checkpoint(layer, h, res, cos, sin, use_reentrant=False)
            else:
                h, res = layer(h, res, cos, sin)
        if not self.last:
            if res is None:
                res = torch.zeros_like(h)
            return torch.cat((h, res), dim=-1)
        h, _ = self.norm(h, res)
        if sp is not None:
            from . import tp as TP
            from ..models.llama import _ScaleGrad
            # every rank computes the full loss on the gathered tokens; the gather's backward sums tp copies
            h = TP.all_gather_from_sequence_parallel_region(h.view(S_full // sp.size, -1), sp).view(1, S_full, -1)
            h = _ScaleGrad.apply(h, 1.0 / sp.size)
        if labels is None:
            return h
        tgt = torch.full_like(labels, -100)
        tgt[..., :-1] = labels[..., 1:]
        w = self.lm_head if self.lm_head is not None else self.tied_embedding.weight
        loss, _ = cross_entropy.fused_linear_cross_entropy(h, w, tgt, loss_scale=loss_scale)
        return loss


def split_model_into_stages(model, num_stages: int, stage: int, costs: Sequence[float] | None = None) -> LlamaStage:
    ranges = split_layers(len(model.model.layers), num_stages, costs)
    return LlamaStage(model, ranges[stage], stage == 0, stage == num_stages - 1)


def split_into_microbatches(batch: dict, num_microbatches: int) -> list[dict]:
    out = [dict() for _ in range(num_microbatches)]
    for k, v in batch.items():
        parts = v.chunk(num_microbatches, dim=0) if torch.is_tensor(v) and v.dim() > 0 else [v] * num_microbatches
        for i, p in enumerate(parts):
            out[i][k] = p
    return out


# ------------------------------------------------------------------------------------------------ runtime
class PipelineRuntime:
    """Executes one schedule on this rank's stage. Activations travel as one packed tensor [mb, S, 2H]."""

    def __init__(self, stage_module: nn.Module, stage: int, num_stages: int, group=None, schedule: str = "1f1b",
                 prev_rank: int | None = None, next_rank: int | None = None, grad_group=None):
        """`group` carries the activations (stage s -> s + 1), `grad_group` the activation gradients (s + 1 -> s).
        On NCCL the two directions need their own communicators: in 1F1B a stage sends its next activation while its
        neighbour sends a gradient back; on ONE communicator each send waits for the matching receive, which is queued
        behind the other rank's own send, and large messages (no eager buffering) dead-lock."""
        self.mod, self.stage, self.P, self.group, self.schedule_name = stage_module, stage, num_stages, group, schedule
        self.grad_group = grad_group if grad_group is not None else group
        self.prev_rank = prev_rank if prev_rank is not None else stage - 1
        self.next_rank = next_rank if next_rank is not None else stage + 1
        self.first, self.last = stage == 0, stage == num_stages - 1
        self.wq = WgradQueue()
        self.stats = {"sent_bytes": 0, "recv_bytes": 0}

    def _send(self, t: torch.Tensor, dst: int, grad: bool = False):
        self.stats["sent_bytes"] += t.numel() * t.element_size()
        return dist.isend(t.contiguous(), dst, group=self.grad_group if grad else self.group)

    def _recv(self, shape, dtype, device, src: int, grad: bool = False):
        buf = torch.empty(shape, dtype=dtype, device=device)
        self.stats["recv_bytes"] += buf.numel() * buf.element_size()
        return buf, dist.irecv(buf, src, group=self.grad_group if grad else self.group)

    def train_step(self, microbatches: Sequence[dict], act_shape: tuple, act_dtype, device,
                   extra_scale: float = 1.0) -> torch.Tensor | None:
        """Runs all micro-batches through this stage; returns the mean loss on the last stage (None elsewhere).
        `act_shape` is the packed activation shape [mb, S, 2H] exchanged between stages; `extra_scale` multiplies
        every micro-batch loss (gradient accumulation over several pipeline steps)."""
        M = len(microbatches)
        acts = create_schedule(self.schedule_name, self.stage, self.P, M)
        split = any(a.op == W_OP for a in acts)
        inputs: dict[int, torch.Tensor] = {}
        outputs: dict[int, torch.Tensor] = {}
        losses = []
        pending = []
        w_marks: dict[int, int] = {}
        for a in acts:
            mb = microbatches[a.mb]
            if a.op == F_OP:
                if self.first:
                    x = mb["input_ids"]
                else:
                    x, work = self._recv(act_shape, act_dtype, device, self.prev_rank)
                    work.wait()
                    x.requires_grad_(True)
                inputs[a.mb] = x
                if self.last:
                    out = self.mod(x, labels=mb.get("labels", mb["input_ids"]), loss_scale=extra_scale / M)
                    losses.append(out.detach())
                else:
                    out = self.mod(x)
                    pending.append(self._send(out.detach(), self.next_rank))
                outputs[a.mb] = out
            elif a.op == B_OP:
                out = outputs.pop(a.mb)
                if self.last:
                    grad = None
                else:
                    grad, work = self._recv(act_shape, act_dtype, device, self.next_rank, grad=True)
                    work.wait()
                before = len(self.wq)
                if split:
                    with self.wq.defer():
                        torch.autograd.backward(out, grad)
                    w_marks[a.mb] = len(self.wq) - before
                else:
                    torch.autograd.backward(out, grad)
                x = inputs.pop(a.mb)
                if not self.first:
                    pending.append(self._send(x.grad, self.prev_rank, grad=True))
            else:   # W: retire the weight-gradient GEMMs parked by B of this micro-batch
                self.wq.run(w_marks.pop(a.mb, None))
        self.wq.run()
        for w in pending:
            w.wait()
        if self.last:
            return torch.stack(losses).sum()
        return None


def allreduce_tied_embedding_grads(stage_module: LlamaStage, group, first_rank: int, last_rank: int) -> None:
    """Tied input / output embeddings live on the first and the last stage: sum their gradients
    (data_pipeline/trainer/distributed/finalize_grads.py:211)."""
    w = None
    if stage_module.first and stage_module.embed_tokens is not None:
        w = stage_module.embed_tokens.weight
    elif getattr(stage_module, "_tied", False):
        w = stage_module.tied_embedding.weight
    if w is None:
        return
    g = w.grad if w.grad is not None else getattr(w, "main_grad", None)
    if g is not None:
        pair = dist.new_group([first_rank, last_rank]) if group is None else group
        dist.all_reduce(g, group=pair)
