"""Zero-bubble pipeline parallelism: the backward of a stage is split into B_input (the gradient that the previous
stage waits for) and B_params (weight gradients, needed only by the optimizer), and B_params work is moved into the
slots where a 1F1B pipeline idles.

API after data_pipeline/trainer/distributed/zbpp.py:59-3709 and the schedule optimiser described in its ZBPP.md:716-960
(`OpType`, `ScheduleSlot`, `StageProfile`, `ScheduleConfig`, `ScheduleResult`, `ZBPPScheduleOptimizer`,
`GradientDecomposer`, `SplitBackwardFunction`, `PipelineStageModule`, `ZBPPOptimizer`, `ZBPPRuntimeEngine`,
`ModelPartitioner`, `ZeroBubblePipeline`, `ZBPPBenchmark`, `create_zbpp_pipeline`).

Execution goes through the executor of `parallel/pipeline.py` (any `nn.Module` stages, in one process or one stage per
rank); the framework decoder's production path is `pp.PipelineRuntime`, where B_params are parked weight-gradient
GEMMs on the tcgen05 kernel (`ops.gemm.WgradQueue`) instead of a second autograd walk.
"""
from __future__ import annotations

import enum
import heapq
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

from . import pipeline as PL
from . import pp as PP
from ..utils.refargs import ANY, reference_kwargs


class OpType(enum.IntEnum):
    FORWARD = 0
    BACKWARD_INPUT = 1
    BACKWARD_PARAMS = 2
    OPTIMIZER_STEP = 3
    SEND_ACTIVATION = 4
    RECV_ACTIVATION = 5
    SEND_GRAD = 6
    RECV_GRAD = 7
    NOOP = 8


class Priority(enum.IntEnum):
    CRITICAL = 0      # B_input: the previous stage is waiting
    HIGH = 1          # forward
    NORMAL = 2        # B_params
    LOW = 3


@dataclass(order=False)
class ScheduleSlot:
    stage_id: int
    microbatch_id: int
    op_type: OpType
    time_slot: int
    priority: Priority
    estimated_cost_us: float = 0.0
    memory_delta_bytes: int = 0
    start_us: float = 0.0

    def __lt__(self, other: "ScheduleSlot") -> bool:
        return (self.time_slot, self.priority) < (other.time_slot, other.priority)


@dataclass
class StageProfile:
    forward_us: float
    b_input_us: float
    b_params_us: float
    activation_bytes: int
    param_bytes: int
    comm_send_us: float = 50.0
    comm_recv_us: float = 50.0

    @property
    def backward_total_us(self) -> float:
        return self.b_input_us + self.b_params_us

    @property
    def total_compute_us(self) -> float:
        return self.forward_us + self.b_input_us + self.b_params_us


@dataclass
class ScheduleConfig:
    num_stages: int
    num_microbatches: int
    memory_limit_bytes: int
    stage_profiles: list[StageProfile]
    enable_sync_bypass: bool = True
    enable_interleaving: bool = True
    max_concurrent_activations: int = -1

    def __post_init__(self) -> None:
        if self.num_stages < 2:
            raise ValueError(f"a pipeline needs at least 2 stages, got {self.num_stages}")
        if self.num_microbatches < self.num_stages:
            raise ValueError(f"M={self.num_microbatches} micro-batches cannot fill P={self.num_stages} stages")
        if len(self.stage_profiles) != self.num_stages:
            raise ValueError("one StageProfile per stage is required")
        if self.max_concurrent_activations < 0:
            self.max_concurrent_activations = self.num_microbatches


@dataclass
class ScheduleResult:
    schedule: dict[int, list[ScheduleSlot]]
    bubble_fraction: float
    peak_memory_bytes: dict[int, int]
    total_time_slots: int
    makespan_us: float

    def actions(self) -> list[list[PP.Action]]:
        """Per-stage (op, micro-batch) lists for the executor."""
        name = {OpType.FORWARD: PP.F_OP, OpType.BACKWARD_INPUT: PP.B_OP, OpType.BACKWARD_PARAMS: PP.W_OP}
        return [[PP.Action(name[s.op_type], s.microbatch_id) for s in self.schedule[st] if s.op_type in name]
                for st in sorted(self.schedule)]


class ZBPPScheduleOptimizer:
    """List scheduling with measured costs.  Every stage keeps three queues (F, B_input, B_params); whenever a stage
    becomes free it starts, in this order of preference: a ready B_input (critical path), a ready F if the stage may
    still take another live activation (1F1B's P - s in flight, tightened by the memory limit), else a pending
    B_params; if nothing is ready it idles until the next arrival.  B_params left over drain at the end."""

    def __init__(self, config: ScheduleConfig):
        self.config = config

    def _activation_cap(self, s: int) -> int:
        c, p = self.config, self.config.stage_profiles[s]
        # 1F1B keeps P - s activations alive on stage s, so only stage 0 is at its peak.  Deferring a B_params keeps
        # its activation longer; letting EVERY stage go up to stage 0's P activations (the ZB-H1 budget) costs no extra
        # peak memory.  Without that bound (enable_interleaving off) only the memory limit applies (ZB-H2 style).
        cap = min(c.max_concurrent_activations, c.num_stages if c.enable_interleaving else c.num_microbatches)
        if p.activation_bytes > 0:
            room = (c.memory_limit_bytes - p.param_bytes) // p.activation_bytes
            cap = min(cap, int(room))
        if cap < 1:
            raise ValueError(f"stage {s}: the memory limit does not hold one micro-batch of activations")
        return cap

    def _evaluate(self, orders: list[list[tuple[str, int]]]) -> ScheduleResult | None:
        """Timeline of fixed per-stage orders [("F"|"B"|"W", micro-batch), ...]; None if an order cannot run."""
        c = self.config
        P, prof = c.num_stages, c.stage_profiles
        t, idx, busy = [0.0] * P, [0] * P, [0.0] * P
        f_done: dict[tuple, float] = {}
        b_done: dict[tuple, float] = {}
        mem = [prof[s].param_bytes for s in range(P)]
        peak = list(mem)
        slots: dict[int, list[ScheduleSlot]] = {s: [] for s in range(P)}
        kinds = {"F": (OpType.FORWARD, Priority.HIGH), "B": (OpType.BACKWARD_INPUT, Priority.CRITICAL),
                 "W": (OpType.BACKWARD_PARAMS, Priority.NORMAL)}
        progressed = True
        while progressed:
            progressed = False
            for s in range(P):
                while idx[s] < len(orders[s]):
                    kind, m = orders[s][idx[s]]
                    if kind == "F":
                        dep = 0.0 if s == 0 else (f_done.get((s - 1, m)))
                        ready = dep if s == 0 else (None if dep is None else dep + prof[s - 1].comm_send_us)
                        cost, dmem = prof[s].forward_us, prof[s].activation_bytes
                    elif kind == "B":
                        if (s, m) not in f_done:
                            ready = None
                        elif s == P - 1:
                            ready = f_done[(s, m)]
                        else:
                            dep = b_done.get((s + 1, m))
                            ready = None if dep is None else dep + prof[s + 1].comm_send_us
                        cost, dmem = prof[s].b_input_us, 0
                    else:
                        ready = b_done.get((s, m))
                        cost, dmem = prof[s].b_params_us, -prof[s].activation_bytes
                    if ready is None:
                        break
                    start = max(t[s], ready)
                    op, pr = kinds[kind]
                    slots[s].append(ScheduleSlot(s, m, op, len(slots[s]), pr, cost, dmem, start))
                    t[s] = start + cost
                    busy[s] += cost
                    mem[s] += dmem
                    peak[s] = max(peak[s], mem[s])
                    if kind == "F":
                        f_done[(s, m)] = t[s]
                    elif kind == "B":
                        b_done[(s, m)] = t[s]
                    idx[s] += 1
                    progressed = True
        if any(idx[s] < len(orders[s]) for s in range(P)):
            return None
        makespan = max(t)
        bubble = (makespan * P - sum(busy)) / (makespan * P) if makespan > 0 else 0.0
        return ScheduleResult(slots, bubble, {s: peak[s] for s in range(P)}, max(len(v) for v in slots.values()),
                              makespan)

    def optimize(self) -> ScheduleResult:
        """The greedy list schedule, unless plain 1F1B (every B_params right after its B_input) fits the memory limit
        and finishes earlier - the greedy choice is a heuristic and can lose a few percent on small pipelines."""
        best = self._greedy()
        c = self.config
        orders = []
        for s in range(c.num_stages):
            lst = []
            for a in PP.one_f_one_b_schedule(s, c.num_stages, c.num_microbatches):
                lst.append((a.op, a.mb))
                if a.op == PP.B_OP:
                    lst.append(("W", a.mb))
            orders.append(lst)
        plain = self._evaluate(orders)
        if plain is not None and plain.makespan_us < best.makespan_us and \
                all(v <= c.memory_limit_bytes for v in plain.peak_memory_bytes.values()):
            return plain
        return best

    def _greedy(self) -> ScheduleResult:
        c = self.config
        P, M = c.num_stages, c.num_microbatches
        prof = c.stage_profiles
        caps = [self._activation_cap(s) for s in range(P)]
        t = [0.0] * P                                   # time at which the stage is free
        f_done: dict[tuple, float] = {}
        b_done: dict[tuple, float] = {}
        next_f, next_b = [0] * P, [0] * P
        w_pending: list[list[int]] = [[] for _ in range(P)]
        live = [0] * P
        mem = [prof[s].param_bytes for s in range(P)]
        peak = list(mem)
        slots: dict[int, list[ScheduleSlot]] = {s: [] for s in range(P)}
        busy = [0.0] * P
        remaining = 3 * P * M

        def f_ready(s):      # arrival time of the next forward's input, or None
            m = next_f[s]
            if m >= M:
                return None
            if s == 0:
                return 0.0
            d = f_done.get((s - 1, m))
            return None if d is None else d + prof[s - 1].comm_send_us

        def b_ready(s):
            m = next_b[s]
            if m >= M or (s, m) not in f_done:
                return None
            if s == P - 1:
                return f_done[(s, m)]
            d = b_done.get((s + 1, m))
            return None if d is None else d + prof[s + 1].comm_send_us

        def emit(s, m, op, start, cost, dmem, pr):
            slots[s].append(ScheduleSlot(s, m, op, len(slots[s]), pr, cost, dmem, start))
            t[s] = start + cost
            busy[s] += cost
            mem[s] += dmem
            peak[s] = max(peak[s], mem[s])

        while remaining:
            # the stage that can start something earliest goes next
            best = None
            for s in range(P):
                cands = []
                br, fr = b_ready(s), f_ready(s)
                if br is not None:
                    cands.append((max(t[s], br), 0, "B"))
                if fr is not None and live[s] < caps[s]:
                    cands.append((max(t[s], fr), 1, "F"))
                if w_pending[s]:
                    # weight gradients fill idle time: only if nothing on the critical path could start by then
                    cands.append((t[s], 2, "W"))
                if not cands:
                    continue
                start, pri, kind = min(cands)
                if kind != "W" and w_pending[s] and start > t[s] + 1e-9:
                    # the stage would idle until `start`: run a B_params there if it ends before the critical-path
                    # work could begin (a weight gradient that overran the gap would delay every later stage)
                    if t[s] + prof[s].b_params_us <= start + 1e-9:
                        start, pri, kind = t[s], 2, "W"
                key = (start, pri, s)
                if best is None or key < best[0]:
                    best = (key, s, kind)
            if best is None:
                raise RuntimeError("zero-bubble schedule cannot progress (memory limit too tight?)")
            (start, _, _), s, kind = best
            if kind == "F":
                m = next_f[s]
                emit(s, m, OpType.FORWARD, start, prof[s].forward_us, prof[s].activation_bytes, Priority.HIGH)
                f_done[(s, m)] = t[s]
                next_f[s] += 1
                live[s] += 1
            elif kind == "B":
                m = next_b[s]
                emit(s, m, OpType.BACKWARD_INPUT, start, prof[s].b_input_us, 0, Priority.CRITICAL)
                b_done[(s, m)] = t[s]
                next_b[s] += 1
                w_pending[s].append(m)
            else:
                m = w_pending[s].pop(0)
                emit(s, m, OpType.BACKWARD_PARAMS, start, prof[s].b_params_us, -prof[s].activation_bytes, Priority.NORMAL)
                live[s] -= 1
            remaining -= 1
        makespan = max(t)
        bubble = (makespan * P - sum(busy)) / (makespan * P) if makespan > 0 else 0.0
        return ScheduleResult(slots, bubble, {s: peak[s] for s in range(P)}, max(len(v) for v in slots.values()),
                              makespan)


# ------------------------------------------------------------------------------------------------ gradient split
class GradientDecomposer:
    """B_input / B_params as two walks over one retained autograd graph."""

    def __init__(self, use_triton: bool = False, dtype: torch.dtype | None = None, accumulate_grads: bool = True):
        """`dtype`: of the gradients the linear forms return (that of their operands when None); `accumulate_grads`:
        default of `compute_b_params(..., accumulate=)` for instances."""
        self._triton = False        # there is no Triton path: autograd + the framework's own kernels do the work
        self.dtype, self.accumulate_grads = dtype, accumulate_grads

    @property
    def using_triton(self) -> bool:
        return self._triton

    @staticmethod
    def _linear_b_input(grad_output: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """dL/dx of y = x W^T: grad_output [.., Out] @ weight [Out, In] (tensor-core GEMM on CUDA bf16)."""
        from ..ops import gemm
        return gemm.matmul_nn(grad_output, weight).view(*grad_output.shape[:-1], weight.shape[1])

    @staticmethod
    def _linear_b_params(input_tensor: torch.Tensor, grad_output: torch.Tensor, weight: torch.Tensor | None = None):
        """dL/dW of y = x W^T: grad_output^T [Out, N] @ input [N, In]."""
        from ..ops import gemm
        go = grad_output.reshape(-1, grad_output.shape[-1])
        return gemm.matmul_tn(go, input_tensor.reshape(-1, input_tensor.shape[-1]))

    @staticmethod
    def compute_b_input(output: torch.Tensor = None, inputs: "Sequence[torch.Tensor] | torch.Tensor" = None,
                        grad_output: torch.Tensor | None = None, retain_graph: bool = True, *,
                        weight: torch.Tensor | None = None) -> "tuple[torch.Tensor | None, ...] | torch.Tensor":
        """`compute_b_input(output, inputs, grad_output)`: input gradients by a walk over the retained graph.
        `compute_b_input(grad_output, weight)` is the closed form for a linear layer
        (data_pipeline/trainer/distributed/zbpp.py GradientDecomposer.compute_b_input)."""
        if weight is not None or torch.is_tensor(inputs):
            return GradientDecomposer._linear_b_input(grad_output if output is None else output,
                                                      weight if weight is not None else inputs)
        ins = [x for x in inputs if torch.is_tensor(x) and x.requires_grad]
        if not ins:
            return tuple(None for _ in inputs)
        gs = iter(torch.autograd.grad(output, ins, grad_output, retain_graph=retain_graph, allow_unused=True))
        return tuple(next(gs) if torch.is_tensor(x) and x.requires_grad else None for x in inputs)

    @staticmethod
    def compute_b_params(output: torch.Tensor = None, params: "Sequence[nn.Parameter] | torch.Tensor" = None,
                         grad_output: torch.Tensor | None = None, accumulate: bool = True, *,
                         input_tensor: torch.Tensor | None = None, weight: torch.Tensor | None = None):
        """`compute_b_params(output, params, grad_output)`: parameter gradients by a second walk over the graph.
        `compute_b_params(input_tensor, grad_output, weight)` is the closed form for a linear layer and returns dL/dW."""
        if input_tensor is not None or (torch.is_tensor(params) and not isinstance(params, nn.Parameter)) \
                or (torch.is_tensor(params) and torch.is_tensor(output) and params.dim() >= 2 and output.dim() >= 2
                    and params.shape[:-1] == output.shape[:-1] and output.grad_fn is None):
            x = input_tensor if input_tensor is not None else output
            go = params if torch.is_tensor(params) else grad_output
            return GradientDecomposer._linear_b_params(x, go, weight)
        ps = [p for p in params if p.requires_grad]
        gs = torch.autograd.grad(output, ps, grad_output, allow_unused=True) if ps else ()
        if accumulate:
            with torch.no_grad():
                for p, g in zip(ps, gs):
                    if g is not None:
                        p.grad = g if p.grad is None else p.grad + g
        return list(gs)


class _StageSplitFunction(torch.autograd.Function):
    """Wraps one stage call inside an outer graph: backward returns only the input gradients and parks the weight
    gradient work (a closure over the retained inner graph) on the stage's queue."""

    @staticmethod
    def forward(ctx, stage: "PipelineStageModule", anchor, *inputs):
        inner_in = [x.detach().requires_grad_(x.requires_grad) if torch.is_tensor(x) else x for x in inputs]
        with torch.enable_grad():
            out = stage.module(*inner_in)
        ctx.stage, ctx.inner_in, ctx.inner_out = stage, inner_in, out
        return out.detach()

    @staticmethod
    def backward(ctx, grad_out):
        stage, out = ctx.stage, ctx.inner_out
        gx = GradientDecomposer.compute_b_input(out, ctx.inner_in, grad_out, retain_graph=True)
        params = [p for p in stage.module.parameters() if p.requires_grad]
        stage._deferred.append(lambda: GradientDecomposer.compute_b_params(out, params, grad_out))
        return (None, None) + tuple(gx)


class SplitBackwardFunction(torch.autograd.Function):
    """One linear layer y = x W^T + b with a split backward: `apply(input_tensor, weight, bias, stage_id, microbatch_id,
    decomposer, memory_manager)`.  Backward returns dL/dx (and the cheap dL/db) at once and returns no dL/dW: input and
    output gradient are left in the memory manager under `stage_<id>_input` / `stage_<id>_grad_output` of the
    micro-batch, for `decomposer.compute_b_params(input, grad_output, weight)` to run in an idle slot
    (data_pipeline/trainer/distributed/zbpp.py:505).  Whole stage modules are split by `PipelineStageModule`."""

    @staticmethod
    def forward(ctx, input_tensor, weight, bias=None, stage_id=0, microbatch_id=0, decomposer=None, memory_manager=None):
        ctx.save_for_backward(input_tensor, weight)
        ctx.has_bias = bias is not None
        ctx.ids, ctx.decomposer, ctx.manager = (stage_id, microbatch_id), decomposer or GradientDecomposer(), memory_manager
        if memory_manager is not None:
            memory_manager.store_activation(microbatch_id=microbatch_id, name=f"stage_{stage_id}_input",
                                            tensor=input_tensor.detach())
        from ..ops import gemm
        return gemm.linear(input_tensor, weight, bias)

    @staticmethod
    def backward(ctx, grad_output):
        x, w = ctx.saved_tensors
        gx = ctx.decomposer.compute_b_input(grad_output, w) if ctx.needs_input_grad[0] else None
        if ctx.manager is not None:
            ctx.manager.store_activation(microbatch_id=ctx.ids[1], name=f"stage_{ctx.ids[0]}_grad_output",
                                         tensor=grad_output.detach())
        gb = grad_output.reshape(-1, grad_output.shape[-1]).sum(0) if ctx.has_bias else None
        return gx, None, gb, None, None, None, None


class PipelineStageModule(nn.Module):
    """A stage whose backward is split: `loss.backward()` through it produces input gradients at once and leaves the
    weight gradients to `execute_deferred_b_params()`."""

    def __init__(self, module: nn.Module, stage_id: int = 0, split_backward: "bool | GradientDecomposer" = True,
                 memory_manager=None, dtype: torch.dtype | None = None, *, decomposer: "GradientDecomposer | None" = None):
        """`PipelineStageModule(module, stage_id, split_backward)`, or the reference's `(module, stage_id, decomposer,
        memory_manager, dtype)`: the memory manager then records each micro-batch's stage input (for
        `forward(input_tensor, microbatch_id)`), `dtype` casts the module
        (data_pipeline/trainer/distributed/zbpp.py:568)."""
        super().__init__()
        if isinstance(split_backward, GradientDecomposer):
            decomposer, split_backward = split_backward, True
        self.module, self.stage_id, self.split_backward = module, stage_id, bool(split_backward)
        self._decomposer, self._memory_manager, self._dtype = decomposer or GradientDecomposer(), memory_manager, dtype
        if dtype is not None:
            self.module.to(dtype)
        self._deferred: list[Callable[[], Any]] = []

    def forward(self, *inputs, input_tensor=None, microbatch_id: int | None = None):
        if input_tensor is not None:
            inputs = (input_tensor,) + inputs
        if len(inputs) == 2 and isinstance(inputs[1], int) and not isinstance(inputs[1], bool) and microbatch_id is None:
            inputs, microbatch_id = inputs[:1], inputs[1]                # (input_tensor, microbatch_id)
        if microbatch_id is not None and self._memory_manager is not None and torch.is_tensor(inputs[0]):
            self._memory_manager.store_activation(microbatch_id=microbatch_id, name=f"stage_{self.stage_id}_input",
                                                  tensor=inputs[0].detach())
        if not (self.split_backward and torch.is_grad_enabled()):
            return self.module(*inputs)
        # the anchor makes autograd visit this node even when no input requires grad (first stage)
        dev = next(self.module.parameters()).device
        return _StageSplitFunction.apply(self, torch.zeros((), requires_grad=True, device=dev), *inputs)

    @property
    def num_deferred(self) -> int:
        return len(self._deferred)

    def execute_deferred_b_params(self, limit: int | None = None) -> int:
        n = len(self._deferred) if limit is None else min(limit, len(self._deferred))
        for _ in range(n):
            self._deferred.pop(0)()
        return n


# ------------------------------------------------------------------------------------------------ optimizer
class ZBPPOptimizer:
    """Per-stage AdamW that does not wait for the other stages ("synchronisation bypass").

    A global gradient-norm clip needs an all-reduce over the stages, which puts a barrier at the end of every step and
    re-creates a bubble.  With the bypass the stage updates optimistically with its LOCAL view (its own gradient norm
    against `max_grad_norm / sqrt(P)`, its own inf/nan check), and `validate()` -- called at the start of the next
    step, when the all-reduced norm has arrived anyway -- rolls the update back and redoes it with the global clip
    factor in the rare step where the global norm exceeds the threshold or another stage saw a non-finite value."""

    def __init__(self, params, lr: float = 1e-4, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 max_grad_norm: float | None = 1.0, num_stages: int = 1, enable_sync_bypass: bool = True, group=None, *,
                 use_triton: bool = False):
        """`use_triton` is accepted and has no effect: the update runs the framework's own fused AdamW kernel."""
        from ..optim import AdamW
        self.params = [p for p in params if p.requires_grad]
        self.inner = AdamW(self.params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        self.param_groups = self.inner.param_groups
        self.max_grad_norm, self.num_stages, self.group = max_grad_norm, max(1, num_stages), group
        self.enable_sync_bypass = enable_sync_bypass
        self._backup: dict | None = None
        self._pending_norm_sq: torch.Tensor | None = None
        self.rollbacks = 0
        self.steps = 0

    def add_param_group(self, param_group) -> None:
        self.inner.add_param_group(param_group)

    def _local_norm_sq(self) -> torch.Tensor:
        gs = [p.grad.float().pow(2).sum() for p in self.params if p.grad is not None]
        return torch.stack(gs).sum() if gs else torch.zeros(())

    def _scale_grads(self, c: float) -> None:
        if c < 1.0:
            for p in self.params:
                if p.grad is not None:
                    p.grad.mul_(c)

    def _all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(t, group=self.group)
        return t

    def step(self, grad_scaler=None) -> bool:
        """Returns False when the step was skipped because of a non-finite local gradient."""
        nsq = self._local_norm_sq()
        if not torch.isfinite(nsq):
            self._pending_norm_sq = None
            self.zero_grad()
            return False
        if not self.enable_sync_bypass:
            total = float(self._all_reduce(nsq.clone()).sqrt())
            if self.max_grad_norm is not None:
                self._scale_grads(min(1.0, self.max_grad_norm / (total + 1e-6)))
            self.inner.step()
            self.steps += 1
            return True
        # optimistic local step; keep what is needed to undo it
        self._backup = {"p": [p.detach().clone() for p in self.params],
                        "g": [None if p.grad is None else p.grad.detach().clone() for p in self.params],
                        "state": {k: ({kk: (vv.clone() if torch.is_tensor(vv) else vv) for kk, vv in v.items()})
                                  for k, v in self.inner.state.items()}}
        if self.max_grad_norm is not None:
            local_cap = self.max_grad_norm / self.num_stages ** 0.5
            self._scale_grads(min(1.0, local_cap / (float(nsq.sqrt()) + 1e-6)))
        self._local_coef = min(1.0, (self.max_grad_norm / self.num_stages ** 0.5) / (float(nsq.sqrt()) + 1e-6)) \
            if self.max_grad_norm is not None else 1.0
        self.inner.step()
        self._pending_norm_sq = nsq
        self.steps += 1
        return True

    def validate(self, global_norm_sq: torch.Tensor | None = None) -> bool:
        """Post-validation of the last optimistic step with the global norm (`global_norm_sq` when the caller has
        already summed the stages, else an all-reduce over `group`).  True = the step stands."""
        if self._pending_norm_sq is None or self._backup is None:
            return True
        total = float((global_norm_sq if global_norm_sq is not None
                       else self._all_reduce(self._pending_norm_sq.clone())).sqrt())
        self._pending_norm_sq = None
        want = 1.0 if self.max_grad_norm is None else min(1.0, self.max_grad_norm / (total + 1e-6))
        ok = torch.isfinite(torch.tensor(total)).item() and abs(want - self._local_coef) < 1e-12
        if ok:
            self._backup = None
            return True
        # undo, then redo with the global factor (or skip when something was non-finite)
        with torch.no_grad():
            for p, old in zip(self.params, self._backup["p"]):
                p.copy_(old)
        self.inner.state.clear()                      # also drops entries that the undone step created
        self.inner.state.update(self._backup["state"])
        if torch.isfinite(torch.tensor(total)).item():
            for p, g in zip(self.params, self._backup["g"]):
                p.grad = None if g is None else g * want
            self.inner.step()
            for p in self.params:
                p.grad = None
        self._backup = None
        self.rollbacks += 1
        return False

    def zero_grad(self) -> None:
        for p in self.params:
            p.grad = None

    def state_dict(self) -> dict[str, Any]:
        return {"inner": self.inner.state_dict(), "steps": self.steps, "rollbacks": self.rollbacks}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        self.inner.load_state_dict(state["inner"])
        self.steps, self.rollbacks = state.get("steps", 0), state.get("rollbacks", 0)


# ------------------------------------------------------------------------------------------------ partitioning
class ModelPartitioner:
    """Cuts a chain of layers into P contiguous stages with the smallest possible heaviest stage (exact dynamic
    programme over prefix sums, O(n^2 P)); cost = parameter count unless measured costs are given."""

    def __init__(self, model: nn.Module | Sequence[nn.Module], num_stages: int,
                 costs: "Sequence[float] | str | None" = None, *, balance_metric: str | None = None):
        """`balance_metric` (when no measured `costs` are given): "params" = parameter count, "flops" = multiply-adds
        per token (2 x the weights of matrix-shaped parameters; vectors cost nothing), "layers" = every layer equal."""
        self.layers = list(model) if isinstance(model, (nn.Sequential, nn.ModuleList, list, tuple)) \
            else list(model.children())
        if len(self.layers) < num_stages:
            raise ValueError(f"{len(self.layers)} layers cannot fill {num_stages} stages")
        self.num_stages = num_stages
        if isinstance(costs, str):                                       # ModelPartitioner(model, num_stages, "flops")
            balance_metric, costs = costs, None
        metric = balance_metric or "params"
        if metric not in ("params", "flops", "layers"):
            raise ValueError(f"balance_metric must be 'params', 'flops' or 'layers', got {metric!r}")
        self.balance_metric = metric
        if costs is not None:
            self.costs = list(costs)
        elif metric == "layers":
            self.costs = [1.0] * len(self.layers)
        elif metric == "flops":
            self.costs = [2.0 * sum(p.numel() for p in l.parameters() if p.dim() >= 2) + 1.0 for l in self.layers]
        else:
            self.costs = [float(sum(p.numel() for p in l.parameters())) + 1.0 for l in self.layers]

    @staticmethod
    def _dp_partition(costs: Sequence[float], k: int) -> list[int]:
        """Boundaries b[0]=0 < b[1] < ... < b[k]=n minimising max_j sum(costs[b[j]:b[j+1]])."""
        n = len(costs)
        pre = [0.0]
        for c in costs:
            pre.append(pre[-1] + c)
        INF = float("inf")
        best = [[INF] * (n + 1) for _ in range(k + 1)]
        cut = [[0] * (n + 1) for _ in range(k + 1)]
        best[0][0] = 0.0
        for j in range(1, k + 1):
            for i in range(j, n - (k - j) + 1):
                for m in range(j - 1, i):
                    v = max(best[j - 1][m], pre[i] - pre[m])
                    if v < best[j][i]:
                        best[j][i], cut[j][i] = v, m
        bounds, i = [n], n
        for j in range(k, 0, -1):
            i = cut[j][i]
            bounds.append(i)
        return bounds[::-1]

    def boundaries(self) -> list[int]:
        return self._dp_partition(self.costs, self.num_stages)

    def partition(self) -> list[nn.Sequential]:
        b = self.boundaries()
        return [nn.Sequential(*self.layers[b[j]:b[j + 1]]) for j in range(self.num_stages)]


# ------------------------------------------------------------------------------------------------ runtime
class _OptimizedSchedule(PL.PipelineSchedule):
    """Executor of `parallel/pipeline.py` driven by a ScheduleResult instead of a closed-form order."""
    schedule_name = "zero_bubble"

    def __init__(self, result: ScheduleResult, *a, **kw):
        super().__init__(*a, **kw)
        self._acts = result.actions()

    def actions(self):
        return self._acts


class ZBPPRuntimeEngine:
    """Profiles the stages, builds the schedule, runs training steps.  `stages`: every stage (one process) or this
    rank's stage (with a `ctx` spanning the pipeline ranks)."""

    def __init__(self, stages: Sequence[nn.Module] | None = None, num_microbatches: "int | ScheduleConfig | None" = None,
                 loss_fn: "Callable | ZBPPOptimizer | None" = None, num_stages: int | None = None,
                 memory_limit_bytes: int = 4 * 2 ** 30, optimizer_factory: Callable | None = None,
                 enable_sync_bypass: bool = True, ctx: PL.DistributedContext | None = None,
                 stage_profiles: Sequence[StageProfile] | None = None, enable_interleaving: bool = True, *,
                 stage_modules: Sequence[nn.Module] | None = None, schedule_config: ScheduleConfig | None = None,
                 optimizer: "ZBPPOptimizer | None" = None, rank: int | None = None, world_size: int | None = None,
                 device=None, dtype: torch.dtype | None = None, grad_scaler=None):
        """`ZBPPRuntimeEngine(stages, num_microbatches, loss_fn, ...)`, or the reference's `(stage_modules,
        schedule_config, optimizer, rank, world_size, device, dtype, grad_scaler)`: sizes, memory limit and stage
        profiles then come from the `ScheduleConfig`, the one optimizer steps after every `train_step`, the loss function
        arrives with `train_step(micro_batches, labels, loss_fn)`, and with `world_size > 1` the pipeline spans the
        default process group (data_pipeline/trainer/distributed/zbpp.py:1356)."""
        stages = stage_modules if stage_modules is not None else stages
        if isinstance(num_microbatches, ScheduleConfig):                 # positional reference form
            ref = (num_microbatches, loss_fn, num_stages, memory_limit_bytes, optimizer_factory)
            schedule_config, optimizer = ref[0], ref[1]
            rank = ref[2] if rank is None and isinstance(ref[2], int) else rank
            world_size = ref[3] if world_size is None and ref[3] != 4 * 2 ** 30 else world_size
            device = ref[4] if device is None else device
            loss_fn, num_stages, memory_limit_bytes, optimizer_factory = None, None, 4 * 2 ** 30, None
        self.grad_scaler, self.dtype, self.device = grad_scaler, dtype, device
        self._single_optimizer = optimizer
        self._reference_form = schedule_config is not None
        if schedule_config is not None:
            num_stages, num_microbatches = schedule_config.num_stages, schedule_config.num_microbatches
            memory_limit_bytes = schedule_config.memory_limit_bytes
            stage_profiles = schedule_config.stage_profiles
            enable_sync_bypass, enable_interleaving = schedule_config.enable_sync_bypass, schedule_config.enable_interleaving
            # the engine splits the backward itself: a stage that splits its own would leave its weight gradients parked
            stages = [m.module if isinstance(m, PipelineStageModule) else m for m in stages]
            if device is not None or dtype is not None:
                stages = [m.to(device=device, dtype=dtype) for m in stages]
            if (world_size or 1) > 1 and ctx is None:
                ctx = PL.DistributedContext(ranks=list(range(world_size)))
        self.ctx = ctx or PL.DistributedContext()
        self.num_stages = num_stages or len(stages)
        self.num_microbatches = num_microbatches
        self.memory_limit_bytes = memory_limit_bytes
        self.enable_sync_bypass, self.enable_interleaving = enable_sync_bypass, enable_interleaving
        self.stages = [m if isinstance(m, PL.PipelineStage) else PL.PipelineStage(m, i, self.num_stages)
                       for i, m in enumerate(stages)]
        self.loss_fn = self._ctor_loss_fn = loss_fn
        self.stage_profiles = list(stage_profiles) if stage_profiles is not None else None
        self.optimizers = [optimizer_factory(st.parameters()) for st in self.stages] if optimizer_factory else []
        if self._single_optimizer is not None:
            self.optimizers = [self._single_optimizer]
        self.step_times: list[float] = []
        self._result: ScheduleResult | None = None
        self._schedule: _OptimizedSchedule | None = None
        self.steps = 0

    def _default_profiles(self) -> list[StageProfile]:
        out = []
        for _ in range(self.num_stages):
            out.append(StageProfile(100.0, 100.0, 100.0, 1, 0, 0.0, 0.0))
        if len(self.stages) == self.num_stages:          # all stages here: weight costs by parameter count
            n = [max(1, sum(p.numel() for p in st.parameters())) for st in self.stages]
            mean = sum(n) / len(n)
            out = [StageProfile(100.0 * k / mean, 100.0 * k / mean, 100.0 * k / mean, 1,
                                sum(p.numel() * p.element_size() for p in st.parameters()), 0.0, 0.0)
                   for k, st in zip(n, self.stages)]
        return out

    def profile_stage(self, stage_index: "int | torch.Tensor" = 0, sample_input: torch.Tensor | None = None,
                      repeats: int = 3, *, num_warmup: int | None = None, num_iterations: int | None = None) -> StageProfile:
        """Wall-clock forward / B_input / B_params of one local stage on `sample_input` (CUDA-synchronised).
        `profile_stage(sample_input, num_warmup, num_iterations)` measures the first local stage."""
        if torch.is_tensor(stage_index):                                 # (sample_input, num_warmup, num_iterations)
            if sample_input is not None and num_warmup is None:
                num_warmup = int(sample_input)
                if repeats != 3 and num_iterations is None:
                    num_iterations = repeats
            stage_index, sample_input = 0, stage_index
        repeats = int(num_iterations) if num_iterations is not None else repeats
        warm = max(1, int(num_warmup)) if num_warmup is not None else 1
        st = self.stages[stage_index]
        dev = st.device
        x = sample_input.to(dev)
        if x.is_floating_point():
            x = x.detach().requires_grad_(True)

        def sync():
            if dev.type == "cuda":
                torch.cuda.synchronize(dev)

        tf = tb = tw = 0.0
        act_bytes = 0
        params = [p for p in st.parameters() if p.requires_grad]
        for i in range(repeats + warm):
            sync()
            t0 = time.perf_counter()
            y = st(x)
            sync()
            t1 = time.perf_counter()
            g = torch.ones_like(y)
            if x.requires_grad:
                torch.autograd.grad(y, [x], g, retain_graph=True)
            sync()
            t2 = time.perf_counter()
            torch.autograd.grad(y, params, g, allow_unused=True)
            sync()
            t3 = time.perf_counter()
            if i >= warm:                              # the first passes are warm-up
                tf, tb, tw = tf + (t1 - t0), tb + (t2 - t1), tw + (t3 - t2)
            act_bytes = y.numel() * y.element_size() + x.numel() * x.element_size()
        k = 1e6 / repeats
        return StageProfile(tf * k, max(tb * k, 1.0), max(tw * k, 1.0), act_bytes,
                            sum(p.numel() * p.element_size() for p in st.parameters()))

    def generate_schedule(self) -> ScheduleResult:
        prof = self.stage_profiles or self._default_profiles()
        cfg = ScheduleConfig(self.num_stages, self.num_microbatches, self.memory_limit_bytes, prof,
                             self.enable_sync_bypass, self.enable_interleaving)
        self._result = ZBPPScheduleOptimizer(cfg).optimize()
        pc = PL.PipelineConfig(num_stages=self.num_stages, num_microbatches=self.num_microbatches,
                               schedule=PL.ScheduleType.ZERO_BUBBLE)
        comm = PL.P2PCommunicator(self.ctx, self.stages[0].device) if self.ctx.is_distributed else None
        self._schedule = _OptimizedSchedule(self._result, self.stages, pc, self.loss_fn, comm, None, self.ctx)
        return self._result

    def train_step(self, input_batches: Sequence[torch.Tensor] | None = None,
                   target_batches: Sequence[torch.Tensor] | None = None, loss_fn: Callable | None = None, *,
                   micro_batches: Sequence[torch.Tensor] | None = None, labels: Sequence[torch.Tensor] | None = None):
        """`train_step(input_batches, target_batches)` -> loss.  The reference's `train_step(micro_batches, labels,
        loss_fn)` -> {"loss", "step_time_s", "throughput_samples_per_s", "bubble_fraction"}; without labels the loss
        function is called with the output alone."""
        reference_form = micro_batches is not None or labels is not None or loss_fn is not None or self._reference_form
        if micro_batches is not None:
            input_batches = micro_batches
        if labels is not None:
            target_batches = labels
        if reference_form:
            if len(input_batches) != self.num_microbatches:
                raise ValueError(f"expected {self.num_microbatches} micro-batches, got {len(input_batches)}")
            fn = loss_fn or self.loss_fn
            if fn is None:
                raise TypeError("a loss function is required: train_step(micro_batches, labels, loss_fn)")
            if target_batches is None:
                target_batches = [torch.zeros((), device=b.device) for b in input_batches]
                fn = (lambda f: lambda out, _unused: f(out))(fn)
            self.loss_fn = fn
            if self._schedule is not None:
                self._schedule.loss_fn = fn
        elif self.loss_fn is not self._ctor_loss_fn:     # a loss function passed to one step does not outlive it
            self.loss_fn = self._ctor_loss_fn
            if self._schedule is not None:
                self._schedule.loss_fn = self.loss_fn
        t0 = time.perf_counter()
        if self._schedule is None:
            self.generate_schedule()
        self.validate_pending()                          # settle last step's optimistic updates first
        loss = self._schedule.run(input_batches, target_batches)
        for opt in self.optimizers:
            opt.step()
            opt.zero_grad()
        self.steps += 1
        if not reference_form:
            return loss
        value = float(loss.detach()) if torch.is_tensor(loss) else float(loss)    # reading the loss waits for the device
        dt = time.perf_counter() - t0
        self.step_times.append(dt)
        n = sum(int(b.shape[0]) for b in input_batches)
        return {"loss": value, "step_time_s": dt, "throughput_samples_per_s": n / dt if dt > 0 else 0.0,
                "bubble_fraction": self._result.bubble_fraction if self._result is not None else 0.0}

    def validate_pending(self) -> int:
        """Global-norm check of the optimistic updates of the previous step: the local stages' squared norms are summed
        here and all-reduced over the pipeline group.  Returns the number of stage updates that were redone."""
        opts = [o for o in self.optimizers if getattr(o, "_pending_norm_sq", None) is not None]
        if not opts:
            return 0
        tot = torch.stack([o._pending_norm_sq.float().cpu() for o in opts]).sum()
        if self.ctx.is_distributed:
            dev = self.stages[0].device
            tot = tot.to(dev)
            dist.all_reduce(tot, group=self.ctx.group)
            tot = tot.cpu()
        return sum(0 if o.validate(tot) else 1 for o in opts)

    @property
    def schedule_result(self) -> ScheduleResult | None:
        return self._result


class ZeroBubblePipeline:
    """Model in, training steps out: partition -> (profile) -> schedule -> run.  In one process it holds every stage
    (on `devices`, or the model's device); with `world_size > 1` each rank keeps stage `rank` and a pipeline group over
    all ranks must exist (`torch.distributed` initialised)."""

    def __init__(self, model: nn.Module, num_stages: int = 4, num_microbatches: int = 8,
                 memory_limit_bytes: int = 4 * 2 ** 30, lr: float = 1e-4, weight_decay: float = 0.01,
                 dtype: torch.dtype | None = None, use_triton: bool = False, enable_sync_bypass: bool = True,
                 rank: int = 0, world_size: int = 1, loss_fn: Callable | None = None,
                 max_grad_norm: float | None = 1.0, costs: Sequence[float] | None = None,
                 devices: Sequence[torch.device | str] | None = None):
        self.num_stages, self.num_microbatches = num_stages, num_microbatches
        self.rank, self.world_size = rank, world_size
        parts = ModelPartitioner(model, num_stages, costs).partition()
        if dtype is not None:
            parts = [p.to(dtype) for p in parts]
        if devices is not None:
            parts = [p.to(devices[i % len(devices)]) for i, p in enumerate(parts)]
        distributed = world_size > 1
        ctx = PL.DistributedContext(ranks=list(range(world_size))) if distributed else PL.DistributedContext()
        mine = [PL.PipelineStage(parts[rank], rank, num_stages)] if distributed else \
            [PL.PipelineStage(p, i, num_stages) for i, p in enumerate(parts)]
        self.loss_fn = loss_fn or nn.functional.mse_loss
        self.engine = ZBPPRuntimeEngine(
            mine, num_microbatches, self.loss_fn, num_stages, memory_limit_bytes,
            lambda ps: ZBPPOptimizer(ps, lr=lr, weight_decay=weight_decay, max_grad_norm=max_grad_norm,
                                     num_stages=num_stages, enable_sync_bypass=enable_sync_bypass,
                                     group=ctx.group if distributed else None),
            enable_sync_bypass, ctx)
        self.stages = mine

    def train_step(self, inputs: "torch.Tensor | Sequence[torch.Tensor] | None" = None,
                   targets: "torch.Tensor | Sequence[torch.Tensor] | None" = None, loss_fn: Callable | None = None, *,
                   micro_batches=None, labels=None):
        """`train_step(inputs, targets)` -> loss (whole batches are cut into the micro-batches).  The reference's
        `train_step(micro_batches, labels, loss_fn)` -> metrics dict, like the engine's."""
        if micro_batches is not None or labels is not None or loss_fn is not None:
            return self.engine.train_step(micro_batches=micro_batches if micro_batches is not None else inputs,
                                          labels=labels if labels is not None else targets, loss_fn=loss_fn or self.loss_fn)
        if torch.is_tensor(inputs):
            inputs = list(inputs.chunk(self.num_microbatches, dim=0))
        if torch.is_tensor(targets):
            targets = list(targets.chunk(self.num_microbatches, dim=0))
        return self.engine.train_step(inputs, targets)

    @reference_kwargs(num_iterations="repeats")
    def profile_stages(self, sample_input: torch.Tensor, repeats: int = 3, *, num_warmup: int | None = None) -> list[StageProfile]:
        """Measures every local stage on a sample micro-batch (chained through the stages) and rebuilds the schedule
        with the measured costs (single-process layout)."""
        profs, x = [], sample_input
        for i, st in enumerate(self.engine.stages):
            profs.append(self.engine.profile_stage(i, x, repeats, num_warmup=num_warmup))
            with torch.no_grad():
                x = st(x.to(st.device))
        if len(profs) == self.num_stages:
            self.engine.stage_profiles = profs
            self.engine.generate_schedule()
        return profs

    @property
    def schedule_result(self) -> ScheduleResult | None:
        return self.engine.schedule_result

    @property
    def bubble_fraction(self) -> float:
        if self.engine.schedule_result is None:
            self.engine.generate_schedule()
        return self.engine.schedule_result.bubble_fraction

    def finalize(self) -> int:
        """Settle the optimistic update of the last step (call before evaluating or saving)."""
        return self.engine.validate_pending()

    def parameters(self):
        for st in self.stages:
            yield from st.parameters()

    def state_dict(self) -> dict[str, Any]:
        self.finalize()
        return {"stages": {st.stage_id: st.state_dict() for st in self.stages},
                "optimizers": {st.stage_id: o.state_dict() for st, o in zip(self.stages, self.engine.optimizers)},
                "steps": self.engine.steps}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        for st, o in zip(self.stages, self.engine.optimizers):
            st.load_state_dict(state["stages"][st.stage_id])
            o.load_state_dict(state["optimizers"][st.stage_id])
        self.engine.steps = state.get("steps", 0)


class ZBPPBenchmark:
    """Self-checks: the gradient split equals a plain backward, the schedule beats 1F1B and respects the memory limit,
    and a throughput measurement."""

    def __init__(self, pipeline: "ZeroBubblePipeline | torch.device | str | None" = None,
                 sample_input: "torch.Tensor | torch.dtype | None" = None, sample_target: torch.Tensor | None = None, *,
                 device=None, dtype: torch.dtype | None = None):
        """`ZBPPBenchmark(pipeline, sample_input, sample_target)` checks that pipeline.  The reference's
        `ZBPPBenchmark(device, dtype)` is free-standing: each check builds what it needs from the sizes it is given and
        returns a bool (data_pipeline/trainer/distributed/zbpp.py:1943)."""
        if not isinstance(pipeline, ZeroBubblePipeline) and pipeline is not None:
            device, pipeline = pipeline, None
            if isinstance(sample_input, torch.dtype):
                dtype, sample_input = sample_input, None
        self.pipeline, self.x, self.y = pipeline, sample_input, sample_target
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.dtype = dtype or torch.float32

    # ---- free-standing checks
    def _linear_decomposition(self, batch_size: int, in_features: int, out_features: int, atol: float, rtol: float) -> bool:
        g = torch.Generator().manual_seed(0)
        x = torch.randn(batch_size, in_features, generator=g).to(self.device, self.dtype).requires_grad_(True)
        w = (torch.randn(out_features, in_features, generator=g) / in_features ** 0.5).to(self.device, self.dtype).requires_grad_(True)
        go = torch.randn(batch_size, out_features, generator=g).to(self.device, self.dtype)
        want_x, want_w = torch.autograd.grad(nn.functional.linear(x.float(), w.float()), [x, w], go.float())
        d = GradientDecomposer(dtype=self.dtype)
        got_x = d.compute_b_input(go, w.detach())
        got_w = d.compute_b_params(x.detach(), go, w.detach())
        return bool(torch.allclose(got_x.float(), want_x.float(), atol=atol, rtol=rtol)
                    and torch.allclose(got_w.float(), want_w.float(), atol=atol, rtol=rtol))

    @staticmethod
    def _uniform_schedule(num_stages: int, num_microbatches: int, memory_limit_bytes: int, activation_bytes: int = 1 << 20):
        prof = [StageProfile(100.0, 100.0, 100.0, activation_bytes, 0, 0.0, 0.0) for _ in range(num_stages)]
        return ZBPPScheduleOptimizer(ScheduleConfig(num_stages, num_microbatches, memory_limit_bytes, prof)).optimize()

    def validate_gradient_decomposition(self, batch_size: "int | float | None" = None, in_features: int = 512,
                                        out_features: int = 256, atol: float | None = None, rtol: float = 1e-2):
        """With a pipeline: its first stage's split backward against a plain backward -> dict.  Free-standing
        (`batch_size, in_features, out_features, atol, rtol`): the closed forms of a linear layer against autograd -> bool."""
        if self.pipeline is None:
            return self._linear_decomposition(int(batch_size or 32), in_features, out_features,
                                              1e-2 if atol is None else atol, rtol)
        if isinstance(batch_size, float) and atol is None:               # validate_gradient_decomposition(1e-5)
            atol = batch_size
        atol = 1e-5 if atol is None else atol
        st = self.pipeline.stages[0]
        x = self.x[: max(1, self.x.shape[0] // self.pipeline.num_microbatches)].to(st.device)
        if x.is_floating_point():
            x = x.detach().requires_grad_(True)
        params = [p for p in st.parameters() if p.requires_grad]
        y = st(x)
        g = torch.randn_like(y)
        want = torch.autograd.grad(y, ([x] if x.requires_grad else []) + params, g, retain_graph=True, allow_unused=True)
        gx = GradientDecomposer.compute_b_input(y, [x], g)
        gp = GradientDecomposer.compute_b_params(y, params, g, accumulate=False)
        got = ([gx[0]] if x.requires_grad else []) + gp
        err = max((float((a - b).abs().max()) for a, b in zip(got, want) if a is not None and b is not None), default=0.0)
        return {"max_abs_error": err, "passed": err <= atol}

    def validate_schedule_optimality(self, num_stages: int | None = None, num_microbatches: int | None = None):
        if self.pipeline is None:
            P, M = int(num_stages or 4), int(num_microbatches or 8)
            r = self._uniform_schedule(P, M, 1 << 40)
            base = PP.simulate([PP.one_f_one_b_schedule(s, P, M) for s in range(P)])["bubble_fraction"]
            return bool(r.bubble_fraction <= base + 1e-9)
        r = self.pipeline.schedule_result or self.pipeline.engine.generate_schedule()
        P, M = self.pipeline.num_stages, self.pipeline.num_microbatches
        base = PP.simulate([PP.one_f_one_b_schedule(s, P, M) for s in range(P)])["bubble_fraction"]
        return {"bubble_fraction": r.bubble_fraction, "one_f_one_b_bubble": base,
                "passed": r.bubble_fraction <= base + 1e-9}

    def validate_memory_compliance(self, num_stages: int | None = None, num_microbatches: int | None = None,
                                   memory_limit_mb: int = 256):
        if self.pipeline is None:
            lim = int(memory_limit_mb) * 2 ** 20
            r = self._uniform_schedule(int(num_stages or 4), int(num_microbatches or 8), lim, activation_bytes=lim // 16)
            return bool(all(v <= lim for v in r.peak_memory_bytes.values()))
        r = self.pipeline.schedule_result or self.pipeline.engine.generate_schedule()
        lim = self.pipeline.engine.memory_limit_bytes
        return {"peak_memory_bytes": r.peak_memory_bytes, "limit": lim,
                "passed": all(v <= lim for v in r.peak_memory_bytes.values())}

    def _free_standing_throughput(self, model, num_stages, num_microbatches, batch_size, seq_len, hidden_dim, num_steps):
        if model is None:
            model = nn.Sequential(*[nn.Sequential(nn.Linear(hidden_dim, hidden_dim), nn.GELU()) for _ in range(2 * num_stages)])
        model = model.to(self.device, self.dtype)
        pipe = ZeroBubblePipeline(model, num_stages, num_microbatches)
        x = torch.randn(batch_size * num_microbatches, seq_len, hidden_dim, device=self.device, dtype=self.dtype)
        y = torch.randn_like(x)
        pipe.train_step(x, y)                                            # warm-up
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        t0 = time.perf_counter()
        for _ in range(num_steps):
            loss = pipe.train_step(x, y)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        dt = (time.perf_counter() - t0) / max(1, num_steps)
        return {"step_ms": dt * 1e3, "samples_per_s": x.shape[0] / dt, "tokens_per_s": x.shape[0] * seq_len / dt,
                "bubble_fraction": pipe.bubble_fraction, "final_loss": float(loss)}

    def benchmark_throughput(self, steps: "int | nn.Module | None" = 3, warmup: int = 1, *, model: nn.Module | None = None,
                             num_stages: int = 4, num_microbatches: int = 8, batch_size: int = 4, seq_len: int = 128,
                             hidden_dim: int = 512, num_steps: int | None = None) -> dict[str, Any]:
        """With a pipeline: `steps` timed steps of it.  Free-standing: builds (or takes) a model of `hidden_dim`, cuts it
        into `num_stages` and times `num_steps` steps on [batch_size * num_microbatches, seq_len, hidden_dim]."""
        if self.pipeline is None:
            if isinstance(steps, nn.Module):
                model = steps
            return self._free_standing_throughput(model, num_stages, num_microbatches, batch_size, seq_len, hidden_dim,
                                                  int(num_steps if num_steps is not None else 5))
        steps = int(num_steps) if num_steps is not None else steps
        dev = self.pipeline.stages[0].device
        for _ in range(warmup):
            self.pipeline.train_step(self.x, self.y)
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        for _ in range(steps):
            self.pipeline.train_step(self.x, self.y)
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)
        dt = (time.perf_counter() - t0) / steps
        return {"step_ms": dt * 1e3, "samples_per_s": self.x.shape[0] / dt}

    def run_all(self) -> dict[str, Any]:
        if self.pipeline is None:
            out = {"gradient_decomposition": {"passed": self.validate_gradient_decomposition()},
                   "schedule": {"passed": self.validate_schedule_optimality()},
                   "memory": {"passed": self.validate_memory_compliance()},
                   "throughput": self.benchmark_throughput(hidden_dim=64, seq_len=16, num_steps=2)}
            out["passed"] = all(v.get("passed", True) for v in out.values())
            return out
        out = {"gradient_decomposition": self.validate_gradient_decomposition(),
               "schedule": self.validate_schedule_optimality(), "memory": self.validate_memory_compliance(),
               "throughput": self.benchmark_throughput()}
        out["passed"] = all(v.get("passed", True) for v in out.values() if isinstance(v, dict))
        return out


def create_zbpp_pipeline(model: nn.Module, num_stages: int = 4, num_microbatches: int = 8, memory_limit_gb: float = 4.0,
                         lr: float = 1e-4, weight_decay: float = 0.01, dtype: torch.dtype | None = None,
                         use_triton: bool = False, enable_sync_bypass: bool = True, rank: int = 0, world_size: int = 1,
                         **kw) -> ZeroBubblePipeline:
    return ZeroBubblePipeline(model, num_stages, num_microbatches, int(memory_limit_gb * 2 ** 30), lr, weight_decay,
                              dtype, use_triton, enable_sync_bypass, rank, world_size, **kw)


CudaEvent = torch.cuda.Event               # name used by data_pipeline/trainer/distributed/zbpp.py
