"""Device-side mixture-of-experts dataflow: routing plan, permute, grouped expert GEMMs, weighted combine.

Tokens are sorted by expert into a buffer whose per-expert segments start on 128-row boundaries (pad rows are zero), so
one persistent tcgen05 GEMM launch serves all experts (`ts_gemm_grouped_bf16`): every 128-row tile reads the weight
slab of its expert.  Nothing here synchronises with the host: buffer sizes use the static upper bound
`ts_moe_padded_rows(n, E)`.

Reference: data_pipeline/trainer/kernels/moe_kernels.py:219-785 (grouped GEMM, permute, top-k weighting) with the
per-expert loop of :1183 as the oracle.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib, activation

_c = ctypes


@dataclass
class MoEPlan:
    n: int                    # routed slots (tokens * top_k)
    k: int
    E: int
    P: int                    # rows of the padded expert-sorted buffer (static upper bound)
    counts: torch.Tensor      # [E] int32
    seg_start: torch.Tensor   # [E + 1] int32, multiples of 128
    tile_expert: torch.Tensor  # [P / 128] int32, -1 for unused tiles
    dest: torch.Tensor        # [n] int32: row of slot i
    src_of_row: torch.Tensor  # [P] int32: slot of row r or -1


def available(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0


def make_plan(expert_ids: torch.Tensor, num_experts: int) -> MoEPlan:
    """expert_ids [T, k] (any integer dtype) -> routing plan; stable order inside every expert."""
    lib = _lib.load("moe")
    T, k = expert_ids.shape
    ids = expert_ids.reshape(-1).to(torch.int32).contiguous()
    n, E = ids.numel(), int(num_experts)
    P = int(lib.ts_moe_padded_rows(n, E))
    dev = ids.device
    i32 = dict(dtype=torch.int32, device=dev)
    rank, counts, seg = torch.empty(n, **i32), torch.empty(E, **i32), torch.empty(E + 1, **i32)
    tile_expert, dest, src = torch.empty(P // 128, **i32), torch.empty(n, **i32), torch.empty(P, **i32)
    rc = lib.ts_moe_plan(_lib.ptr(ids), n, E, _lib.ptr(rank), _lib.ptr(counts), _lib.ptr(seg), _lib.ptr(tile_expert),
                         _lib.ptr(dest), _lib.ptr(src), _lib.stream_ptr())
    _lib.check(rc, "ts_moe_plan")
    return MoEPlan(n, k, E, P, counts, seg, tile_expert, dest, src)


def _permute_raw(x2, plan: MoEPlan, slot_scale=None):
    lib = _lib.load("moe")
    out = torch.empty(plan.P, x2.shape[1], dtype=x2.dtype, device=x2.device)
    rc = lib.ts_moe_permute(_lib.ptr(x2), _lib.ptr(plan.src_of_row), _lib.ptr(slot_scale), _lib.ptr(out), plan.P,
                            x2.shape[1], plan.k, _lib.stream_ptr())
    _lib.check(rc, "ts_moe_permute")
    return out


def _combine_raw(y, plan: MoEPlan, w=None):
    lib = _lib.load("moe")
    T = plan.n // plan.k
    out = torch.empty(T, y.shape[1], dtype=y.dtype, device=y.device)
    rc = lib.ts_moe_combine(_lib.ptr(y), _lib.ptr(plan.dest), _lib.ptr(w), _lib.ptr(out), T, y.shape[1], plan.k,
                            _lib.stream_ptr())
    _lib.check(rc, "ts_moe_combine")
    return out


class _PermuteFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, plan):
        ctx.plan = plan
        return _permute_raw(x2.contiguous(), plan)

    @staticmethod
    def backward(ctx, dxp):
        return _combine_raw(dxp.contiguous(), ctx.plan), None


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, w, plan):
        wf = w.reshape(-1).float().contiguous()
        ctx.save_for_backward(y, wf)
        ctx.plan, ctx.w_dtype, ctx.w_shape = plan, w.dtype, w.shape
        return _combine_raw(y.contiguous(), plan, wf)

    @staticmethod
    def backward(ctx, dout):
        lib = _lib.load("moe")
        y, wf = ctx.saved_tensors
        plan = ctx.plan
        dout = dout.contiguous()
        dy = _permute_raw(dout, plan, wf)                         # dy[dest(t, j)] = w[t, j] * dout[t]; pad rows zero
        dw = torch.empty(plan.n, dtype=torch.float32, device=y.device)
        rc = lib.ts_moe_combine_dw(_lib.ptr(dout), _lib.ptr(y), _lib.ptr(plan.dest), _lib.ptr(dw), plan.n, y.shape[1],
                                   plan.k, _lib.stream_ptr())
        _lib.check(rc, "ts_moe_combine_dw")
        return dy, dw.view(ctx.w_shape).to(ctx.w_dtype), None


def _grouped(mode, A, B, out, M, N, K, lda, ldb, ldc, a_mn, b_mn, accumulate, groups, E):
    lib = _lib.load("gemm")
    rc = lib.ts_gemm_grouped_bf16(_lib.ptr(A), _lib.ptr(B), _lib.ptr(out), mode, M, N, K, lda, ldb, ldc, int(a_mn),
                                  int(b_mn), int(out.dtype == torch.float32), int(accumulate), _c.c_float(1.0),
                                  _lib.ptr(groups), E, _lib.stream_ptr())
    _lib.check(rc, "ts_gemm_grouped_bf16")
    _lib.LAUNCHES += 1


class _GroupedLinearFn(torch.autograd.Function):
    """y[r] = x[r] @ W[e(r)]^T on the padded expert-sorted buffer; W is [E, N, K]."""

    @staticmethod
    def forward(ctx, xp, W, plan):
        E, N, K = W.shape
        y = torch.empty(plan.P, N, dtype=xp.dtype, device=xp.device)
        _grouped(1, xp, W, y, plan.P, N, K, K, K, N, False, False, False, plan.tile_expert, E)
        # rows of unused tiles (tile_expert == -1) are never written nor read back by the combine
        ctx.save_for_backward(xp, W)
        ctx.plan = plan
        return y

    @staticmethod
    def backward(ctx, dy):
        xp, W = ctx.saved_tensors
        plan = ctx.plan
        E, N, K = W.shape
        dy = dy.contiguous()
        dx = dW = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(xp)
            # dx[r] = dy[r] @ W[e]: B = W stacked along the reduction axis ([E*N][K], N-contiguous rows are K wide)
            _grouped(1, dy, W, dx, plan.P, K, N, N, K, K, False, True, False, plan.tile_expert, E)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(W, "main_grad", None)
            if main_grad is not None:
                tgt, acc = main_grad.view(W.shape), bool(getattr(W, "grad_added", False))
                W.grad_added = True
            else:
                tgt, acc = torch.empty_like(W), False
            # dW[e] = dy_seg^T @ x_seg, reduced over the expert's row segment
            _grouped(2, dy, xp, tgt, N, K, plan.P, N, K, K, True, True, acc, plan.seg_start, E)
            dW = None if main_grad is not None else tgt
        return dx, dW, None


def grouped_linear(xp: torch.Tensor, W: torch.Tensor, plan: MoEPlan) -> torch.Tensor:
    return _GroupedLinearFn.apply(xp, W, plan)


def moe_ffn(x2: torch.Tensor, expert_ids: torch.Tensor, weights: torch.Tensor, w_gate_up: torch.Tensor,
            w_down: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """Top-k expert feed-forward: out[t] = sum_j weights[t, j] * FFN_{ids[t, j]}(x2[t]).
    w_gate_up [E, 2I, H], w_down [E, H, I]."""
    plan = make_plan(expert_ids, w_gate_up.shape[0])
    xp = _PermuteFn.apply(x2, plan)
    h = grouped_linear(xp, w_gate_up, plan)
    h = activation.glu(h, act)
    y = grouped_linear(h, w_down, plan)
    return _CombineFn.apply(y, weights, plan)


def moe_ffn_reference(x2: torch.Tensor, expert_ids: torch.Tensor, weights: torch.Tensor, w_gate_up: torch.Tensor,
                      w_down: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """Same result as `moe_ffn` by a loop over the experts (fp32 accumulation); differentiable.  CPU / non-bf16 path."""
    out = torch.zeros(x2.shape, dtype=torch.float32, device=x2.device)
    for e in range(w_gate_up.shape[0]):
        tok, slot = (expert_ids == e).nonzero(as_tuple=True)
        if tok.numel():
            h = activation.glu(x2[tok].float() @ w_gate_up[e].float().t(), act)
            out = out.index_add(0, tok, (h @ w_down[e].float().t()) * weights[tok, slot].float().unsqueeze(1))
    return out.to(x2.dtype)


class _TopKSoftmaxFn(torch.autograd.Function):
    """Router softmax + top-k on the device kernel; the (small, [T, E]) backward is written with torch ops."""

    @staticmethod
    def forward(ctx, logits, k, normalize):
        lib = _lib.load("moe")
        T, E = logits.shape
        lg = logits.float().contiguous()
        probs = torch.empty_like(lg)
        w = torch.empty(T, k, dtype=torch.float32, device=lg.device)
        idx = torch.empty(T, k, dtype=torch.int32, device=lg.device)
        rc = lib.ts_moe_topk_softmax(_lib.ptr(lg), _lib.ptr(probs), _lib.ptr(w), _lib.ptr(idx), T, E, int(k),
                                     int(bool(normalize)), _lib.stream_ptr())
        _lib.check(rc, "ts_moe_topk_softmax")
        idx64 = idx.long()
        ctx.save_for_backward(probs, w, idx64)
        ctx.normalize, ctx.in_dtype = bool(normalize), logits.dtype
        ctx.mark_non_differentiable(idx64)
        return w, idx64, probs

    @staticmethod
    def backward(ctx, dw, _didx, dprobs):
        probs, w, idx = ctx.saved_tensors
        dp = torch.zeros_like(probs) if dprobs is None else dprobs.float().clone()
        if dw is not None:
            dw = dw.float()
            if ctx.normalize:
                raw = probs.gather(1, idx)
                s = raw.sum(-1, keepdim=True).clamp(min=1e-9)
                dsel = (dw - (dw * w).sum(-1, keepdim=True)) / s
            else:
                dsel = dw
            dp.scatter_add_(1, idx, dsel)
        dlogits = probs * (dp - (dp * probs).sum(-1, keepdim=True))
        return dlogits.to(ctx.in_dtype), None, None


def topk_softmax(logits: torch.Tensor, k: int, normalize: bool = True):
    """(weights [T, k] fp32, experts [T, k] int64, probs [T, E] fp32) of the router logits."""
    if logits.is_cuda and logits.shape[1] <= 1024 and k <= 32:
        return _TopKSoftmaxFn.apply(logits, k, normalize)
    probs = torch.softmax(logits.float(), dim=-1)
    w, idx = probs.topk(k, dim=-1)
    if normalize:
        w = w / w.sum(-1, keepdim=True).clamp(min=1e-9)
    return w, idx, probs
