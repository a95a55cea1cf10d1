"""bf16 tensor-core GEMM (tcgen05 + TMEM + TMA) and the autograd linear built on it.

`gemm(a, b, ...)` computes ``alpha * a @ b.T`` style products for every operand layout the training
step needs, so a linear layer's forward, dgrad and wgrad are three launches of the same kernel with
no transpose copies.  Replaces `F.linear` on the reference's hot path
(data_pipeline/trainer/distributed/tensor_parallel.py:1061,1214).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_c = ctypes


def _use_cuda(*ts: torch.Tensor) -> bool:
    return all(t.is_cuda for t in ts)


def gemm_raw(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, M: int, N: int, K: int, lda: int, ldb: int,
             ldc: int, a_mn: bool, b_mn: bool, accumulate: bool = False, alpha: float = 1.0, bn: int = 0) -> None:
    lib = _lib.load("gemm")
    rc = lib.ts_gemm_bf16(_lib.ptr(a), _lib.ptr(b), _lib.ptr(out), M, N, K, lda, ldb, ldc, int(a_mn), int(b_mn),
                          int(out.dtype == torch.float32), int(accumulate), _c.c_float(alpha), bn, _lib.stream_ptr())
    _lib.check(rc, "ts_gemm_bf16")


def _rows2d(t: torch.Tensor) -> torch.Tensor:
    t = t.reshape(-1, t.shape[-1])
    if t.stride(-1) != 1 or (t.stride(0) * t.element_size()) % 16 != 0 or t.data_ptr() % 16 != 0:
        t = t.contiguous()
    return t


def matmul_nt(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, out_dtype=None,
              accumulate: bool = False, alpha: float = 1.0, bn: int = 0) -> torch.Tensor:
    """out[M,N] = alpha * a[M,K] @ b[N,K]^T (+ out)."""
    a2, b2 = _rows2d(a), _rows2d(b)
    M, K = a2.shape
    N = b2.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
    if not _use_cuda(a2, b2):
        r = alpha * (a2.float() @ b2.float().t())
        out.copy_((out.float() + r) if accumulate else r)
        return out
    gemm_raw(a2, b2, out, M, N, K, a2.stride(0), b2.stride(0), out.stride(0), False, False, accumulate, alpha, bn)
    return out


def matmul_nn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, out_dtype=None,
              accumulate: bool = False, alpha: float = 1.0, bn: int = 0) -> torch.Tensor:
    """out[M,N] = alpha * a[M,K] @ b[K,N] (+ out); b is read in place as an MN-major operand."""
    a2, b2 = _rows2d(a), _rows2d(b)
    M, K = a2.shape
    N = b2.shape[1]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
    if not _use_cuda(a2, b2):
        r = alpha * (a2.float() @ b2.float())
        out.copy_((out.float() + r) if accumulate else r)
        return out
    gemm_raw(a2, b2, out, M, N, K, a2.stride(0), b2.stride(0), out.stride(0), False, True, accumulate, alpha, bn)
    return out


def matmul_tn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, out_dtype=None,
              accumulate: bool = False, alpha: float = 1.0, bn: int = 0) -> torch.Tensor:
    """out[M,N] = alpha * a[K,M]^T @ b[K,N] (+ out); both operands are read as MN-major (weight gradient)."""
    a2, b2 = _rows2d(a), _rows2d(b)
    K, M = a2.shape
    N = b2.shape[1]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
    if not _use_cuda(a2, b2):
        r = alpha * (a2.float().t() @ b2.float())
        out.copy_((out.float() + r) if accumulate else r)
        return out
    gemm_raw(a2, b2, out, M, N, K, a2.stride(0), b2.stride(0), out.stride(0), True, True, accumulate, alpha, bn)
    return out


class WgradQueue:
    """Deferred weight-gradient GEMMs (zero-bubble pipeline schedules): inside `with queue.defer():` a linear's
    backward only runs the input-gradient GEMM and parks (dy, x, w); `queue.run()` executes the parked
    weight-gradient GEMMs later, when the schedule has a bubble to fill."""

    _active: "WgradQueue | None" = None

    def __init__(self):
        self.items: list = []

    class _Ctx:
        def __init__(self, q):
            self.q = q

        def __enter__(self):
            self.prev = WgradQueue._active
            WgradQueue._active = self.q
            return self.q

        def __exit__(self, *a):
            WgradQueue._active = self.prev

    def defer(self):
        return WgradQueue._Ctx(self)

    def push(self, dy2, x, w):
        self.items.append((dy2, x, w))

    def run(self, max_items: int | None = None) -> int:
        n = 0
        while self.items and (max_items is None or n < max_items):
            dy2, x, w = self.items.pop(0)
            _accumulate_wgrad(dy2, x, w)
            n += 1
        return n

    def __len__(self):
        return len(self.items)


def _accumulate_wgrad(dy2, x, w):
    """dW += dy^T x into w.main_grad when the engine owns one, else into w.grad."""
    x2 = _rows2d(x)
    main_grad = getattr(w, "main_grad", None)
    if main_grad is not None:
        if dy2.is_cuda and dy2.dtype == torch.bfloat16:
            matmul_tn(dy2, x2, out=main_grad.view(w.shape), accumulate=getattr(w, "grad_added", False))
        else:
            g = dy2.float().t() @ x2.float()
            main_grad.view(w.shape).copy_(main_grad.view(w.shape).float() + g if getattr(w, "grad_added", False) else g)
        w.grad_added = True
        return
    g = matmul_tn(dy2, x2) if (dy2.is_cuda and dy2.dtype == torch.bfloat16) else (dy2.float().t() @ x2.float()).to(w.dtype)
    w.grad = g if w.grad is None else w.grad + g


def linear_bwd(dy, x, w, need_dx: bool = True, need_dw: bool = True):
    """Backward of y = x @ w^T on the tcgen05 kernels. Returns (dx, dw); dw is None when the weight gradient was
    accumulated into `w.main_grad` by the GEMM epilogue or parked on the active `WgradQueue`."""
    dy2 = _rows2d(dy)
    dx = dw = None
    if need_dx:
        dx = matmul_nn(dy2, w).view_as(x)
    if need_dw and WgradQueue._active is not None:
        WgradQueue._active.push(dy2, x, w)
    elif need_dw:
        main_grad = getattr(w, "main_grad", None)
        if main_grad is not None:
            # gradient accumulated straight into the owner's buffer (fp32 or bf16) by the epilogue
            matmul_tn(dy2, x, out=main_grad.view(w.shape), accumulate=getattr(w, "grad_added", False))
            w.grad_added = True
        else:
            dw = matmul_tn(dy2, x)
    return dx, dw


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        # the result is allocated in its final shape (not returned as a view of a 2-D buffer), so that a following
        # in-place op (the rotary embedding on q|k) is legal for autograd
        y = torch.empty(*x.shape[:-1], w.shape[0], dtype=x.dtype, device=x.device)
        matmul_nt(x, w, out=y.view(-1, w.shape[0]))
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        return linear_bwd(dy, x, w, ctx.needs_input_grad[0], ctx.needs_input_grad[1])


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """y = x @ w.T (+ bias). bf16 CUDA tensors run on the tcgen05 kernel; anything else on PyTorch."""
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        y = _LinearFn.apply(x, w)
        return y if bias is None else y + bias
    if WgradQueue._active is not None and w.requires_grad:
        y = _SplitLinearCPU.apply(x, w)
        return y if bias is None else y + bias
    return torch.nn.functional.linear(x, w, bias)


class _SplitLinearCPU(torch.autograd.Function):
    """PyTorch-op linear whose weight gradient can be deferred (CPU / fp32 path of the zero-bubble split)."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return torch.nn.functional.linear(x, w)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dx = (dy2 @ w).view_as(x) if ctx.needs_input_grad[0] else None
        if WgradQueue._active is not None:
            WgradQueue._active.push(dy2, x, w)
            return dx, None
        return dx, (dy2.t() @ x.reshape(-1, x.shape[-1])).to(w.dtype)
