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


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        y = matmul_nt(x, w)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = _rows2d(dy)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = matmul_nn(dy2, w).view_as(x)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(w, "main_grad", None)
            if main_grad is not None:
                # gradient accumulated straight into the owner's buffer (fp32 or bf16) by the epilogue
                matmul_tn(dy2, x, out=main_grad.view(w.shape), accumulate=getattr(w, "grad_added", False))
                w.grad_added = True
                dw = None
            else:
                dw = matmul_tn(dy2, x)
        return dx, dw


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """y = x @ w.T (+ bias). bf16 CUDA tensors run on the tcgen05 kernel; anything else on PyTorch."""
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        y = _LinearFn.apply(x, w)
        return y if bias is None else y + bias
    return torch.nn.functional.linear(x, w, bias)
