"""Block-scaled fp8 (E4M3) ops on the sm_100a kernels: quantise / dequantise and the tcgen05 kind::f8f6f4 GEMM.

Activations: one fp32 scale per 1 x 128 block (stored [K/128, M]); weights: one per 128 x 128 block ([N/128, K/128]).
`fp8_linear` runs forward and dgrad in fp8 (the gradient w.r.t. the output is re-quantised along its own reduction
axis) and keeps wgrad in bf16.  Reference: data_pipeline/trainer/kernels/fp8_kernels.py:203-553 (quantise, block- and
row-scaled matmul) with `block_dequantize_fp8` (:704) as the oracle.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib, gemm

_ll = ctypes.c_longlong


def available(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 128 == 0


def quant_act(x2: torch.Tensor):
    """x2 [M, K] bf16 -> (q uint8-viewed e4m3 [M, K], scale fp32 [K/128, M])."""
    lib = _lib.load("fp8")
    M, K = x2.shape
    x2 = x2 if x2.is_contiguous() else x2.contiguous()
    q = torch.empty(M, K, dtype=torch.float8_e4m3fn, device=x2.device)
    s = torch.empty(K // 128, M, dtype=torch.float32, device=x2.device)
    _lib.check(lib.ts_fp8_quant_act(_lib.ptr(x2), _lib.ptr(q), _lib.ptr(s), _ll(M), K, _lib.stream_ptr()),
               "ts_fp8_quant_act")
    return q, s


def quant_block(w: torch.Tensor):
    """w [N, K] bf16 -> (q e4m3 [N, K], scale fp32 [ceil(N/128), K/128])."""
    lib = _lib.load("fp8")
    N, K = w.shape
    w = w if w.is_contiguous() else w.contiguous()
    q = torch.empty(N, K, dtype=torch.float8_e4m3fn, device=w.device)
    s = torch.empty((N + 127) // 128, K // 128, dtype=torch.float32, device=w.device)
    _lib.check(lib.ts_fp8_quant_block(_lib.ptr(w), _lib.ptr(q), _lib.ptr(s), N, K, _lib.stream_ptr()),
               "ts_fp8_quant_block")
    return q, s


def quant_row(x2: torch.Tensor):
    """Per-row scales: (q [M, K], scale [M])."""
    lib = _lib.load("fp8")
    M, K = x2.shape
    x2 = x2 if x2.is_contiguous() else x2.contiguous()
    q = torch.empty(M, K, dtype=torch.float8_e4m3fn, device=x2.device)
    s = torch.empty(M, dtype=torch.float32, device=x2.device)
    _lib.check(lib.ts_fp8_quant_row(_lib.ptr(x2), _lib.ptr(q), _lib.ptr(s), _ll(M), K, _lib.stream_ptr()),
               "ts_fp8_quant_row")
    return q, s


def dequant(q: torch.Tensor, scale: torch.Tensor, layout: str) -> torch.Tensor:
    """layout: 'block' (128x128), 'act' (1x128, scale [K/128, M]) or 'row'."""
    lib = _lib.load("fp8")
    R, K = q.shape
    out = torch.empty(R, K, dtype=torch.bfloat16, device=q.device)
    code = {"block": 0, "act": 1, "row": 2}[layout]
    _lib.check(lib.ts_fp8_dequant(_lib.ptr(q), _lib.ptr(scale), _lib.ptr(out), _ll(R), K, code, _lib.stream_ptr()),
               "ts_fp8_dequant")
    return out


def gemm_fp8(aq, sa, bq, sb, N: int, b_mn: bool = False, out_dtype=torch.bfloat16) -> torch.Tensor:
    """C = block-scaled aq [M, K] x B.  b_mn=False: bq [N, K], sb [N/128, K/128].  b_mn=True: bq is the stored weight
    [K, N] (the reduction runs over its rows) and sb is its [K/128, N/128] block-scale matrix."""
    lib = _lib.load("fp8")
    M, K = aq.shape
    out = torch.empty(M, N, dtype=out_dtype, device=aq.device)
    if not b_mn:
        sb_n, sb_k = sb.stride(0), sb.stride(1)
    else:
        sb_n, sb_k = sb.stride(1), sb.stride(0)
    rc = lib.ts_fp8_gemm(_lib.ptr(aq), _lib.ptr(sa), _lib.ptr(bq), _lib.ptr(sb), _ll(sb_n), _ll(sb_k), _lib.ptr(out), M,
                         N, K, aq.stride(0), bq.stride(0), out.stride(0), int(b_mn), int(out_dtype == torch.float32),
                         _lib.stream_ptr())
    _lib.check(rc, "ts_fp8_gemm")
    _lib.LAUNCHES += 1
    return out


class _FP8LinearFn(torch.autograd.Function):
    """y = x @ w^T with fp8 forward and dgrad.  `wq`/`ws` may be given (a frozen pre-quantised weight) or are produced
    from the bf16 weight on the fly (fp8 training)."""

    @staticmethod
    def forward(ctx, x, w, wq, ws):
        x2 = x.reshape(-1, x.shape[-1])
        if wq is None:
            wq, ws = quant_block(w)
        xq, xs = quant_act(x2)
        y = gemm_fp8(xq, xs, wq, ws, wq.shape[0])
        ctx.save_for_backward(x2, wq, ws, w if w is not None and w.requires_grad else None)
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], wq.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, wq, ws, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        dx = dw = None
        N, K = wq.shape
        if ctx.needs_input_grad[0]:
            if N % 128 == 0:
                dq, ds = quant_act(dy2)                                   # blocks along N, the dgrad reduction axis
                dx = gemm_fp8(dq, ds, wq, ws, K, b_mn=True).view(ctx.x_shape)
            else:
                dx = gemm.matmul_nn(dy2, dequant(wq, ws, "block")).view(ctx.x_shape)
        if w is not None and ctx.needs_input_grad[1]:
            _, dw = gemm.linear_bwd(dy2, x2, w, False, True)              # wgrad stays in bf16
        return dx, dw, None, None


def fp8_linear(x: torch.Tensor, w: torch.Tensor | None = None, wq: torch.Tensor | None = None,
               ws: torch.Tensor | None = None) -> torch.Tensor:
    """Linear layer with block-scaled fp8 operands (see module docstring)."""
    return _FP8LinearFn.apply(x, w, wq, ws)
