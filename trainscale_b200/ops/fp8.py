"""fp8 ops on the sm_100a kernels: quantise / dequantise and the tcgen05 kind::f8f6f4 GEMMs.

Two recipes.  "rowwise" (default of `fp8_linear`): every scale is constant along the reduction axis (one per token /
per feature), applied in the GEMM epilogue; forward, dgrad AND wgrad run at the full fp8 tensor-core rate on the
paired-CTA kernel of csrc/fp8_rowwise.cu, gradients optionally in E5M2.  "block": the 1 x 128 / 128 x 128 recipe below.

Block recipe:

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
               ws: torch.Tensor | None = None, recipe: str = "block", grad_format: str = "e4m3") -> torch.Tensor:
    """Linear layer with fp8 operands.  recipe "rowwise": fwd + dgrad + wgrad in fp8 at the full tensor-core rate
    (falls back to "block" for shapes whose fp8 rows would not be 16-byte aligned); "block": 1 x 128 / 128 x 128
    scales, fwd + dgrad in fp8, wgrad in bf16 (also the path of a frozen pre-quantised weight `wq` / `ws`)."""
    if recipe == "rowwise" and wq is None and w is not None and rowwise_available(x, w):
        return fp8_linear_rowwise(x, w, grad_format)
    return _FP8LinearFn.apply(x, w, wq, ws)


# ---------------------------------------------------------------------------------------------------------------
# rowwise recipe (csrc/fp8_rowwise.cu)
# ---------------------------------------------------------------------------------------------------------------
_FMT = {"e4m3": 0, "e5m2": 1}
_TORCH_FP8 = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}
_FMAX = {"e4m3": 448.0, "e5m2": 57344.0}


def rowwise_available(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Every leading dimension of the three GEMMs must keep fp8 rows 16-byte aligned."""
    T = x.numel() // x.shape[-1]
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 16 == 0 and
            w.shape[0] % 16 == 0 and T % 16 == 0)


def quant_rowwise(x2: torch.Tensor, fmt: str = "e4m3"):
    """x2 [R, C] bf16 -> (q fp8 [R, C], scale fp32 [R]): one scale per row."""
    lib = _lib.load("fp8_rowwise")
    R, C = x2.shape
    if x2.stride(1) != 1 or x2.stride(0) % 8 != 0:
        x2 = x2.contiguous()
    q = torch.empty(R, C, dtype=_TORCH_FP8[fmt], device=x2.device)
    s = torch.empty(R, dtype=torch.float32, device=x2.device)
    _lib.check(lib.ts_fp8_quant_rowwise(_lib.ptr(x2), _ll(x2.stride(0)), _lib.ptr(q), _lib.ptr(s), _ll(R), C, _FMT[fmt],
                                        _lib.stream_ptr()), "ts_fp8_quant_rowwise")
    return q, s


def quant_colwise(x2: torch.Tensor, fmt: str = "e4m3"):
    """x2 [R, C] bf16 -> (q fp8 [R, C] in the same layout, scale fp32 [C]): one scale per column."""
    lib = _lib.load("fp8_rowwise")
    R, C = x2.shape
    if x2.stride(1) != 1 or x2.stride(0) % 8 != 0:
        x2 = x2.contiguous()
    q = torch.empty(R, C, dtype=_TORCH_FP8[fmt], device=x2.device)
    s = torch.empty(C, dtype=torch.float32, device=x2.device)
    work = torch.empty(C, dtype=torch.int32, device=x2.device)
    _lib.check(lib.ts_fp8_quant_colwise(_lib.ptr(x2), _ll(x2.stride(0)), _lib.ptr(q), _lib.ptr(s), _lib.ptr(work),
                                        _ll(R), C, _FMT[fmt], _lib.stream_ptr()), "ts_fp8_quant_colwise")
    return q, s


def gemm_rowwise(a, sa, b, sb, M: int, N: int, K: int, a_mn: bool = False, b_mn: bool = False, out=None,
                 out_dtype=torch.bfloat16, accumulate: bool = False) -> torch.Tensor:
    """out[M, N] (+)= sa[m] * sb[n] * sum_k A[m, k] B[n, k].  a: [M, K] (a_mn False) or [K, M] (a_mn True) fp8;
    b: [N, K] (b_mn False) or [K, N] (b_mn True) fp8; formats are read from the tensors' dtypes."""
    lib = _lib.load("fp8_rowwise")
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    fa = 1 if a.dtype == torch.float8_e5m2 else 0
    fb = 1 if b.dtype == torch.float8_e5m2 else 0
    rc = lib.ts_fp8_rowwise_gemm(_lib.ptr(a), _lib.ptr(sa), _lib.ptr(b), _lib.ptr(sb), _lib.ptr(out), M, N, K,
                                 a.stride(0), b.stride(0), out.stride(0), int(a_mn), int(b_mn), fa, fb,
                                 int(out.dtype == torch.float32), int(accumulate), _lib.stream_ptr())
    _lib.check(rc, "ts_fp8_rowwise_gemm")
    return out


def dequant_rowwise(q: torch.Tensor, s: torch.Tensor, axis: int) -> torch.Tensor:
    """fp32 values of a rowwise (axis 0) or colwise (axis 1) quantised matrix (test oracle)."""
    return q.float() * (s.view(-1, 1) if axis == 0 else s.view(1, -1))


# Weights change only in the optimizer step, but a step quantises each of them once per forward (row scales) and once
# per backward (column scales) of every micro-batch.  The engines bump WEIGHT_EPOCH when they update (or reload) the
# parameters; inside one epoch both quantised copies of a weight are made once and reused.  (The optimizer kernels write
# through raw pointers, so torch's own version counter cannot be the key.)
WEIGHT_EPOCH = [0]
_W_CACHE: dict = {}
_W_CACHE_BYTES = [0]
# the two fp8 copies take as many bytes as the bf16 weight itself: the cache stops growing at this size (the weights
# that do not fit are simply re-quantised on every use)
W_CACHE_LIMIT_BYTES = int(float(__import__("os").environ.get("TS_FP8_WEIGHT_CACHE_GB", "8")) * 2 ** 30)


def bump_weight_epoch() -> None:
    WEIGHT_EPOCH[0] += 1
    _W_CACHE.clear()
    _W_CACHE_BYTES[0] = 0


def _quant_weight(w: torch.Tensor, which: str):
    """Row-scaled (`which` "row": forward) or column-scaled ("col": dgrad) fp8 copy of a weight and its scales.  Both
    copies are made together and cached per weight epoch while the cache has room; beyond that only the requested one
    is made."""
    import weakref
    key = (id(w), w._version)       # (a re-gathered ZeRO-3 weight keeps its identity and its values inside an epoch)
    hit = _W_CACHE.get(key)
    if hit is not None and hit[0] == WEIGHT_EPOCH[0] and hit[2]() is w:
        wq, sw, wc, swc = hit[1]
        return (wq, sw) if which == "row" else (wc, swc)
    if _W_CACHE_BYTES[0] + 2 * w.numel() > W_CACHE_LIMIT_BYTES:
        return quant_rowwise(w) if which == "row" else quant_colwise(w)
    wq, sw = quant_rowwise(w)
    wc, swc = quant_colwise(w)
    _W_CACHE[key] = (WEIGHT_EPOCH[0], (wq, sw, wc, swc), weakref.ref(w))
    _W_CACHE_BYTES[0] += 2 * w.numel()
    return (wq, sw) if which == "row" else (wc, swc)


class _FP8RowwiseLinearFn(torch.autograd.Function):
    """y = x @ w^T with all three GEMMs in fp8.  Saved for backward: the column-scaled fp8 copy of x (half the bytes
    of the bf16 activation) and the weight."""

    @staticmethod
    def forward(ctx, x, w, grad_fmt):
        x2 = x.reshape(-1, x.shape[-1])
        T, K = x2.shape
        N = w.shape[0]
        xq, sx = quant_rowwise(x2)
        wq, sw = _quant_weight(w, "row") if w.requires_grad else quant_rowwise(w)
        y = gemm_rowwise(xq, sx, wq, sw, T, N, K)
        need_dw = w.requires_grad
        if need_dw:
            xc, sxc = quant_colwise(x2)                  # operand of wgrad: scales per input feature, over all tokens
        else:
            xc = sxc = None
        ctx.save_for_backward(xc, sxc, w)
        ctx.x_shape, ctx.grad_fmt = x.shape, grad_fmt
        return y.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        xc, sxc, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        T, N = dy2.shape
        K = w.shape[1]
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dq, sd = quant_rowwise(dy2, ctx.grad_fmt)    # scales per token
            wc, swc = _quant_weight(w, "col")            # scales per input feature k; stored [N][K] = MN-major B
            dx = gemm_rowwise(dq, sd, wc, swc, T, K, N, b_mn=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            dc, sdc = quant_colwise(dy2, ctx.grad_fmt)   # scales per output feature n, over all tokens
            main_grad = getattr(w, "main_grad", None)
            if main_grad is not None:
                gemm_rowwise(dc, sdc, xc, sxc, N, K, T, a_mn=True, b_mn=True, out=main_grad.view(w.shape),
                             accumulate=getattr(w, "grad_added", False))
                w.grad_added = True
            else:
                dw = gemm_rowwise(dc, sdc, xc, sxc, N, K, T, a_mn=True, b_mn=True, out_dtype=w.dtype)
        return dx, dw, None


def fp8_linear_rowwise(x: torch.Tensor, w: torch.Tensor, grad_format: str = "e4m3") -> torch.Tensor:
    """Linear layer whose forward, dgrad and wgrad GEMMs all run in fp8 with row / column scales (module docstring)."""
    return _FP8RowwiseLinearFn.apply(x, w, grad_format)
