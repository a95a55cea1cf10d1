"""RMSNorm (optionally fused with the residual add) on the sm_100a kernels, with autograd.

Reference behaviour: data_pipeline/trainer/kernels/triton_kernels.py:477-682 (forward stores rstd in fp32,
backward dx = rstd*(dy*w - xhat*mean(dy*w*xhat)), dw = sum_rows dy*xhat) and the fused add+norm of
data_pipeline/trainer/kernels/layernorm_kernels.py:496.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def rmsnorm_reference(x, w, eps=1e-5, residual=None, w_offset=0.0):
    """fp32 PyTorch math; returns (y, new_residual)."""
    h = x if residual is None else (x.float() + residual.float()).to(x.dtype)
    hf = h.float()
    y = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * (w.float() + w_offset)
    return y.to(x.dtype), h


def rmsnorm_fwd_raw(x2, r2, w, eps, w_offset=0.0):
    """Kernel call on 2-D contiguous bf16 rows. Returns (y, h, rstd) with h = x (+ residual), the tensor the
    backward needs."""
    lib = _lib.load("elementwise")
    rows, H = x2.shape
    y = torch.empty_like(x2)
    rstd = torch.empty(rows, dtype=torch.float32, device=x2.device)
    res_out = torch.empty_like(x2) if r2 is not None else None
    rc = lib.ts_rmsnorm_fwd(_lib.ptr(x2), _lib.ptr(r2), _lib.ptr(w), _lib.ptr(y), _lib.ptr(res_out),
                            _lib.ptr(rstd), ctypes.c_longlong(rows), H, ctypes.c_float(eps),
                            ctypes.c_float(w_offset), _lib.stream_ptr())
    _lib.check(rc, "ts_rmsnorm_fwd")
    return y, (x2 if r2 is None else res_out), rstd


def rmsnorm_bwd_raw(dy2, h, w, rstd, dres2, w_offset=0.0):
    """Returns (dx, dw). dw is None when the weight gradient went straight into `w.main_grad`."""
    lib = _lib.load("elementwise")
    rows, H = h.shape
    dx = torch.empty_like(h)
    parts = lib.ts_rmsnorm_bwd_parts(ctypes.c_longlong(rows))
    partial = torch.empty(parts, H, dtype=torch.float32, device=h.device)
    main_grad = getattr(w, "main_grad", None)
    if main_grad is not None:
        acc = bool(getattr(w, "grad_added", False))
        f32 = main_grad if main_grad.dtype == torch.float32 else None
        b16 = main_grad if main_grad.dtype == torch.bfloat16 else None
        dw_out = None
        w.grad_added = True
    else:
        acc = False
        dw_out = torch.empty(H, dtype=torch.float32, device=h.device)
        f32, b16 = dw_out, None
    rc = lib.ts_rmsnorm_bwd(_lib.ptr(dy2), _lib.ptr(h), _lib.ptr(w), _lib.ptr(rstd), _lib.ptr(dres2), _lib.ptr(dx),
                            _lib.ptr(partial), _lib.ptr(f32), _lib.ptr(b16), int(acc), ctypes.c_longlong(rows), H,
                            ctypes.c_float(w_offset), _lib.stream_ptr())
    _lib.check(rc, "ts_rmsnorm_bwd")
    return dx, (None if dw_out is None else dw_out.to(w.dtype))


def _rows(t, H):
    t2 = t.reshape(-1, H)
    return t2 if t2.is_contiguous() else t2.contiguous()


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, residual, eps, w_offset):
        H = x.shape[-1]
        y, h, rstd = rmsnorm_fwd_raw(_rows(x, H), None if residual is None else _rows(residual, H), w, eps, w_offset)
        ctx.save_for_backward(h, w, rstd)
        ctx.w_offset = w_offset
        ctx.has_res = residual is not None
        ctx.shape = x.shape
        if residual is None:
            return y.view(x.shape)
        return y.view(x.shape), h.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dres=None):
        h, w, rstd = ctx.saved_tensors
        H = h.shape[1]
        dx, dw = rmsnorm_bwd_raw(_rows(dy, H), h, w, rstd, None if dres is None else _rows(dres, H), ctx.w_offset)
        dxv = dx.view(ctx.shape)
        # with a residual input, d(residual) == d(x): both feed h = x + residual
        return dxv, dw, (dxv if ctx.has_res else None), None, None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-5, residual: torch.Tensor | None = None,
            w_offset: float = 0.0):
    """Returns (normed, new_residual). `new_residual` is x (+ residual) and is what the next block adds to."""
    H = x.shape[-1]
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and H % 8 == 0 and H <= 8192:
        if residual is None:
            return _RMSNormFn.apply(x, w, None, eps, w_offset), x
        return _RMSNormFn.apply(x, w, residual, eps, w_offset)
    return rmsnorm_reference(x, w, eps, residual, w_offset)


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps):
        lib = _lib.load("elementwise")
        H = x.shape[-1]
        x2 = _rows(x, H)
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty_like(mean)
        rc = lib.ts_layernorm_fwd(_lib.ptr(x2), _lib.ptr(w), _lib.ptr(b), _lib.ptr(y), _lib.ptr(mean), _lib.ptr(rstd),
                                  ctypes.c_longlong(rows), H, ctypes.c_float(eps), _lib.stream_ptr())
        _lib.check(rc, "ts_layernorm_fwd")
        ctx.save_for_backward(x2, w, mean, rstd)
        ctx.has_bias, ctx.shape = b is not None, x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        lib = _lib.load("elementwise")
        x2, w, mean, rstd = ctx.saved_tensors
        rows, H = x2.shape
        dy2 = _rows(dy, H)
        dx = torch.empty_like(x2)
        parts = lib.ts_rmsnorm_bwd_parts(ctypes.c_longlong(rows))
        partial = torch.empty(parts, 2, H, dtype=torch.float32, device=x2.device)
        dw = torch.empty(H, dtype=torch.float32, device=x2.device)
        db = torch.empty(H, dtype=torch.float32, device=x2.device) if ctx.has_bias else None
        rc = lib.ts_layernorm_bwd(_lib.ptr(dy2), _lib.ptr(x2), _lib.ptr(w), _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(dx),
                                  _lib.ptr(partial), _lib.ptr(dw), _lib.ptr(db), ctypes.c_longlong(rows), H,
                                  _lib.stream_ptr())
        _lib.check(rc, "ts_layernorm_bwd")
        return dx.view(ctx.shape), dw.to(w.dtype), (db.to(w.dtype) if db is not None else None), None


def layernorm(x, w, b=None, eps=1e-5):
    """LayerNorm over the last dimension (sm_100a kernel for bf16 CUDA rows up to 8192 wide, PyTorch otherwise).
    Reference kernels: data_pipeline/trainer/kernels/layernorm_kernels.py:143-621."""
    H = x.shape[-1]
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and H % 8 == 0 and H <= 8192 \
            and (b is None or b.dtype == torch.bfloat16):
        return _LayerNormFn.apply(x, w, b, eps)
    return torch.nn.functional.layer_norm(x, (H,), w, b, eps)
