"""Optimizer step kernels: flat AdamW over fp32 master/moment shards with a bf16 write-back, Lion, and the
squared-norm reduction that feeds a device-side clip coefficient (no host sync anywhere in the step).

Update rule (decoupled AdamW, data_pipeline/trainer/optimizers/adamw.py:182-260):
  g <- g*grad_scale; m <- b1 m + (1-b1) g; v <- b2 v + (1-b2) g^2;
  p <- p (1 - lr wd) - lr (m/bc1) / (sqrt(v/bc2) + eps)
Clip coefficient min(1, max_norm / (norm + 1e-6)) as in data_pipeline/trainer/distributed/sota_utils.py:1294-1299.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_f = ctypes.c_float
_ll = ctypes.c_longlong


def sumsq_(out: torch.Tensor, x: torch.Tensor, nonfinite_flag: torch.Tensor | None = None, mul: float = 1.0) -> None:
    """out[0] += sum((x*mul)^2) ; sets nonfinite_flag[0] = 1 when the partial sum is inf/nan."""
    if x.is_cuda:
        lib = _lib.load("elementwise")
        xf = x.reshape(-1)
        rc = lib.ts_sumsq(_lib.ptr(xf), int(x.dtype == torch.bfloat16), _ll(xf.numel()), _lib.ptr(out),
                          _lib.ptr(nonfinite_flag), _f(mul), _lib.stream_ptr())
        _lib.check(rc, "ts_sumsq")
    else:
        s = (x.float() * mul).pow(2).sum()
        out += s
        if nonfinite_flag is not None and not torch.isfinite(s):
            nonfinite_flag.fill_(1.0)


def adamw_flat_(master: torch.Tensor, m: torch.Tensor, v: torch.Tensor, grad: torch.Tensor,
                param_lowp: torch.Tensor | None, *, lr: float, beta1: float, beta2: float, eps: float,
                weight_decay: float, step: int, grad_mul: float = 1.0, sumsq: torch.Tensor | None = None,
                max_norm: float = 0.0, skip_flag: torch.Tensor | None = None) -> None:
    """One fused AdamW step over flat buffers. `sumsq` (device fp32 scalar, already multiplied by
    grad_mul^2 by the caller's reduction) gives the clip coefficient when max_norm > 0."""
    n = master.numel()
    if master.is_cuda:
        lib = _lib.load("elementwise")
        rc = lib.ts_adamw_flat(_lib.ptr(master), _lib.ptr(m), _lib.ptr(v), _lib.ptr(grad),
                               int(grad.dtype == torch.bfloat16), _lib.ptr(param_lowp), _ll(n), _f(lr), _f(beta1),
                               _f(beta2), _f(eps), _f(weight_decay), int(step), _f(grad_mul), _lib.ptr(sumsq),
                               _f(max_norm), _lib.ptr(skip_flag), _lib.stream_ptr())
        _lib.check(rc, "ts_adamw_flat")
        return
    if skip_flag is not None and float(skip_flag) != 0.0:
        return
    coef = 1.0
    if sumsq is not None and max_norm > 0:
        coef = min(1.0, max_norm / (float(sumsq.sqrt()) + 1e-6))
    g = grad.float() * (grad_mul * coef)
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
    master.mul_(1 - lr * weight_decay).addcdiv_(m / bc1, (v / bc2).sqrt() + eps, value=-lr)
    if param_lowp is not None:
        param_lowp.copy_(master)


def lion_flat_(master, m, grad, param_lowp, *, lr, beta1, beta2, weight_decay, grad_mul=1.0) -> None:
    if master.is_cuda:
        lib = _lib.load("elementwise")
        rc = lib.ts_lion_flat(_lib.ptr(master), _lib.ptr(m), _lib.ptr(grad), int(grad.dtype == torch.bfloat16),
                              _lib.ptr(param_lowp), _ll(master.numel()), _f(lr), _f(beta1), _f(beta2),
                              _f(weight_decay), _f(grad_mul), _lib.stream_ptr())
        _lib.check(rc, "ts_lion_flat")
        return
    g = grad.float() * grad_mul
    u = (beta1 * m + (1 - beta1) * g).sign()
    master.mul_(1 - lr * weight_decay).add_(u, alpha=-lr)
    m.mul_(beta2).add_(g, alpha=1 - beta2)
    if param_lowp is not None:
        param_lowp.copy_(master)


def scale_cast_(dst: torch.Tensor, src: torch.Tensor, mul: float = 1.0, accumulate: bool = False) -> None:
    """dst (+)= src * mul with bf16/fp32 conversion."""
    if dst.is_cuda:
        kind = {(torch.bfloat16, torch.bfloat16): 0, (torch.float32, torch.bfloat16): 1,
                (torch.bfloat16, torch.float32): 2, (torch.float32, torch.float32): 3}[(dst.dtype, src.dtype)]
        lib = _lib.load("elementwise")
        rc = lib.ts_scale_cast(_lib.ptr(dst), _lib.ptr(src), _ll(dst.numel()), _f(mul), int(accumulate), kind,
                               _lib.stream_ptr())
        _lib.check(rc, "ts_scale_cast")
        return
    r = src.float() * mul
    dst.copy_(dst.float() + r if accumulate else r)
