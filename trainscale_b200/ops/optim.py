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


# ---------------------------------------------------------------------------------------------------------------
# Per-tensor optimizer kernels (library "optim"): 8-bit AdamW, LAMB, Sophia-G, schedule-free AdamW, ADOPT, AdaFactor.
# Parameters / gradients may be bf16 or fp32; every data-dependent scalar stays on the device.
# ---------------------------------------------------------------------------------------------------------------
QUANT_BLOCKS = (256, 1024, 2048, 4096)


def _kind(p: torch.Tensor, g: torch.Tensor | None) -> int:
    for t in (p, g):
        if t is not None and t.dtype not in (torch.float32, torch.bfloat16):
            raise TypeError(f"optimizer kernels take fp32 or bf16 tensors, got {t.dtype}")
    return int(p.dtype == torch.bfloat16) | (int(g is not None and g.dtype == torch.bfloat16) << 1)


def native_ok(p: torch.Tensor, g: torch.Tensor | None = None) -> bool:
    """True when the CUDA kernels can take this parameter / gradient pair in place."""
    ts = [p] if g is None else [p, g]
    return all(t.is_cuda and t.is_contiguous() and t.dtype in (torch.float32, torch.bfloat16) for t in ts)


def quant8(x: torch.Tensor, block: int = 256):
    """Block-wise absmax int8: returns (q int8 [nblocks, block], scale fp32 [nblocks])."""
    n = x.numel()
    nb = (n + block - 1) // block
    q = torch.empty((nb, block), dtype=torch.int8, device=x.device)
    s = torch.empty(nb, dtype=torch.float32, device=x.device)
    xf = x.reshape(-1).float().contiguous()
    rc = _lib.load("optim").ts_quant8(_lib.ptr(xf), _lib.ptr(q), _lib.ptr(s), _ll(n), int(block), _lib.stream_ptr())
    _lib.check(rc, "ts_quant8")
    return q, s


def dequant8(q: torch.Tensor, s: torch.Tensor, shape, numel: int) -> torch.Tensor:
    out = torch.empty(numel, dtype=torch.float32, device=q.device)
    rc = _lib.load("optim").ts_dequant8(_lib.ptr(q), _lib.ptr(s), _lib.ptr(out), _ll(numel), int(q.shape[1]),
                                        _lib.stream_ptr())
    _lib.check(rc, "ts_dequant8")
    return out.view(shape)


def adam8bit_(p, g, m_q, m_s, v_q, v_s, *, lr, beta1, beta2, eps, weight_decay, step) -> None:
    rc = _lib.load("optim").ts_adam8bit(_lib.ptr(p), _lib.ptr(g), _kind(p, g), _lib.ptr(m_q), _lib.ptr(m_s),
                                        _lib.ptr(v_q), _lib.ptr(v_s), _ll(p.numel()), int(m_q.shape[1]), _f(lr),
                                        _f(beta1), _f(beta2), _f(eps), _f(weight_decay), int(step), _lib.stream_ptr())
    _lib.check(rc, "ts_adam8bit")


def lamb_(p, g, m, v, upd, norms, *, lr, beta1, beta2, eps, weight_decay, step, trust_lo, trust_hi) -> None:
    """`upd` (fp32, p.numel()) is scratch; `norms` (fp32[2]) is zeroed here."""
    lib = _lib.load("optim")
    norms.zero_()
    k = _kind(p, g)
    rc = lib.ts_lamb_moments(_lib.ptr(p), _lib.ptr(g), k, _lib.ptr(m), _lib.ptr(v), _lib.ptr(upd), _lib.ptr(norms),
                             _ll(p.numel()), _f(beta1), _f(beta2), _f(eps), _f(weight_decay), int(step),
                             _lib.stream_ptr())
    _lib.check(rc, "ts_lamb_moments")
    rc = lib.ts_lamb_apply(_lib.ptr(p), k, _lib.ptr(upd), _lib.ptr(norms), _ll(p.numel()), _f(lr), _f(trust_lo),
                           _f(trust_hi), _lib.stream_ptr())
    _lib.check(rc, "ts_lamb_apply")


def sophia_step_(p, g, m, h, *, lr, beta1, rho, weight_decay, eps) -> None:
    rc = _lib.load("optim").ts_sophia_step(_lib.ptr(p), _lib.ptr(g), _kind(p, g), _lib.ptr(m), _lib.ptr(h),
                                           _ll(p.numel()), _f(lr), _f(beta1), _f(rho), _f(weight_decay), _f(eps),
                                           _lib.stream_ptr())
    _lib.check(rc, "ts_sophia_step")


def sophia_hessian_(g, h, *, beta2, scale) -> None:
    rc = _lib.load("optim").ts_sophia_hessian(_lib.ptr(g), _kind(h, g), _lib.ptr(h), _ll(h.numel()), _f(beta2),
                                              _f(scale), _lib.stream_ptr())
    _lib.check(rc, "ts_sophia_hessian")


def schedule_free_(p, g, z, v, *, lr, beta1, beta2, eps, weight_decay, c) -> None:
    rc = _lib.load("optim").ts_schedule_free(_lib.ptr(p), _lib.ptr(g), _kind(p, g), _lib.ptr(z), _lib.ptr(v),
                                             _ll(p.numel()), _f(lr), _f(beta1), _f(beta2), _f(eps), _f(weight_decay),
                                             _f(c), _lib.stream_ptr())
    _lib.check(rc, "ts_schedule_free")


def adopt_(p, g, m, v, *, lr, beta1, beta2, eps, weight_decay, clip) -> None:
    rc = _lib.load("optim").ts_adopt_step(_lib.ptr(p), _lib.ptr(g), _kind(p, g), _lib.ptr(m), _lib.ptr(v),
                                          _ll(p.numel()), _f(lr), _f(beta1), _f(beta2), _f(eps), _f(weight_decay),
                                          _f(clip if clip is not None else 0.0), _lib.stream_ptr())
    _lib.check(rc, "ts_adopt_step")


def adafactor_(p, g, st: dict, *, lr, beta2, eps0, eps1, clip, scale_parameter, beta1, weight_decay) -> None:
    """One AdaFactor step on a 2-D (factored: st has 'row', 'col') or any-shape (st has 'v') tensor.
    Scratch in st: 'u' (fp32 like p), 'sums' (fp32[2]), 'col_tmp' (factored)."""
    lib = _lib.load("optim")
    k = _kind(p, g)
    sums = st["sums"]
    sums.zero_()
    if "row" in st:
        R, C = p.shape
        st["col_tmp"].zero_()
        rc = lib.ts_adafactor_stats(_lib.ptr(g), k, _lib.ptr(st["row"]), _lib.ptr(st["col_tmp"]), int(R), int(C),
                                    _f(beta2), _f(eps0), _lib.stream_ptr())
        _lib.check(rc, "ts_adafactor_stats")
        st["col"].mul_(beta2).add_(st["col_tmp"], alpha=(1.0 - beta2) / R)
        row_mean = st["row"].mean().reshape(1)
        rc = lib.ts_adafactor_update(_lib.ptr(p), _lib.ptr(g), k, _lib.ptr(st["row"]), _lib.ptr(st["col"]),
                                     _lib.ptr(row_mean), _lib.ptr(None), _lib.ptr(st["u"]), _lib.ptr(sums), int(R), int(C),
                                     _f(beta2), _f(eps0), _lib.stream_ptr())
    else:
        rc = lib.ts_adafactor_update(_lib.ptr(p), _lib.ptr(g), k, _lib.ptr(None), _lib.ptr(None), _lib.ptr(None), _lib.ptr(st["v"]),
                                     _lib.ptr(st["u"]), _lib.ptr(sums), 1, int(p.numel()), _f(beta2), _f(eps0),
                                     _lib.stream_ptr())
    _lib.check(rc, "ts_adafactor_update")
    rc = lib.ts_adafactor_apply(_lib.ptr(p), k, _lib.ptr(st["u"]), _lib.ptr(st.get("m")), _lib.ptr(sums),
                                _ll(p.numel()), _f(lr), _f(eps1), int(bool(scale_parameter)), _f(clip),
                                _f(beta1 if beta1 is not None else 0.0), _f(weight_decay), _lib.stream_ptr())
    _lib.check(rc, "ts_adafactor_apply")
