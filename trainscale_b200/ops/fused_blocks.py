"""Norm->linear and GLU->linear blocks that keep only the GEMM-side tensors for backward.

A plain `rmsnorm` followed by `linear` stores the normalised activations twice over (the linear saves its input);
`glu` followed by `linear` stores the gated product.  These blocks store only what is expensive to rebuild (the
residual stream, the rstd vector, the gate|up projection) and re-run the cheap elementwise kernel in backward, so a
decoder layer holds x, qkv, attention output, the post-attention residual and gate|up: about two thirds of the plain
footprint, with no GEMM or attention recomputation.  This is the operator-level selective recomputation mode of
data_pipeline/trainer/distributed/activation_checkpoint.py (OP_SELECTIVE), specialised to the framework decoder.
"""
from __future__ import annotations

import torch

from . import activation, gemm, norm


class _NormLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, norm_w, w, eps, w_offset):
        H = x.shape[-1]
        x2 = norm._rows(x, H)
        r2 = None if residual is None else norm._rows(residual, H)
        y, h, rstd = norm.rmsnorm_fwd_raw(x2, r2, norm_w, eps, w_offset)
        out = torch.empty(*x.shape[:-1], w.shape[0], dtype=x.dtype, device=x.device)     # final shape, not a view
        gemm.matmul_nt(y, w, out=out.view(-1, w.shape[0]))
        ctx.save_for_backward(h, norm_w, rstd, w)
        ctx.eps, ctx.w_offset, ctx.has_res, ctx.shape = eps, w_offset, residual is not None, x.shape
        if residual is None:
            return out
        return out, h.view(x.shape)

    @staticmethod
    def backward(ctx, dout, dres=None):
        h, norm_w, rstd, w = ctx.saved_tensors
        H = h.shape[1]
        y, _, _ = norm.rmsnorm_fwd_raw(h, None, norm_w, ctx.eps, ctx.w_offset)      # rebuilt, never stored
        dy, dw = gemm.linear_bwd(dout, y, w, True, ctx.needs_input_grad[3])
        dx, dnw = norm.rmsnorm_bwd_raw(norm._rows(dy, H), h, norm_w, rstd,
                                       None if dres is None else norm._rows(dres, H), ctx.w_offset)
        dxv = dx.view(ctx.shape)
        return dxv, (dxv if ctx.has_res else None), dnw, dw, None, None


class _GluLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up, w, act_id):
        I2 = gate_up.shape[-1]
        gu = gate_up.reshape(-1, I2)
        gu = gu if gu.is_contiguous() else gu.contiguous()
        out = gemm.matmul_nt(activation.glu_fwd_raw(gu, act_id), w)
        ctx.save_for_backward(gu, w)
        ctx.act_id, ctx.in_shape = act_id, gate_up.shape
        return out.view(*gate_up.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dout):
        gu, w = ctx.saved_tensors
        g = activation.glu_fwd_raw(gu, ctx.act_id)                                   # rebuilt, never stored
        dg, dw = gemm.linear_bwd(dout, g, w, True, ctx.needs_input_grad[1])
        return activation.glu_bwd_raw(dg.reshape(-1, g.shape[1]), gu, ctx.act_id).view(ctx.in_shape), dw, None


def supported(x: torch.Tensor, *weights: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and all(w.dtype == torch.bfloat16 for w in weights) \
        and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192


def norm_linear(x, residual, norm_w, w, eps: float = 1e-5, w_offset: float = 0.0):
    """(rmsnorm(x + residual) @ w^T, x + residual). Falls back to the separate ops off the CUDA bf16 path."""
    if supported(x, norm_w, w):
        if residual is None:
            return _NormLinearFn.apply(x, None, norm_w, w, eps, w_offset), x
        return _NormLinearFn.apply(x, residual, norm_w, w, eps, w_offset)
    y, h = norm.rmsnorm(x, norm_w, eps, residual, w_offset)
    return gemm.linear(y, w), h


def glu_linear(gate_up, w, act: str = "silu"):
    """glu(gate_up) @ w^T."""
    I = gate_up.shape[-1] // 2
    if gate_up.is_cuda and gate_up.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and I % 8 == 0:
        return _GluLinearFn.apply(gate_up, w, activation._ACT[act])
    return gemm.linear(activation.glu(gate_up, act), w)
