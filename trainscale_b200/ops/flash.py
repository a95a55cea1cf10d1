"""Binding of the tcgen05 flash-attention kernels (csrc/attention.cu) with autograd.

Inputs are token-major: a fused qkv buffer [B, S, (Hq + 2 Hkv) * D] (or separate q / k / v views of it); the
kernels address heads through TMA coordinates, so nothing is split, transposed or made contiguous first.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _lib

_ll = ctypes.c_longlong
_f = ctypes.c_float


def supported(head_dim: int, window=None, softcap=0.0) -> bool:
    """Sliding windows and logit soft-capping run inside the kernels."""
    return head_dim in (64, 128)


def _fwd(qkv2d, Hq, Hkv, D, B, S, cu_seqlens, max_len, causal, scale, window=0, softcap=0.0):
    lib = _lib.load("attention")
    rows, width = qkv2d.shape
    o = torch.empty(rows, Hq * D, dtype=qkv2d.dtype, device=qkv2d.device)
    lse = torch.empty(Hq, rows, dtype=torch.float32, device=qkv2d.device)
    rc = lib.ts_flash_fwd_ex(_lib.ptr(qkv2d), _lib.ptr(qkv2d), _lib.ptr(qkv2d), _lib.ptr(o), _lib.ptr(lse), _ll(rows),
                             width, width, width, Hq * D, 0, Hq * D, (Hq + Hkv) * D, Hq, Hkv, D, B, S,
                             _lib.ptr(cu_seqlens), max_len, int(causal), _f(scale), int(window or 0),
                             _f(float(softcap or 0.0)), _lib.stream_ptr())
    _lib.check(rc, "ts_flash_fwd")
    return o, lse


def _bwd(qkv2d, o, lse, dout, Hq, Hkv, D, B, S, cu_seqlens, max_len, causal, scale, window=0, softcap=0.0):
    lib = _lib.load("attention")
    rows, width = qkv2d.shape
    dqkv = torch.empty_like(qkv2d)
    delta = torch.empty(Hq, rows, dtype=torch.float32, device=qkv2d.device)
    rc = lib.ts_attn_delta(_lib.ptr(o), _lib.ptr(dout), _lib.ptr(delta), _ll(rows), Hq, D, Hq * D, _lib.stream_ptr())
    _lib.check(rc, "ts_attn_delta")
    rc = lib.ts_flash_bwd_ex(_lib.ptr(qkv2d), _lib.ptr(qkv2d), _lib.ptr(qkv2d), _lib.ptr(dout), _lib.ptr(lse),
                             _lib.ptr(delta), _lib.ptr(dqkv), _ll(rows), width, Hq * D, 0, Hq * D, (Hq + Hkv) * D, Hq,
                             Hkv, D, B, S, _lib.ptr(cu_seqlens), max_len, int(causal), _f(scale), int(window or 0),
                             _f(float(softcap or 0.0)), _lib.stream_ptr())
    _lib.check(rc, "ts_flash_bwd")
    return dqkv


class _FlashQKV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, Hq, Hkv, D, causal, scale, cu_seqlens, max_len, window=0, softcap=0.0):
        B, S, W = qkv.shape
        q2 = qkv.reshape(B * S, W)
        if not q2.is_contiguous():
            q2 = q2.contiguous()
        if cu_seqlens is not None:
            nb, ml = cu_seqlens.numel() - 1, int(max_len or S * B)
            o, lse = _fwd(q2, Hq, Hkv, D, nb, 0, cu_seqlens, ml, causal, scale, window, softcap)
        else:
            o, lse = _fwd(q2, Hq, Hkv, D, B, S, None, S, causal, scale, window, softcap)
        ctx.save_for_backward(q2, o, lse, cu_seqlens)
        ctx.args = (Hq, Hkv, D, B, S, causal, scale, max_len, window, softcap)
        return o.view(B, S, Hq * D)

    @staticmethod
    def backward(ctx, dout):
        q2, o, lse, cu = ctx.saved_tensors
        Hq, Hkv, D, B, S, causal, scale, max_len, window, softcap = ctx.args
        d2 = dout.reshape(B * S, Hq * D)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        if cu is not None:
            dqkv = _bwd(q2, o, lse, d2, Hq, Hkv, D, cu.numel() - 1, 0, cu, int(max_len or S * B), causal, scale, window,
                        softcap)
        else:
            dqkv = _bwd(q2, o, lse, d2, Hq, Hkv, D, B, S, None, S, causal, scale, window, softcap)
        return dqkv.view(B, S, -1), None, None, None, None, None, None, None, None, None


def flash_attention_qkv(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, causal: bool = True,
                        scale: float | None = None, cu_seqlens: torch.Tensor | None = None,
                        max_seqlen: int | None = None, window: int | None = None, softcap: float = 0.0) -> torch.Tensor:
    scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    if cu_seqlens is not None:
        cu_seqlens = cu_seqlens.to(torch.int32)
    return _FlashQKV.apply(qkv, n_heads, n_kv_heads, head_dim, causal, scale, cu_seqlens, max_seqlen,
                           int(window or 0), float(softcap or 0.0))


def flash_forward_only(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, causal: bool = True,
                       scale: float | None = None, cu_seqlens: torch.Tensor | None = None, max_seqlen: int | None = None):
    """(out [B,S,Hq*D], lse [Hq, B*S]) without autograd."""
    B, S, W = qkv.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    q2 = qkv.reshape(B * S, W)
    if cu_seqlens is not None:
        cu = cu_seqlens.to(torch.int32)
        o, lse = _fwd(q2, n_heads, n_kv_heads, head_dim, cu.numel() - 1, 0, cu, int(max_seqlen or B * S), causal, scale)
    else:
        o, lse = _fwd(q2, n_heads, n_kv_heads, head_dim, B, S, None, S, causal, scale)
    return o.view(B, S, -1), lse
