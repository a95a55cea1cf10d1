"""Gated activations (SwiGLU / GeGLU) over a fused gate|up projection output.

Reference: data_pipeline/trainer/kernels/triton_kernels.py:1042-1295.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib

_ACT = {"silu": 0, "swiglu": 0, "gelu": 1, "geglu": 1, "gelu_tanh": 2}


def glu_reference(gate_up: torch.Tensor, act: str = "silu") -> torch.Tensor:
    g, u = gate_up.float().chunk(2, dim=-1)
    a = F.silu(g) if _ACT[act] == 0 else F.gelu(g, approximate="tanh" if _ACT[act] == 2 else "none")
    return (a * u).to(gate_up.dtype)


def glu_fwd_raw(gu, act_id: int):
    """gu: contiguous [rows, 2I] bf16 -> [rows, I]."""
    lib = _lib.load("elementwise")
    I = gu.shape[1] // 2
    out = torch.empty(gu.shape[0], I, dtype=gu.dtype, device=gu.device)
    rc = lib.ts_glu_fwd(_lib.ptr(gu), _lib.ptr(out), ctypes.c_longlong(gu.shape[0]), I, 2 * I, act_id, _lib.stream_ptr())
    _lib.check(rc, "ts_glu_fwd")
    return out


def glu_bwd_raw(d, gu, act_id: int):
    lib = _lib.load("elementwise")
    I = gu.shape[1] // 2
    dgu = torch.empty_like(gu)
    rc = lib.ts_glu_bwd(_lib.ptr(d), _lib.ptr(gu), _lib.ptr(dgu), ctypes.c_longlong(gu.shape[0]), I, 2 * I, act_id,
                        _lib.stream_ptr())
    _lib.check(rc, "ts_glu_bwd")
    return dgu


class _GluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up, act):
        I = gate_up.shape[-1] // 2
        gu = gate_up.reshape(-1, 2 * I)
        gu = gu if gu.is_contiguous() else gu.contiguous()
        out = glu_fwd_raw(gu, act)
        ctx.save_for_backward(gu)
        ctx.act = act
        ctx.in_shape = gate_up.shape
        return out.view(*gate_up.shape[:-1], I)

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        I = gu.shape[1] // 2
        d = dout.reshape(-1, I)
        d = d if d.is_contiguous() else d.contiguous()
        return glu_bwd_raw(d, gu, ctx.act).view(ctx.in_shape), None


def glu(gate_up: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """act(gate) * up for gate_up = [..., gate | up]."""
    I = gate_up.shape[-1] // 2
    if gate_up.is_cuda and gate_up.dtype == torch.bfloat16 and I % 8 == 0:
        return _GluFn.apply(gate_up, _ACT[act])
    return glu_reference(gate_up, act)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up for separate tensors (API parity with the reference's swiglu_forward)."""
    return glu(torch.cat((gate, up), dim=-1), "silu")


class _ActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, act_id):
        lib = _lib.load("elementwise")
        xc = x if x.is_contiguous() else x.contiguous()
        y = torch.empty_like(xc)
        _lib.check(lib.ts_act_fwd(_lib.ptr(xc), _lib.ptr(y), ctypes.c_longlong(xc.numel()), act_id, _lib.stream_ptr()),
                   "ts_act_fwd")
        ctx.save_for_backward(xc)
        ctx.act_id = act_id
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib.load("elementwise")
        (xc,) = ctx.saved_tensors
        d = dy if dy.is_contiguous() else dy.contiguous()
        dx = torch.empty_like(xc)
        _lib.check(lib.ts_act_bwd(_lib.ptr(d), _lib.ptr(xc), _lib.ptr(dx), ctypes.c_longlong(xc.numel()), ctx.act_id,
                                  _lib.stream_ptr()), "ts_act_bwd")
        return dx, None


def act(x: torch.Tensor, name: str = "gelu") -> torch.Tensor:
    """Un-gated SiLU / GELU (erf or tanh form) on the vectorised kernel for bf16 CUDA tensors, PyTorch otherwise
    (data_pipeline/trainer/kernels/triton_kernels.py:1295)."""
    kind = _ACT[name]
    if x.is_cuda and x.dtype == torch.bfloat16 and x.numel() % 8 == 0:
        return _ActFn.apply(x, kind)
    if kind == 0:
        return F.silu(x)
    return F.gelu(x, approximate="tanh" if kind == 2 else "none")


def gelu(x: torch.Tensor, approximate: str = "none") -> torch.Tensor:
    return act(x, "gelu_tanh" if approximate == "tanh" else "gelu")


class _SoftmaxFn(torch.autograd.Function):
    """Row softmax over the last dimension on the row kernel (bf16 CUDA rows whose pitch is a multiple of 8 elements);
    backward dx = y * (dy - sum(dy * y))."""

    @staticmethod
    def forward(ctx, x):
        V = x.shape[-1]
        x2 = x.reshape(-1, V).contiguous()
        y = torch.empty_like(x2)
        lib = _lib.load("elementwise")
        rc = lib.ts_softmax_rows(_lib.ptr(x2), _lib.ptr(y), ctypes.c_longlong(x2.shape[0]), V, _lib.stream_ptr())
        _lib.check(rc, "ts_softmax_rows")
        ctx.save_for_backward(y)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        yf, df = y.float(), dy.reshape(y.shape).float()
        return (yf * (df - (df * yf).sum(-1, keepdim=True))).to(dy.dtype).view(dy.shape)


def softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    if x.is_cuda and x.dtype == torch.bfloat16 and dim in (-1, x.dim() - 1) and x.shape[-1] % 8 == 0:
        return _SoftmaxFn.apply(x)
    return torch.softmax(x.float(), dim).to(x.dtype)
