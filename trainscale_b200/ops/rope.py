"""Rotary position embedding: frequency tables (with the scaling schemes of the reference) and the
in-place sm_100a kernel applied to the q|k heads of a fused qkv buffer.

Reference: data_pipeline/trainer/kernels/rope_kernels.py:37-45,198-315 (scaling), :385-956 (kernels),
data_pipeline/trainer/kernels/triton_kernels.py:713-1007.
"""
from __future__ import annotations

import math

import torch

from . import _lib


def rope_inv_freq(dim: int, theta: float = 10000.0, scaling: str = "none", factor: float = 1.0,
                  original_max_pos: int = 8192, max_pos: int | None = None, beta_fast: float = 32.0,
                  beta_slow: float = 1.0, low_freq_factor: float = 1.0, high_freq_factor: float = 4.0,
                  long_factor=None, short_factor=None) -> torch.Tensor:
    """Inverse frequencies [dim/2] for none | linear | ntk | dynamic_ntk | yarn | llama3 | longrope scaling.

    longrope (data_pipeline/trainer/kernels/rope_kernels.py:298-313): every rotary dimension has its own searched
    rescale factor; `long_factor` applies when the table covers more than `original_max_pos` positions, `short_factor`
    otherwise (both [dim/2]).  Asking for it without the factor list it needs is an error, not a silent fallback."""
    half = dim // 2
    idx = torch.arange(0, half, dtype=torch.float64)
    scaling = (scaling or "none").lower()
    if scaling in ("ntk", "dynamic_ntk"):
        f = factor
        if scaling == "dynamic_ntk" and max_pos is not None:
            f = max(1.0, (factor * max_pos / original_max_pos) - (factor - 1))
        theta = theta * f ** (dim / max(dim - 2, 1))
    inv = 1.0 / (theta ** (2 * idx / dim))
    if scaling == "longrope":
        use_long = max_pos is not None and max_pos > original_max_pos
        fac = long_factor if use_long else (short_factor if short_factor is not None else None)
        if fac is None and not use_long:
            return inv.float()               # inside the original window without short factors: plain RoPE
        if fac is None:
            raise ValueError("rope scaling 'longrope' beyond the original context needs `long_factor` "
                             f"(a list of {half} per-dimension factors)")
        fac = torch.as_tensor(fac, dtype=torch.float64).reshape(-1)
        if fac.numel() < half:
            raise ValueError(f"longrope factor list has {fac.numel()} entries, the rotary dimension needs {half}")
        return (inv / fac[:half]).float()
    if scaling == "linear":
        inv = inv / factor
    elif scaling == "yarn":
        def corr_dim(rot):
            return dim * math.log(original_max_pos / (rot * 2 * math.pi)) / (2 * math.log(theta))
        low = max(math.floor(corr_dim(beta_fast)), 0)
        high = min(math.ceil(corr_dim(beta_slow)), half - 1)
        ramp = ((idx - low) / max(high - low, 1e-3)).clamp(0, 1)
        inv = inv / factor * ramp + inv * (1 - ramp)
    elif scaling == "llama3":
        wavelen = 2 * math.pi / inv
        low_w = original_max_pos / low_freq_factor
        high_w = original_max_pos / high_freq_factor
        smooth = (original_max_pos / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
        scaled = torch.where(wavelen > low_w, inv / factor, inv)
        mid = (wavelen <= low_w) & (wavelen >= high_w)
        inv = torch.where(mid, (1 - smooth) * inv / factor + smooth * inv, scaled)
    return inv.float()


def longrope_attention_factor(max_pos: int, original_max_pos: int) -> float:
    """Magnitude correction LongRoPE applies to cos / sin when the context is extended (sqrt(1 + ln s / ln L0))."""
    s = max_pos / original_max_pos
    return 1.0 if s <= 1.0 else math.sqrt(1.0 + math.log(s) / math.log(original_max_pos))


def rope_tables(max_pos: int, dim: int, theta: float = 10000.0, device=None, **scaling) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables, fp32 [max_pos, dim/2]."""
    attention_factor = scaling.pop("attention_factor", None)
    if str(scaling.get("scaling", "")).lower() in ("longrope", "dynamic_ntk"):
        scaling.setdefault("max_pos", max_pos)
    inv = rope_inv_freq(dim, theta, **scaling)
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv)
    cos, sin = ang.cos(), ang.sin()
    if str(scaling.get("scaling", "")).lower() == "longrope":
        m = attention_factor or longrope_attention_factor(max_pos, scaling.get("original_max_pos", 8192))
        cos, sin = cos * m, sin * m
    return cos.to(device).contiguous(), sin.to(device).contiguous()


def _rope_reference(x, cos, sin, positions, interleaved, sign):
    # x: [rows, n_heads, D]
    D = x.shape[-1]
    c = cos[positions].unsqueeze(1).float()
    s = sin[positions].unsqueeze(1).float() * sign
    xf = x.float()
    if interleaved:
        a, b = xf[..., 0::2], xf[..., 1::2]
        out = torch.stack((a * c - b * s, b * c + a * s), dim=-1).flatten(-2)
    else:
        a, b = xf[..., : D // 2], xf[..., D // 2:]
        out = torch.cat((a * c - b * s, b * c + a * s), dim=-1)
    return out.to(x.dtype)


def _apply_inplace(buf2d, n_heads, D, cos, sin, positions, seq, offset, interleaved, backward):
    rows = buf2d.shape[0]
    if buf2d.is_cuda and buf2d.dtype == torch.bfloat16:
        import ctypes
        lib = _lib.load("elementwise")
        pos = None
        if positions is not None:
            pos = positions.reshape(-1).to(torch.int32)
        rc = lib.ts_rope(_lib.ptr(buf2d), _lib.ptr(cos), _lib.ptr(sin), _lib.ptr(pos), ctypes.c_longlong(rows),
                         buf2d.stride(0), n_heads, D, seq, offset, int(interleaved), int(backward), _lib.stream_ptr())
        _lib.check(rc, "ts_rope")
        return
    if positions is None:
        positions = (torch.arange(rows, device=buf2d.device) % seq) + offset
    else:
        positions = positions.reshape(-1).long()
    v = buf2d[:, : n_heads * D].reshape(rows, n_heads, D)
    out = _rope_reference(v, cos, sin, positions, interleaved, -1.0 if backward else 1.0)
    buf2d[:, : n_heads * D] = out.reshape(rows, n_heads * D)


class _RopeFn(torch.autograd.Function):
    """Out-of-place form: rotates a copy (the input may be a view, a leaf, or needed by somebody else)."""

    @staticmethod
    def forward(ctx, qkv, n_heads, D, cos, sin, positions, seq, offset, interleaved):
        out = qkv.clone()
        buf = out.view(-1, out.shape[-1])
        _apply_inplace(buf, n_heads, D, cos, sin, positions, seq, offset, interleaved, False)
        ctx.args = (n_heads, D, seq, offset, interleaved)
        ctx.save_for_backward(cos, sin, positions)
        return out

    @staticmethod
    def backward(ctx, g):
        cos, sin, positions = ctx.saved_tensors
        n_heads, D, seq, offset, interleaved = ctx.args
        g = g.clone()
        _apply_inplace(g.view(-1, g.shape[-1]), n_heads, D, cos, sin, positions, seq, offset, interleaved, True)
        return g, None, None, None, None, None, None, None, None


class _RopeInplaceFn(torch.autograd.Function):
    """In-place form for the projection output that only the attention reads: no copy in forward (the buffer is
    marked dirty for autograd) and none in backward (the incoming gradient, produced for this node alone by the
    attention backward, is rotated where it is).  One pass over the q|k heads instead of a copy of q|k|v plus a pass."""

    @staticmethod
    def forward(ctx, qkv, n_heads, D, cos, sin, positions, seq, offset, interleaved):
        ctx.mark_dirty(qkv)
        _apply_inplace(qkv.view(-1, qkv.shape[-1]), n_heads, D, cos, sin, positions, seq, offset, interleaved, False)
        ctx.args = (n_heads, D, seq, offset, interleaved)
        ctx.save_for_backward(cos, sin, positions)
        return qkv

    @staticmethod
    def backward(ctx, g):
        cos, sin, positions = ctx.saved_tensors
        n_heads, D, seq, offset, interleaved = ctx.args
        if not g.is_contiguous():
            g = g.contiguous()
        _apply_inplace(g.view(-1, g.shape[-1]), n_heads, D, cos, sin, positions, seq, offset, interleaved, True)
        return g, None, None, None, None, None, None, None, None


def apply_rope_qkv(qkv: torch.Tensor, n_rot_heads: int, head_dim: int, cos: torch.Tensor, sin: torch.Tensor,
                   positions: torch.Tensor | None = None, seq_len: int | None = None, offset: int = 0,
                   interleaved: bool = False, inplace: bool = False) -> torch.Tensor:
    """Rotate the first `n_rot_heads` heads (q heads then k heads) of a fused [..., (Hq+2Hkv)*D] buffer.

    Each k head is rotated once (no per-q-head redundant writes as in the reference's GQA path).
    `positions` ([..., seq] ints) overrides `arange(seq) + offset` for packed documents / CP shards.
    `inplace`: the caller owns `qkv` (a projection output nobody else reads) and allows it to be rotated where it is;
    honoured only when autograd permits it (see below), otherwise a copy is rotated as without the flag.
    """
    seq = seq_len if seq_len is not None else qkv.shape[-2]
    # in place when the buffer is a fresh, contiguous result (not a view of something else, not a leaf that wants a
    # gradient) on the CUDA path; anything else is rotated in a copy
    inplace = (inplace and qkv.is_cuda and qkv.dtype == torch.bfloat16 and qkv._base is None and qkv.is_contiguous()
               and not (qkv.is_leaf and qkv.requires_grad) and not torch.is_inference(qkv))
    fn = _RopeInplaceFn if inplace else _RopeFn
    return fn.apply(qkv, n_rot_heads, head_dim, cos, sin, positions, seq, offset, interleaved)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor | None = None,
               offset: int = 0, interleaved: bool = False) -> torch.Tensor:
    """x: [B, S, H, D] -> rotated copy."""
    B, S, H, D = x.shape
    flat = x.reshape(B * S, H * D)
    out = _RopeFn.apply(flat, H, D, cos, sin, positions, S, offset, interleaved)
    return out.view(B, S, H, D)
