"""fp8 / int8 quantisation helpers: 128x128 block and per-row fp8 (E4M3 / E5M2) quantise-dequantise, delayed-scaling
amax history, an `FP8Linear` that stores block-scaled fp8 weights, NF4-style 4-bit dequantisation and memory estimates.

After data_pipeline/trainer/kernels/fp8_kernels.py:144-1055 (block amax -> scale = amax / 448, saturating cast,
row-wise activation quantisation, `FP8Linear`) and data_pipeline/trainer/quantization.py:47-322 (`QuantizationConfig`,
`fast_dequantize`, `estimate_memory_usage`).  On CUDA bf16 inputs `FP8Linear` runs the native block-scaled
kind::f8f6f4 tcgen05 GEMM of ops/fp8.py (forward and dgrad); elsewhere it dequantises block-wise and uses the plain
matmul, which is also the oracle.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from .ops import gemm

FP8_MAX = {torch.float8_e4m3fn: 448.0, torch.float8_e5m2: 57344.0}


@dataclass
class QuantizationConfig:
    bits: int = 8
    format: str = "fp8_e4m3"       # fp8_e4m3 | fp8_e5m2 | int8 | nf4
    block_size: int = 128
    per_row_activations: bool = True
    amax_history_len: int = 16


def block_quantize_fp8(w: torch.Tensor, block: int = 128, dtype=torch.float8_e4m3fn):
    """w [M, N] -> (q fp8 [M, N], scales fp32 [ceil(M/b), ceil(N/b)]) with w ~= q * scale (per 128x128 block)."""
    M, N = w.shape
    mb, nb = -(-M // block), -(-N // block)
    pad = torch.zeros(mb * block, nb * block, dtype=torch.float32, device=w.device)
    pad[:M, :N] = w.float()
    blocks = pad.view(mb, block, nb, block)
    amax = blocks.abs().amax(dim=(1, 3)).clamp(min=1e-12)
    scale = amax / FP8_MAX[dtype]
    q = (blocks / scale[:, None, :, None]).clamp(-FP8_MAX[dtype], FP8_MAX[dtype]).to(dtype)
    return q.view(mb * block, nb * block)[:M, :N].contiguous(), scale


def block_dequantize_fp8(q: torch.Tensor, scale: torch.Tensor, block: int = 128, dtype=torch.bfloat16) -> torch.Tensor:
    M, N = q.shape
    s = scale.repeat_interleave(block, 0)[:M].repeat_interleave(block, 1)[:, :N]
    return (q.float() * s).to(dtype)


def row_quantize_fp8(x: torch.Tensor, dtype=torch.float8_e4m3fn):
    """Per-row (per-token) quantisation: (q, scale [rows, 1])."""
    amax = x.float().abs().amax(dim=-1, keepdim=True).clamp(min=1e-12)
    scale = amax / FP8_MAX[dtype]
    return (x.float() / scale).clamp(-FP8_MAX[dtype], FP8_MAX[dtype]).to(dtype), scale


def row_dequantize_fp8(q: torch.Tensor, scale: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    return (q.float() * scale).to(dtype)


class AmaxHistory:
    """Delayed scaling: scale for step t comes from the max amax of the last `length` steps."""

    def __init__(self, length: int = 16, dtype=torch.float8_e4m3fn, margin: float = 0.0):
        self.length, self.dtype, self.margin = length, dtype, margin
        self.history: list[float] = []

    def update(self, x: torch.Tensor) -> None:
        self.history.append(float(x.detach().abs().max()))
        self.history = self.history[-self.length:]

    def scale(self) -> float:
        amax = max(self.history) if self.history else 1.0
        return max(amax, 1e-12) * (2.0 ** self.margin) / FP8_MAX[self.dtype]


class _FP8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, wq, wscale, block, quantize_act):
        w = block_dequantize_fp8(wq, wscale, block, x.dtype)
        if quantize_act:
            xq, xs = row_quantize_fp8(x.reshape(-1, x.shape[-1]))
            x_used = row_dequantize_fp8(xq, xs, x.dtype).view_as(x)
        else:
            x_used = x
        ctx.save_for_backward(w)
        return gemm.linear(x_used, w)

    @staticmethod
    def backward(ctx, dy):
        (w,) = ctx.saved_tensors
        dx = gemm.matmul_nn(dy.reshape(-1, dy.shape[-1]), w) if dy.is_cuda and dy.dtype == torch.bfloat16 \
            else dy.reshape(-1, dy.shape[-1]) @ w
        return dx.view(*dy.shape[:-1], w.shape[1]), None, None, None, None


class FP8Linear(nn.Module):
    """Frozen block-scaled fp8 weight (1 byte / parameter + one fp32 scale per 128x128 block); gradients flow to the
    input (adapters / earlier layers train), as in the reference's FP8Linear."""

    def __init__(self, weight: torch.Tensor, block: int = 128, dtype=torch.float8_e4m3fn, quantize_activations: bool = True):
        super().__init__()
        q, s = block_quantize_fp8(weight.detach(), block, dtype)
        self.register_buffer("weight_q", q)
        self.register_buffer("weight_scale", s)
        self.block, self.quantize_activations = block, quantize_activations
        self.out_features, self.in_features = weight.shape

    def forward(self, x):
        from .ops import fp8 as fp8_ops
        if self.block == 128 and self.quantize_activations and fp8_ops.available(x) \
                and self.weight_q.dtype == torch.float8_e4m3fn:
            return fp8_ops.fp8_linear(x, None, self.weight_q, self.weight_scale)
        return _FP8LinearFn.apply(x, self.weight_q, self.weight_scale, self.block, self.quantize_activations)

    def dequantized_weight(self, dtype=torch.bfloat16):
        return block_dequantize_fp8(self.weight_q, self.weight_scale, self.block, dtype)


NF4_LEVELS = torch.tensor([-1.0, -0.6961928, -0.5250730, -0.3949175, -0.2844414, -0.1848449, -0.0910500, 0.0, 0.0795803,
                           0.1609302, 0.2461123, 0.3379152, 0.4407098, 0.5626170, 0.7229568, 1.0])


def quantize_nf4(w: torch.Tensor, block: int = 64):
    flat = w.float().reshape(-1)
    pad = (-flat.numel()) % block
    flat = torch.cat((flat, flat.new_zeros(pad))).view(-1, block)
    absmax = flat.abs().amax(1, keepdim=True).clamp(min=1e-12)
    idx = ((flat / absmax).unsqueeze(-1) - NF4_LEVELS.to(w.device)).abs().argmin(-1).to(torch.uint8)
    packed = (idx[:, 0::2] << 4) | idx[:, 1::2]
    return packed, absmax.squeeze(1), w.shape


def fast_dequantize(packed: torch.Tensor, absmax: torch.Tensor, shape, dtype=torch.bfloat16) -> torch.Tensor:
    hi, lo = (packed >> 4).long(), (packed & 0xF).long()
    idx = torch.stack((hi, lo), dim=-1).flatten(1)
    vals = NF4_LEVELS.to(packed.device)[idx] * absmax.unsqueeze(1)
    n = 1
    for s in shape:
        n *= s
    return vals.reshape(-1)[:n].view(shape).to(dtype)


def estimate_memory_usage(n_params: float, weight_bits: int = 16, trainable_fraction: float = 1.0,
                          optimizer_bytes_per_param: float = 12.0, grad_bits: int = 16) -> dict:
    gb = 1 / 2 ** 30
    weights = n_params * weight_bits / 8
    grads = n_params * trainable_fraction * grad_bits / 8
    opt = n_params * trainable_fraction * optimizer_bytes_per_param
    return {"weights_gb": weights * gb, "gradients_gb": grads * gb, "optimizer_gb": opt * gb,
            "total_gb": (weights + grads + opt) * gb}
