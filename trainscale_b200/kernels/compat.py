"""Remaining names of the reference's kernel layer, on this framework's kernels.

Covers what data_pipeline/trainer/kernels/{rope_kernels,layernorm_kernels,fp8_kernels,flash_attention,fast_lora_mlp,
compiler,triton_kernels}.py export and `kernels/__init__.py` did not have yet.  The reference implements these as
Triton kernels behind `torch.autograd.Function` classes, with PyTorch fallbacks; here each entry point is a thin
adapter (argument order, tensor layout, return convention) over the sm_100a kernels in `ops/`, whose own autograd
functions supply the backward passes.  Nothing here is Triton; names containing "triton" are kept so that code written
against the reference imports unchanged.
"""
from __future__ import annotations

import contextlib
import functools
import gc
from dataclasses import dataclass, field
from typing import Any, Callable, NamedTuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import activation as _act
from ..ops import norm as _norm
from ..ops import rope as _rope

DEFAULT_EPS_RMS, DEFAULT_EPS_LN, MAX_FUSED_SIZE = 1e-6, 1e-5, 65536


# ------------------------------------------------------------------------------------------------ forward / backward pair
class _FunctionPair:
    """Gives an `apply`-style adapter the `forward(ctx, ...)` / `backward(ctx, *grad_outputs)` statics of a
    `torch.autograd.Function`, for code that embeds the op in its own autograd function.  `forward` runs `apply` on
    detached copies of the tensor arguments with gradients enabled and keeps that small graph on `ctx`; `backward`
    differentiates it and returns one gradient (or None) per positional argument.  `ctx` may be any object."""

    @classmethod
    def forward(cls, ctx, *args, **kwargs):
        leaves = [a.detach().requires_grad_(True) if torch.is_tensor(a) and a.is_floating_point() else a for a in args]
        with torch.enable_grad():
            out = cls.apply(*leaves, **kwargs)
        ctx._ts_leaves, ctx._ts_out = leaves, out
        if torch.is_tensor(out):
            return out.detach()
        return tuple(o.detach() if torch.is_tensor(o) else o for o in out)

    @classmethod
    def backward(cls, ctx, *grad_outputs):
        out = ctx._ts_out
        outs = [out] if torch.is_tensor(out) else [o for o in out if torch.is_tensor(o)]
        pairs = [(o, g) for o, g in zip(outs, grad_outputs) if g is not None and o.requires_grad]
        ins = [a for a in ctx._ts_leaves if torch.is_tensor(a) and a.requires_grad]
        got = iter(torch.autograd.grad([o for o, _ in pairs], ins, [g for _, g in pairs], allow_unused=True)
                   if pairs and ins else [None] * len(ins))
        return tuple(next(got) if torch.is_tensor(a) and a.requires_grad else None for a in ctx._ts_leaves)


# ------------------------------------------------------------------------------------------------ device queries
def get_device_capability(device_id: int = 0) -> tuple[int, int]:
    return torch.cuda.get_device_capability(device_id) if torch.cuda.is_available() else (0, 0)


get_cuda_capability = get_device_capability


def supports_bf16(device_id: int = 0) -> bool:
    return get_device_capability(device_id)[0] >= 8


def get_optimal_block_size(head_dim: int) -> int:
    """Smallest of 64 / 128 / 256 that holds a head (the reference's Triton block choice; the rotary kernel here
    vectorises over whole heads and needs no such parameter)."""
    return 64 if head_dim <= 64 else (128 if head_dim <= 128 else 256)


def calculate_settings(n: int) -> tuple[int, int]:
    """(block size, warps) the reference's row kernels would use for rows of `n` values
    (data_pipeline/trainer/kernels/layernorm_kernels.py:69-105): next power of two, capped at 65536.  Informational
    here: the norm kernels pick warp-per-row (n <= 4096) or CTA-per-row themselves."""
    block = 1 << max(0, (max(int(n), 1) - 1).bit_length())
    if block > MAX_FUSED_SIZE:
        raise RuntimeError(f"row of {n} values exceeds the fused-kernel limit of {MAX_FUSED_SIZE}")
    warps = 4 if block < 2048 else (8 if block < 8192 else (16 if block < 32768 else 32))
    return block, warps


def calculate_multi_row_settings(n_cols: int, n_rows: int) -> tuple[int, int, int]:
    """(columns per block, rows per block, warps): several short rows share a block."""
    block_n = max(128, min(1 << max(0, (max(int(n_cols), 1) - 1).bit_length()), 4096))
    block_m = 8 if n_cols <= 256 else (4 if n_cols <= 512 else (2 if n_cols <= 1024 else 1))
    return block_n, max(1, min(block_m, int(n_rows))), 4 if block_n * block_m <= 2048 else 8


def get_layernorm_info() -> dict:
    return {"triton_available": False, "native_kernels": torch.cuda.is_available(),
            "device_capability": get_device_capability(), "max_fused_size": MAX_FUSED_SIZE,
            "default_eps_rms": DEFAULT_EPS_RMS, "default_eps_ln": DEFAULT_EPS_LN}


# ------------------------------------------------------------------------------------------------ rotary embedding
def compute_rope_frequencies(config, seq_len: int, device=None, dtype=torch.float32):
    """(cos, sin) [seq_len, dim / 2] for a `RoPEConfig` with any of its scaling schemes."""
    kind = getattr(config.scaling_type, "value", config.scaling_type)
    cos, sin = _rope.rope_tables(seq_len, config.dim, getattr(config, "theta", 10000.0), device, scaling=kind,
                                 factor=config.scaling_factor,
                                 original_max_pos=getattr(config, "original_max_position", 8192),
                                 long_factor=getattr(config, "longrope_long_factor", None),
                                 short_factor=getattr(config, "longrope_short_factor", None))
    return cos.to(dtype), sin.to(dtype)


def _tables32(cos, sin):
    return cos.float().contiguous(), sin.float().contiguous()


class RoPEFunction(_FunctionPair):
    """`apply(x, cos, sin, position_ids, position_offset, interleaved, inplace)` on x [B, S, H, D]."""

    @staticmethod
    def apply(x, cos, sin, position_ids=None, position_offset: int = 0, interleaved: bool = False,
              inplace: bool = False):
        cos, sin = _tables32(cos, sin)
        out = _rope.apply_rope(x, cos, sin, position_ids, position_offset, interleaved)
        if inplace and not x.requires_grad:
            x.copy_(out)
            return x
        return out


class FusedRoPEQKFunction(_FunctionPair):
    """`apply(Q, K, cos, sin, position_offset, interleaved)` -> (Q', K'); both [B, S, H, D]."""

    @staticmethod
    def apply(Q, K, cos, sin, position_offset: int = 0, interleaved: bool = False):
        cos, sin = _tables32(cos, sin)
        return (_rope.apply_rope(Q, cos, sin, None, position_offset, interleaved),
                _rope.apply_rope(K, cos, sin, None, position_offset, interleaved))


Fast_RoPE = FusedRoPEQKFunction


def apply_rope_qk(Q, K, cos, sin, position_offset: int = 0, interleaved: bool = False):
    return FusedRoPEQKFunction.apply(Q, K, cos, sin, position_offset, interleaved)


class RotaryEmbedding(nn.Module):
    """Rotary-embedding module with cached tables that grow on demand; `scaling_type` none | linear | pi | ntk |
    dynamic_ntk | yarn | llama3 | longrope (data_pipeline/trainer/kernels/rope_kernels.py:1357-1492)."""

    def __init__(self, dim: int, max_seq_len: int = 8192, base: float = 10000.0, scaling_type: str = "none",
                 scaling_factor: float = 1.0, interleaved: bool = False, **kwargs):
        super().__init__()
        from . import RoPEConfig, RoPEScalingType
        kind = {"pi": "linear"}.get(scaling_type.lower(), scaling_type.lower())
        self.dim, self.max_seq_len, self.base, self.interleaved = dim, max_seq_len, base, interleaved
        self.config = RoPEConfig(dim=dim, max_position=max_seq_len, theta=base, scaling_type=RoPEScalingType(kind),
                                 scaling_factor=scaling_factor, interleaved=interleaved, **kwargs)
        cos, sin = compute_rope_frequencies(self.config, max_seq_len)
        self.register_buffer("cos_cached", cos, persistent=False)
        self.register_buffer("sin_cached", sin, persistent=False)

    def _update_cache(self, seq_len: int, device) -> None:
        if seq_len > self.cos_cached.shape[0]:
            self.cos_cached, self.sin_cached = compute_rope_frequencies(self.config, seq_len, device)
        elif self.cos_cached.device != torch.device(device):
            self.cos_cached, self.sin_cached = self.cos_cached.to(device), self.sin_cached.to(device)

    def forward(self, x, position_ids=None, position_offset: int = 0):
        self._update_cache(x.shape[1] + position_offset, x.device)
        return _rope.apply_rope(x, self.cos_cached, self.sin_cached, position_ids, position_offset, self.interleaved)

    def forward_qk(self, Q, K, position_ids=None, position_offset: int = 0):
        self._update_cache(Q.shape[1] + position_offset, Q.device)
        return (_rope.apply_rope(Q, self.cos_cached, self.sin_cached, position_ids, position_offset, self.interleaved),
                _rope.apply_rope(K, self.cos_cached, self.sin_cached, position_ids, position_offset, self.interleaved))

    def get_freqs(self, seq_len: int):
        return self.cos_cached[:seq_len], self.sin_cached[:seq_len]


def _time_cuda(fn, warmup: int, iters: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def benchmark_rope(batch_size: int = 4, seq_len: int = 2048, n_heads: int = 32, head_dim: int = 128,
                   num_warmup: int = 10, num_iters: int = 100, dtype: torch.dtype = torch.bfloat16) -> dict:
    """Mean ms of rotating Q and K [B, S, H, D] and the bandwidth that corresponds to (read + write of both)."""
    if not torch.cuda.is_available():
        raise RuntimeError("benchmark_rope needs a CUDA device")
    Q = torch.randn(batch_size, seq_len, n_heads, head_dim, device="cuda", dtype=dtype)
    K = torch.randn_like(Q)
    cos, sin = _rope.rope_tables(seq_len, head_dim, device="cuda")
    ms = _time_cuda(lambda: apply_rope_qk(Q, K, cos, sin), num_warmup, num_iters)
    return {"mean_ms": ms, "gb_per_s": 4 * Q.numel() * Q.element_size() / ms / 1e6}


# ------------------------------------------------------------------------------------------------ normalisation
class RMSLayerNormFunction(_FunctionPair):
    """`apply(X, weight, eps, compute_weight_grad)`; the weight gradient is always formed when the weight wants one."""

    @staticmethod
    def apply(X, weight, eps: float = DEFAULT_EPS_RMS, compute_weight_grad: bool = True):
        return _norm.rmsnorm(X, weight if compute_weight_grad else weight.detach(), eps)[0]


class LayerNormFunction(_FunctionPair):
    @staticmethod
    def apply(X, weight=None, bias=None, eps: float = DEFAULT_EPS_LN, compute_weight_grad: bool = True):
        if weight is None:
            return F.layer_norm(X, (X.shape[-1],), None, None, eps)
        if not compute_weight_grad:
            weight, bias = weight.detach(), None if bias is None else bias.detach()
        return _norm.layernorm(X, weight, bias, eps)


class FusedAddRMSLayerNormFunction(_FunctionPair):
    """`apply(X, residual, weight, eps, store_residual)` -> (norm(X + residual), X + residual or None): the sum is
    formed inside the norm kernel."""

    @staticmethod
    def apply(X, residual, weight, eps: float = DEFAULT_EPS_RMS, store_residual: bool = True):
        y, h = _norm.rmsnorm(X, weight, eps, residual)
        return y, (h if store_residual else None)


def rms_layernorm(X, weight, eps: float = DEFAULT_EPS_RMS):
    return RMSLayerNormFunction.apply(X, weight, eps, True)


def fused_add_layernorm(X, residual, weight, bias, eps: float = DEFAULT_EPS_LN):
    return LayerNormFunction.apply(X + residual, weight, bias, eps)


class FusedRMSNorm(nn.Module):
    """Residual add + RMSNorm in one kernel; forward(X, residual, return_residual=False)."""

    def __init__(self, hidden_size: int, eps: float = DEFAULT_EPS_RMS, device=None, dtype=torch.float32):
        super().__init__()
        self.hidden_size, self.eps = hidden_size, eps
        self.weight = nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))

    def forward(self, X, residual, return_residual: bool = False):
        y, h = _norm.rmsnorm(X, self.weight, self.eps, residual)
        return (y, h) if return_residual else y

    def extra_repr(self) -> str:
        return f"{self.hidden_size}, eps={self.eps}"


class LayerNorm(nn.Module):
    """Drop-in `torch.nn.LayerNorm` on the row kernel (a multi-dimensional `normalized_shape` takes torch's path)."""

    def __init__(self, normalized_shape, eps: float = DEFAULT_EPS_LN, elementwise_affine: bool = True, bias: bool = True,
                 device=None, dtype=torch.float32):
        super().__init__()
        self.normalized_shape = (normalized_shape,) if isinstance(normalized_shape, int) else tuple(normalized_shape)
        self.eps, self.elementwise_affine = eps, elementwise_affine
        if elementwise_affine:
            self.weight = nn.Parameter(torch.ones(self.normalized_shape, device=device, dtype=dtype))
            self.bias = nn.Parameter(torch.zeros(self.normalized_shape, device=device, dtype=dtype)) if bias else None
        else:
            self.weight = self.bias = None

    def forward(self, X):
        if len(self.normalized_shape) > 1 or self.weight is None:
            return F.layer_norm(X, self.normalized_shape, self.weight, self.bias, self.eps)
        return _norm.layernorm(X, self.weight, self.bias, self.eps)

    def extra_repr(self) -> str:
        return f"{self.normalized_shape}, eps={self.eps}, elementwise_affine={self.elementwise_affine}"


# ------------------------------------------------------------------------------------------------ fp8
class FP8Spec(NamedTuple):
    format: Any
    max_val: float
    dtype: torch.dtype
    mantissa_bits: int
    exponent_bits: int


def get_fp8_spec(fp8_format) -> FP8Spec:
    from . import FP8Format
    if FP8Format(getattr(fp8_format, "value", fp8_format)) is FP8Format.E4M3:
        return FP8Spec(FP8Format.E4M3, 448.0, torch.float8_e4m3fn, 3, 4)
    return FP8Spec(FP8Format.E5M2, 57344.0, torch.float8_e5m2, 2, 5)


class FP8TensorMeta:
    """Delayed-scaling state of one tensor: a ring of recent amax values and the scale derived from their maximum
    (scale = amax / fmax * 2^margin, so that x / scale fills the fp8 range)."""
    __slots__ = ("scale", "scale_inv", "amax", "amax_history", "fp8_spec", "_history_idx")

    def __init__(self, fp8_spec: FP8Spec, device=None, history_len: int = 1024):
        self.fp8_spec = fp8_spec
        self.scale = torch.ones(1, device=device)
        self.scale_inv = torch.ones(1, device=device)
        self.amax = torch.zeros(1, device=device)
        self.amax_history = torch.zeros(history_len, device=device)
        self._history_idx = 0

    def update_amax(self, amax: torch.Tensor) -> None:
        self.amax_history[self._history_idx] = amax.detach().reshape(())
        self._history_idx = (self._history_idx + 1) % self.amax_history.numel()
        self.amax = self.amax_history.max().reshape(1)

    def compute_scale(self, margin: float = 0.0):
        self.scale = self.amax.clamp(min=1e-12) / self.fp8_spec.max_val * (2.0 ** margin)
        self.scale_inv = 1.0 / self.scale
        return self.scale, self.scale_inv


def get_fp8_capability() -> dict:
    cap = get_device_capability()
    return {"cuda_available": torch.cuda.is_available(), "triton_available": False,
            "fp8_hardware": cap >= (8, 9), "native_tcgen05_fp8": cap[0] == 10, "device_capability": cap,
            "device_name": torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu",
            "recommended_block_size": 128}


def fp8_linear_forward(X, weight_fp8, weight_scale, bias=None, block_size: int = 128):
    """X @ dequant(weight_fp8, weight_scale)^T (+ bias) for a block-scaled fp8 weight [N, K] with one fp32 scale per
    `block_size` x `block_size` block.  bf16 CUDA inputs with 128-blocks run the block-scaled tcgen05 GEMM (activations
    quantised per 1 x 128 block on the fly); gradients flow to X."""
    from ..ops import fp8 as fp8_ops
    from ..quantization import _FP8LinearFn
    if block_size == 128 and fp8_ops.available(X) and weight_fp8.dtype == torch.float8_e4m3fn:
        y = fp8_ops.fp8_linear(X, None, weight_fp8, weight_scale)
    else:
        y = _FP8LinearFn.apply(X, weight_fp8, weight_scale, block_size, True)
    return y if bias is None else y + bias


class FP8LinearFunction(_FunctionPair):
    apply = staticmethod(fp8_linear_forward)


def convert_model_to_fp8(model: nn.Module, block_size: int = 128, exclude_layers: list | None = None) -> nn.Module:
    """Replace every `nn.Linear` (except the named ones) by a frozen block-scaled fp8 linear
    (`quantization.FP8Linear`); biases are kept in their dtype."""
    from ..quantization import FP8Linear as _StoredFP8Linear
    skip = set(exclude_layers or [])

    class _WithBias(nn.Module):
        def __init__(self, inner, bias):
            super().__init__()
            self.inner, self.bias = inner, nn.Parameter(bias.detach().clone(), requires_grad=bias.requires_grad)

        def forward(self, x):
            return self.inner(x) + self.bias

    for name, module in list(model.named_modules()):
        if isinstance(module, nn.Linear) and name not in skip and name.rsplit(".", 1)[-1] not in skip:
            parent = model.get_submodule(name.rsplit(".", 1)[0]) if "." in name else model
            q = _StoredFP8Linear(module.weight, block_size)
            setattr(parent, name.rsplit(".", 1)[-1], q if module.bias is None else _WithBias(q, module.bias))
    return model


# ------------------------------------------------------------------------------------------------ flash attention
def is_flash_attn_triton_available() -> bool:
    return False


def get_flash_attn_version() -> str | None:
    """Version of an external flash-attn package in use: none - the attention kernels are the framework's own."""
    return None


def get_attention_backend() -> str:
    from . import supports_tcgen05
    return "tcgen05_flash" if supports_tcgen05() else "reference"


def triton_flash_attention(q, k, v, causal: bool = True, scale: float | None = None,
                           sliding_window: int | None = None):
    """[B, H, M, D] x [B, Hkv, N, D] -> [B, H, M, D] on the flash kernels (GQA when Hkv divides H)."""
    from . import flash_attention
    return flash_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal, scale,
                           sliding_window).transpose(1, 2)


class FlashAttentionTritonFunction(_FunctionPair):
    @staticmethod
    def apply(q, k, v, causal: bool = True, scale: float | None = None, sliding_window: int | None = None,
              num_kv_groups: int = 1):
        if q.shape[1] != k.shape[1] * num_kv_groups:
            raise ValueError(f"{q.shape[1]} query heads, {k.shape[1]} key heads, num_kv_groups={num_kv_groups}")
        return triton_flash_attention(q, k, v, causal, scale, sliding_window)


def benchmark_attention(batch: int = 4, heads: int = 32, seq_len: int = 2048, head_dim: int = 128,
                        dtype: torch.dtype = torch.bfloat16, device: str = "cuda", warmup: int = 10,
                        iterations: int = 100) -> dict:
    """{backend: mean ms} for causal attention [B, H, S, D]: the framework kernel and torch SDPA."""
    if not torch.cuda.is_available():
        raise RuntimeError("benchmark_attention needs a CUDA device")
    q, k, v = (torch.randn(batch, heads, seq_len, head_dim, dtype=dtype, device=device) for _ in range(3))
    out = {"pytorch_sdpa": _time_cuda(lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True), warmup, iterations)}
    if dtype == torch.bfloat16:
        out[get_attention_backend()] = _time_cuda(lambda: triton_flash_attention(q, k, v, True), warmup, iterations)
    return out


# ------------------------------------------------------------------------------------------------ LoRA helpers
def dequantize_weight(W, quant_state=None):
    """The dense weight behind `W`: unchanged without a quantisation state, NF4-unpacked with one
    (`quantization.QuantState`, as `quantize_nf4_param` attaches)."""
    if quant_state is None:
        return W
    from ..quantization import fast_dequantize
    if getattr(quant_state, "absmax", None) is None or getattr(quant_state, "shape", None) is None:
        return W
    return fast_dequantize(W, quant_state.absmax, quant_state.shape, getattr(quant_state, "dtype", torch.bfloat16))


def _lora_parts(module):
    """(W, quant_state, A, B, scaling) of a linear module with optional adapters; understands plain tensors /
    parameters, PEFT's `lora_A.default.weight` nesting and per-adapter scaling dictionaries."""
    W = module.weight
    A, B = getattr(module, "lora_A", None), getattr(module, "lora_B", None)
    for _ in range(2):
        A = getattr(A, "default", A) if not isinstance(A, torch.Tensor) else A
        B = getattr(B, "default", B) if not isinstance(B, torch.Tensor) else B
        A = getattr(A, "weight", A) if not isinstance(A, torch.Tensor) else A
        B = getattr(B, "weight", B) if not isinstance(B, torch.Tensor) else B
    s = getattr(module, "scaling", 1.0)
    s = s.get("default", 1.0) if isinstance(s, dict) else s
    return W, getattr(W, "quant_state", None), A, B, float(s)


def _lora_linear(module, X):
    from . import matmul_lora
    W, qs, A, B, s = _lora_parts(module)
    y = matmul_lora(X, dequantize_weight(W, qs), A, B, s)
    bias = getattr(module, "bias", None)
    return y if bias is None else y + bias


def apply_lora_o(o_proj: nn.Module, X):
    return _lora_linear(o_proj, X)


class FusedLoRAMLP(nn.Module):
    """Gated MLP over existing gate / up / down projection modules (with or without adapters): adapter products are
    accumulated by the GEMM epilogue and the gate runs on the fused GLU kernel."""

    def __init__(self, gate_proj: nn.Module, up_proj: nn.Module, down_proj: nn.Module, inplace: bool = True):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj, self.inplace = gate_proj, up_proj, down_proj, inplace

    def forward(self, X):
        h = _act.swiglu(_lora_linear(self.gate_proj, X), _lora_linear(self.up_proj, X))
        return _lora_linear(self.down_proj, h)


class FusedLoRAQKV(nn.Module):
    def __init__(self, q_proj: nn.Module, k_proj: nn.Module, v_proj: nn.Module, inplace: bool = True):
        super().__init__()
        self.q_proj, self.k_proj, self.v_proj, self.inplace = q_proj, k_proj, v_proj, inplace

    def forward(self, X):
        return _lora_linear(self.q_proj, X), _lora_linear(self.k_proj, X), _lora_linear(self.v_proj, X)


def swiglu_backward(dH, gate, up):
    """For h = silu(gate) * up: returns (h, d_up, d_gate) (the reference's order)."""
    g, u, d = gate.float(), up.float(), dH.float()
    sig = torch.sigmoid(g)
    silu = g * sig
    h = silu * u
    d_up = d * silu
    d_gate = d * u * sig * (1 + g * (1 - sig))
    return h.to(gate.dtype), d_up.to(up.dtype), d_gate.to(gate.dtype)


def swiglu_backward_triton(dH, gate, up):
    """(d_gate, d_up) on the fused GLU backward kernel for bf16 CUDA tensors, else by the formula."""
    I = gate.shape[-1]
    if dH.is_cuda and dH.dtype == torch.bfloat16 and I % 8 == 0:
        gu = torch.cat((gate.reshape(-1, I), up.reshape(-1, I)), dim=-1).contiguous()
        dgu = _act.glu_bwd_raw(dH.reshape(-1, I).contiguous(), gu, _act._ACT["silu"])
        return dgu[:, :I].reshape(gate.shape), dgu[:, I:].reshape(up.shape)
    _, d_up, d_gate = swiglu_backward(dH, gate, up)
    return d_gate, d_up


# ------------------------------------------------------------------------------------------------ compiler surface
@dataclass
class CUDAGraphConfig:
    enabled: bool = True
    warmup_iterations: int = 3
    capture_stream: Any = None
    pool: Any = None
    capture_error_mode: str = "global"


@dataclass
class DynamicShapeConfig:
    """Shape policy of the reference's tracing compiler.  Graph replay here is keyed by the exact input shapes, so
    "dynamic" means one captured graph per distinct shape."""
    enabled: bool = True
    assume_static_by_default: bool = False
    automatic_dynamic_shapes: bool = True
    specialize_int: bool = True
    capture_dynamic_output_shape_ops: bool = True
    capture_scalar_outputs: bool = False


@dataclass
class InductorConfig:
    """Options the reference hands to TorchInductor; recorded and, on request, applied for USER code that calls
    torch.compile itself (`utils.cuda_graphs.InductorConfigManager`).  The framework's own hot path is not traced."""
    triton_cudagraphs: bool = True
    triton_unique_kernel_names: bool = True
    triton_descriptive_names: bool = False
    coordinate_descent_tuning: bool = True
    max_autotune: bool = True
    max_autotune_gemm: bool = True
    max_autotune_pointwise: bool = True
    autotune_in_subproc: bool = True
    fx_graph_cache: bool = True
    fx_graph_remote_cache: bool = False
    epilogue_fusion: bool = True
    shape_padding: bool = True
    extra: dict = field(default_factory=dict)


class CompiledFunctionWrapper:
    """A function run under CUDA-graph replay (one graph per input-shape signature) with an eager fallback: the first
    failure of capture or replay is remembered and the function runs eagerly from then on.  Counts calls, replays and
    fallbacks (`stats`)."""

    def __init__(self, func: Callable, config=None):
        from ..utils.cuda_graphs import CompilationConfig, CUDAGraphManager
        self.func = func
        self.config = config or CompilationConfig()
        self.manager = CUDAGraphManager(self.config)
        self.stats = {"calls": 0, "graph_replays": 0, "eager_calls": 0, "failed": False}
        functools.update_wrapper(self, func)

    def __call__(self, *args, **kwargs):
        self.stats["calls"] += 1
        tensors_only = not kwargs and all(torch.is_tensor(a) or isinstance(a, (int, float, bool, str, type(None)))
                                          for a in args)
        use_graph = (tensors_only and not self.stats["failed"] and not _DISABLED[0] and torch.cuda.is_available()
                     and getattr(self.config, "mode", "cuda_graphs") != "none" and not torch.is_grad_enabled()
                     and any(torch.is_tensor(a) and a.is_cuda for a in args))
        if use_graph:
            try:
                out = self.manager.run(self.func, *args)
                self.stats["graph_replays"] += 1
                return out
            except RuntimeError:
                self.stats["failed"] = True
                self.manager.clear()
        self.stats["eager_calls"] += 1
        return self.func(*args, **kwargs)

    def reset(self) -> None:
        """Forget captured graphs, counters and a remembered failure: the next call tries graph replay again."""
        self.manager.clear()
        self.stats = {"calls": 0, "graph_replays": 0, "eager_calls": 0, "failed": False}


def compile_function(func: Callable, fullgraph: bool = False, dynamic: bool = True, mode: str = "max-autotune",
                     backend: str = "inductor") -> Callable:
    """The reference traces `func` with torch.compile; here it is wrapped for CUDA-graph replay of its launches
    (inference-mode calls on CUDA tensors), which is the launch-overhead remedy this framework has.  `mode="none"` /
    `backend="eager"` return `func` unchanged."""
    if mode in ("none", "default-eager") or backend == "eager":
        return func
    return CompiledFunctionWrapper(func)


def compiled(mode: str = "max-autotune", backend: str = "inductor", fullgraph: bool = False, dynamic: bool = True):
    def decorator(func):
        return compile_function(func, fullgraph, dynamic, mode, backend)
    return decorator


_DISABLED = [False]


@contextlib.contextmanager
def compilation_context(mode: str = "max-autotune", backend: str = "inductor", disable: bool = False):
    """Scope in which calls of `CompiledFunctionWrapper` objects run eagerly (`disable=True`) or as they are."""
    prev = _DISABLED[0]
    _DISABLED[0] = disable
    try:
        yield
    finally:
        _DISABLED[0] = prev


_GLOBAL_COMPILER = [None]


def get_compiler(config=None):
    from ..utils.cuda_graphs import ModelCompiler
    if _GLOBAL_COMPILER[0] is None:
        _GLOBAL_COMPILER[0] = ModelCompiler(config)
    return _GLOBAL_COMPILER[0]


def clear_compilation_cache() -> None:
    """Drop every captured graph of the global compiler and return cached device memory."""
    if _GLOBAL_COMPILER[0] is not None:
        _GLOBAL_COMPILER[0].graphs.clear()
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
