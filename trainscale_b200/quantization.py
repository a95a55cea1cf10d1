"""fp8 / int8 quantisation helpers: 128x128 block and per-row fp8 (E4M3 / E5M2) quantise-dequantise, delayed-scaling
amax history, an `FP8Linear` that stores block-scaled fp8 weights, NF4-style 4-bit dequantisation and memory estimates.

After data_pipeline/trainer/kernels/fp8_kernels.py:144-1055 (block amax -> scale = amax / 448, saturating cast,
row-wise activation quantisation, `FP8Linear`) and data_pipeline/trainer/quantization.py:47-322 (`QuantizationConfig`,
`fast_dequantize`, `estimate_memory_usage`).  On CUDA bf16 inputs `FP8Linear` runs the native block-scaled
kind::f8f6f4 tcgen05 GEMM of ops/fp8.py (forward and dgrad); elsewhere it dequantises block-wise and uses the plain
matmul, which is also the oracle.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum

import torch
import torch.nn as nn

from .ops import gemm

FP8_MAX = {torch.float8_e4m3fn: 448.0, torch.float8_e5m2: 57344.0}


class QuantizationType(Enum):
    """Weight formats a model can be held in (data_pipeline/trainer/quantization.py:29-37)."""
    NONE = "none"
    INT8 = "int8"
    INT4 = "int4"
    FP8_E4M3 = "fp8_e4m3"
    FP8_E5M2 = "fp8_e5m2"
    DYNAMIC = "dynamic"


class QuantizationFormat(Enum):
    """4-bit code books (data_pipeline/trainer/quantization.py:39-43)."""
    NF4 = "nf4"
    FP4 = "fp4"
    INT4 = "int4"


@dataclass
class QuantizationConfig:
    """How the base weights are stored.  The `load_in_*` / `bnb_*` / `llm_int8_*` fields are the reference's
    (data_pipeline/trainer/quantization.py:47-100); `format`, `block_size`, `per_row_activations` and
    `amax_history_len` steer this framework's own fp8 path (`FP8Linear`, `ops/fp8.py`)."""
    bits_override: int | None = None
    format: str = "fp8_e4m3"       # fp8_e4m3 | fp8_e5m2 | int8 | nf4
    block_size: int = 128
    per_row_activations: bool = True
    amax_history_len: int = 16
    load_in_4bit: bool = False
    load_in_8bit: bool = False
    load_in_fp8: bool = False
    bnb_4bit_quant_type: str = "nf4"
    bnb_4bit_compute_dtype: torch.dtype = torch.bfloat16
    bnb_4bit_use_double_quant: bool = True
    fp8_format: str = "e4m3"
    llm_int8_threshold: float = 6.0
    llm_int8_skip_modules: list = field(default_factory=lambda: ["lm_head"])
    llm_int8_has_fp16_weight: bool = False

    def __post_init__(self):
        if self.load_in_4bit + self.load_in_8bit + self.load_in_fp8 > 1:
            raise ValueError("only one of load_in_4bit / load_in_8bit / load_in_fp8 can be set")
        if self.bnb_4bit_quant_type not in ("nf4", "fp4"):
            raise ValueError(f"invalid 4-bit quant type {self.bnb_4bit_quant_type!r}")
        if self.fp8_format not in ("e4m3", "e5m2"):
            raise ValueError(f"invalid fp8 format {self.fp8_format!r}")
        if self.load_in_fp8:
            self.format = f"fp8_{self.fp8_format}"
        elif self.load_in_4bit:
            self.format = self.bnb_4bit_quant_type
        elif self.load_in_8bit:
            self.format = "int8"

    @property
    def is_quantized(self) -> bool:
        return self.load_in_4bit or self.load_in_8bit or self.load_in_fp8

    @property
    def bits(self) -> int:
        if self.bits_override is not None:
            return self.bits_override
        return 4 if self.load_in_4bit else (8 if self.load_in_8bit or self.load_in_fp8 else 16)

    def to_bnb_config(self) -> dict:
        return {"load_in_4bit": self.load_in_4bit, "load_in_8bit": self.load_in_8bit,
                "bnb_4bit_quant_type": self.bnb_4bit_quant_type,
                "bnb_4bit_compute_dtype": self.bnb_4bit_compute_dtype,
                "bnb_4bit_use_double_quant": self.bnb_4bit_use_double_quant,
                "llm_int8_threshold": self.llm_int8_threshold, "llm_int8_skip_modules": list(self.llm_int8_skip_modules)}


def get_4bit_config(compute_dtype: torch.dtype = torch.bfloat16, quant_type: str = "nf4",
                    double_quant: bool = True) -> QuantizationConfig:
    return QuantizationConfig(load_in_4bit=True, bnb_4bit_quant_type=quant_type, bnb_4bit_compute_dtype=compute_dtype,
                              bnb_4bit_use_double_quant=double_quant)


def get_8bit_config(threshold: float = 6.0, skip_modules: list | None = None) -> QuantizationConfig:
    return QuantizationConfig(load_in_8bit=True, llm_int8_threshold=threshold,
                              llm_int8_skip_modules=skip_modules or ["lm_head"])


def get_fp8_config(format: str = "e4m3") -> QuantizationConfig:      # noqa: A002 - the reference's keyword
    return QuantizationConfig(load_in_fp8=True, fp8_format=format)


def get_16bit_config(dtype: torch.dtype = torch.bfloat16) -> QuantizationConfig:
    return QuantizationConfig(bnb_4bit_compute_dtype=dtype)


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


def fast_dequantize(packed: torch.Tensor = None, absmax: torch.Tensor = None, shape=None, dtype=torch.bfloat16, *,
                    weight: torch.Tensor | None = None, quant_state=None, out_dtype=None) -> torch.Tensor:
    """NF4 codes + per-block absmax -> dense tensor.  The reference's form `fast_dequantize(weight, quant_state,
    out_dtype)` is taken too: a floating-point `weight` is only cast; a packed one uses `quant_state` (or the state
    attached to it by `quantize_nf4_param`)."""
    if weight is not None or absmax is None or isinstance(absmax, QuantState):
        weight = weight if weight is not None else packed
        quant_state = quant_state if quant_state is not None else (absmax if isinstance(absmax, QuantState) else None)
        dtype = out_dtype or (shape if isinstance(shape, torch.dtype) else dtype)
        if weight.is_floating_point():
            return weight.to(dtype)
        qs = quant_state or get_quant_state(weight)
        if qs is None:
            raise ValueError("a packed weight needs its quant_state")
        return fast_dequantize(weight, qs.absmax, tuple(qs.shape), dtype)
    dtype = out_dtype or dtype
    hi, lo = (packed >> 4).long(), (packed & 0xF).long()
    idx = torch.stack((hi, lo), dim=-1).flatten(1)
    vals = NF4_LEVELS.to(packed.device)[idx] * absmax.unsqueeze(1)
    n = 1
    for s in shape:
        n *= s
    return vals.reshape(-1)[:n].view(shape).to(dtype)


def estimate_memory_usage(n_params: float = None, weight_bits: int = 16, trainable_fraction: float = 1.0,
                          optimizer_bytes_per_param: float = 12.0, grad_bits: int = 16, *,
                          model_size_billion: float | None = None, config: "QuantizationConfig | None" = None,
                          batch_size: int = 1, seq_length: int = 2048) -> dict:
    """Weights + gradients + optimizer state in GiB.  The reference's form (`model_size_billion`, a
    `QuantizationConfig`, batch size, sequence length - by name, or positionally when the second argument is a config)
    returns its keys: model_gb, lora_gb (2 % of the base), activation_gb, gradient_gb, total_gb
    (data_pipeline/trainer/quantization.py:264-297)."""
    if model_size_billion is not None or isinstance(weight_bits, QuantizationConfig) or weight_bits is None:
        if model_size_billion is None:
            model_size_billion, config = n_params, weight_bits
        config = config if config is not None else QuantizationConfig()       # no configuration: 16-bit weights
        bits = 4 if config.load_in_4bit else 8 if (config.load_in_8bit or getattr(config, "load_in_fp8", False)) else 16
        quantized = bits < 16
        model_gb = model_size_billion * 1e9 * bits / 8 / 2 ** 30
        lora_gb = 0.02 * model_gb
        act_gb = batch_size * seq_length * int(model_size_billion * 1000) * 2 * 4 / 2 ** 30
        grad_gb = lora_gb if quantized else model_gb
        return {"model_gb": round(model_gb, 2), "lora_gb": round(lora_gb, 2), "activation_gb": round(act_gb, 2),
                "gradient_gb": round(grad_gb, 2), "total_gb": round(model_gb + lora_gb + act_gb + grad_gb, 2)}
    gb = 1 / 2 ** 30
    weights = n_params * weight_bits / 8
    grads = n_params * trainable_fraction * grad_bits / 8
    opt = n_params * trainable_fraction * optimizer_bytes_per_param
    return {"weights_gb": weights * gb, "gradients_gb": grads * gb, "optimizer_gb": opt * gb,
            "total_gb": (weights + grads + opt) * gb}


@dataclass
class QuantState:
    """Block-quantisation state of a 4-bit tensor: per-block absmax, the code book, and (double quantisation) the
    state the absmax values themselves were quantised with (data_pipeline/trainer/quantization.py:159-167)."""
    absmax: torch.Tensor
    code: torch.Tensor
    blocksize: int = 64
    dtype: torch.dtype = torch.bfloat16
    shape: tuple | None = None
    offset: torch.Tensor | None = None
    state2: "QuantState | None" = None


def get_quant_state(weight: torch.Tensor) -> QuantState | None:
    """`QuantState` of a weight that carries one (`weight.quant_state`, as bitsandbytes parameters and the tensors
    packed by `quantize_nf4_param` do), else None."""
    qs = getattr(weight, "quant_state", None)
    if qs is None:
        return None
    if isinstance(qs, QuantState):
        return qs
    return QuantState(absmax=getattr(qs, "absmax", None), code=getattr(qs, "code", None),
                      blocksize=getattr(qs, "blocksize", 64), dtype=getattr(qs, "dtype", torch.bfloat16),
                      shape=getattr(qs, "shape", None), offset=getattr(qs, "offset", None))


def quantize_nf4_param(w: torch.Tensor, block: int = 64) -> torch.Tensor:
    """Pack `w` to NF4 and return the packed uint8 tensor with its `quant_state` attached, so that
    `get_quant_state` / `fast_dequantize(packed, qs.absmax, qs.shape)` can restore it."""
    packed, absmax, shape = quantize_nf4(w, block)
    packed.quant_state = QuantState(absmax=absmax, code=NF4_LEVELS.clone(), blocksize=block, dtype=w.dtype,
                                    shape=tuple(shape))
    return packed


def prepare_model_for_quantization(model: nn.Module, config: QuantizationConfig) -> nn.Module:
    """Get a model ready for training on quantised base weights (data_pipeline/trainer/quantization.py:223-249):
    activation checkpointing on where the model offers it, and - when the base is quantised - every remaining
    half-precision parameter that is still trainable (norms, biases, embeddings) promoted to fp32, and inputs made
    to require grad so that checkpointed blocks behind frozen embeddings still back-propagate."""
    if hasattr(model, "gradient_checkpointing_enable"):
        model.gradient_checkpointing_enable()
    if config.is_quantized:
        for p in model.parameters():
            if p.requires_grad and p.dtype in (torch.float16, torch.bfloat16) and p.dim() <= 1:
                p.data = p.data.float()
        if hasattr(model, "enable_input_require_grads"):
            model.enable_input_require_grads()
    return model


_LORA_TARGETS = {
    "phi": ["q_proj", "k_proj", "v_proj", "dense", "fc1", "fc2"],
    "gpt2": ["c_attn", "c_proj", "c_fc"],
    "falcon": ["query_key_value", "dense", "dense_h_to_4h", "dense_4h_to_h"],
}


def get_target_modules(model_type: str) -> list[str]:
    """Default LoRA target modules of a model family (data_pipeline/trainer/quantization.py:252-261): the seven
    projections for the Llama-shaped families, family-specific names otherwise, q/v for unknown types."""
    mt = (model_type or "").lower()
    for fam in ("llama", "qwen", "gemma", "mistral", "mixtral", "yi", "deepseek"):
        if fam in mt:
            return ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]
    for fam, t in _LORA_TARGETS.items():
        if fam in mt:
            return list(t)
    return ["q_proj", "v_proj"]
