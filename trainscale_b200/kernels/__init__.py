"""The kernel layer under the reference's names (data_pipeline/trainer/kernels/__init__.py:13-270): functional entry
points, `autograd.Function` classes and `nn.Module` wrappers for normalisation, activations, cross-entropy, attention,
rotary embeddings, fused LoRA, MoE, fp8 and the collective helpers, plus the capability probe.

Everything here forwards to `trainscale_b200.ops` (hand-written sm_100a kernels: tcgen05 GEMM / attention, TMA, fused
row kernels) with PyTorch maths as the CPU fall-back.  There is no Triton in this framework: `is_triton_available()`
is False by construction and the `Triton*` module names are kept only so that code written against the reference
imports unchanged.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from enum import Enum
from typing import List, NamedTuple, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import activation as _act
from ..ops import attention as _attn
from ..ops import cross_entropy as _ce
from ..ops import fp8 as _fp8
from ..ops import gemm as _gemm
from ..ops import moe as _moe
from ..ops import norm as _norm
from ..ops import rope as _rope
from ..losses import FusedCrossEntropyFunction  # noqa: F401
from ..utils.explicit_backward import ExplicitBackward as _ExplicitBackward
from ..utils.refargs import ANY, reference_kwargs
from ..parallel.dist_kernels import (DistributedBackend, DistributedConfig, DistributedKernels,  # noqa: F401
                                     get_distributed_backend, get_world_info, pinned_memory_transfer)
from ..utils.cuda_graphs import CompilationConfig, compile_model  # noqa: F401
from ..utils.cuda_graphs import InductorConfigManager as InductorConfig  # noqa: F401


# ------------------------------------------------------------------------------------------------ capabilities
class CompilationMode(str, Enum):
    DEFAULT = "default"
    REDUCE_OVERHEAD = "reduce-overhead"
    MAX_AUTOTUNE = "max-autotune"


class CompilationBackend(str, Enum):
    CUDA_GRAPHS = "cuda_graphs"
    EAGER = "none"


class PrecisionMode(str, Enum):
    FP32 = "fp32"
    BF16 = "bf16"
    FP8 = "fp8"


class AcceleratorArch(str, Enum):
    BLACKWELL = "blackwell"
    HOPPER = "hopper"
    AMPERE = "ampere"
    OTHER = "other"
    CPU = "cpu"


def is_triton_available() -> bool:
    return False


@reference_kwargs(device_id="device")
def get_accelerator_arch(device: int = 0) -> AcceleratorArch:
    if not torch.cuda.is_available():
        return AcceleratorArch.CPU
    major = torch.cuda.get_device_capability(device)[0]
    return {10: AcceleratorArch.BLACKWELL, 9: AcceleratorArch.HOPPER, 8: AcceleratorArch.AMPERE}.get(
        major, AcceleratorArch.OTHER)


@reference_kwargs(device_id="device")
def supports_tma(device: int = 0) -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_capability(device)[0] >= 9


@reference_kwargs(device_id="device")
def supports_wgmma(device: int = 0) -> bool:
    """wgmma is the Hopper instruction; Blackwell's tensor-core path is tcgen05 (see `supports_tcgen05`)."""
    return torch.cuda.is_available() and torch.cuda.get_device_capability(device)[0] == 9


def supports_tcgen05(device: int = 0) -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_capability(device)[0] == 10


def get_kernel_capabilities() -> dict[str, bool]:
    """What the kernel layer can run on this machine (the CUDA libraries need an sm_100 device)."""
    from ..ops.build import lib_path, sources
    built = {src.stem: lib_path(src.stem).exists() for src in sources()}
    gpu = supports_tcgen05()
    return {"cuda": torch.cuda.is_available(), "triton": False, "tma": supports_tma(), "wgmma": supports_wgmma(),
            "tcgen05": gpu, "bf16": True, "fp8": gpu and built.get("fp8", False),
            "flash_attention": gpu and built.get("attention", False), "fused_layernorm": gpu and built.get("elementwise", False),
            "fused_cross_entropy": gpu and built.get("elementwise", False), "grouped_gemm": gpu and built.get("gemm", False),
            "moe": gpu and built.get("moe", False), "fused_collectives": gpu and built.get("comm", False),
            "fused_tp_gemm": gpu and built.get("tp_gemm", False), "optimizer_kernels": gpu and built.get("optim", False),
            "libraries_built": all(built.values()) if built else False}


# ------------------------------------------------------------------------------------------------ normalisation / activations
@dataclass
class LayerNormConfig:
    eps: float = 1e-5
    elementwise_affine: bool = True
    bias: bool = True
    rms: bool = False


def fused_layer_norm(x, weight, bias=None, eps: float = 1e-5):
    return _norm.layernorm(x, weight, bias, eps)


@reference_kwargs(X="x")
def fast_rms_layernorm(x, weight, eps: float = 1e-6, gemma: bool = False):
    return _norm.rmsnorm(x, weight, eps, None, 1.0 if gemma else 0.0)[0]


@reference_kwargs(X="x")
def fused_add_rms_layernorm(x, residual, weight, eps: float = 1e-6, return_residual: bool = False):
    """norm(x + residual), the sum being formed inside the norm kernel; with `return_residual` the pair
    (norm(x + residual), x + residual)."""
    y, h = _norm.rmsnorm(x, weight, eps, residual)
    return (y, h) if return_residual else y


def layernorm(X, weight=None, bias=None, eps: float = 1e-5):
    """LayerNorm over the last dimension with the reference's argument names
    (data_pipeline/trainer/kernels/layernorm_kernels.py); the op itself is `ops.norm.layernorm`."""
    if weight is None:
        return F.layer_norm(X, (X.shape[-1],), None, None, eps)
    return _norm.layernorm(X, weight, bias, eps)


def fused_softmax(x, dim: int = -1):
    return _act.softmax(x, dim)


@reference_kwargs(approx="approximate")
def fused_gelu(x, approximate: str | bool = "tanh"):
    """`approximate`: "tanh" / "none" (or the reference's boolean: True = tanh form)."""
    if isinstance(approximate, bool):
        approximate = "tanh" if approximate else "none"
    return _act.gelu(x, approximate)


def swiglu_forward(gate, up):
    return _act.swiglu(gate, up)


@reference_kwargs(approx="approximate")
def geglu_forward(gate, up, approximate: str | bool = "tanh"):
    if isinstance(approximate, bool):
        approximate = "tanh" if approximate else "none"
    return _act.glu(torch.cat((gate, up), dim=-1), "gelu_tanh" if approximate == "tanh" else "gelu")


def fast_cross_entropy_loss(logits, labels, ignore_index: int = -100, label_smoothing: float = 0.0,
                            reduction: str = "mean", logit_softcapping: float = 0.0, logit_scaling: float = 0.0,
                            n_items: int | None = None):
    """logits [..., V], labels [...] -> scalar (mean over non-ignored tokens) or per-token losses (reduction="none").
    `logit_scaling` multiplies and `logit_softcapping` (c tanh(z / c)) caps the logits first; `n_items` replaces the
    count of non-ignored tokens as the mean's denominator (data_pipeline/trainer/kernels/triton_kernels.py:427)."""
    if logit_scaling:
        logits = logits * logit_scaling
    if logit_softcapping:
        logits = logit_softcapping * torch.tanh(logits / logit_softcapping)
    z, y = logits.reshape(-1, logits.shape[-1]), labels.reshape(-1)
    if z.is_cuda and z.dtype == torch.bfloat16:
        rows = _ce.cross_entropy_rows(z, y, ignore_index, label_smoothing)
    else:
        rows = F.cross_entropy(z.float(), y, ignore_index=ignore_index, label_smoothing=label_smoothing, reduction="none")
    if reduction == "none":
        return rows.view(labels.shape)
    s = rows.sum()
    if reduction != "mean":
        return s
    return s / (n_items if n_items is not None else (y != ignore_index).sum().clamp(min=1))


# ---- `apply`-style entry points with the reference's argument order (data_pipeline/trainer/kernels/triton_kernels.py);
# the backward passes are those of the ops underneath.  `forward(ctx, ...)` / `backward(ctx, ...)` exist for code that
# embeds the op in its own autograd function.
from .compat import _FunctionPair  # noqa: E402


class Fast_RMS_LayerNorm(_FunctionPair):
    """`apply(X, weight, eps)` -> RMS-normalised X."""

    @staticmethod
    def apply(X, weight, eps: float = 1e-6):
        return _norm.rmsnorm(X, weight, eps)[0]

    @classmethod
    def forward(cls, ctx, X, weight, eps: float = 1e-6):
        return super().forward(ctx, X, weight, eps)

    @classmethod
    def backward(cls, ctx, dY):
        return super().backward(ctx, dY)


class Fast_SwiGLU(_FunctionPair):
    """`apply(gate, up)` -> silu(gate) * up."""

    @staticmethod
    def apply(gate, up):
        return _act.swiglu(gate, up)

    @classmethod
    def forward(cls, ctx, gate, up):
        return super().forward(ctx, gate, up)


class Fast_GeGLU(_FunctionPair):
    """`apply(gate, up, approx=False)` -> gelu(gate) * up (tanh approximation when `approx`)."""

    @staticmethod
    def apply(gate, up, approx: bool = False):
        return geglu_forward(gate, up, bool(approx))

    @classmethod
    def forward(cls, ctx, gate, up, approx: bool = False):
        return super().forward(ctx, gate, up, approx)


class Fast_CrossEntropyLoss(_FunctionPair):
    """`apply(logits [N, V], labels [N], logit_softcapping=0, logit_scaling=0)` -> per-row losses [N] (0 for ignored
    rows); the mean over the non-ignored rows is `fast_cross_entropy_loss`."""

    @staticmethod
    def apply(logits, labels, logit_softcapping: float = 0.0, logit_scaling: float = 0.0):
        return fast_cross_entropy_loss(logits, labels, reduction="none", logit_softcapping=logit_softcapping,
                                       logit_scaling=logit_scaling)

    @classmethod
    def forward(cls, ctx, logits, labels, logit_softcapping: float = 0.0, logit_scaling: float = 0.0):
        return super().forward(ctx, logits, labels, logit_softcapping, logit_scaling)

    @classmethod
    def backward(cls, ctx, dlosses):
        return super().backward(ctx, dlosses)


class TritonRMSNorm(nn.Module):
    """RMSNorm module on the fused row kernel (name kept from the reference; nothing here is Triton)."""

    def __init__(self, hidden_size: int, eps: float = 1e-6, dtype=None, device=None, *, elementwise_affine: bool = True):
        """`elementwise_affine=False`: no learnable scale (the kernel runs with a constant vector of ones)."""
        super().__init__()
        if isinstance(dtype, bool):                          # RMSNorm(hidden_size, eps, elementwise_affine, device, dtype)
            elementwise_affine, dtype = dtype, None
        if device is not None and isinstance(device, torch.dtype):
            dtype, device = device, None
        self.hidden_size, self.eps, self.elementwise_affine = hidden_size, eps, bool(elementwise_affine)
        ones = torch.ones(hidden_size, dtype=dtype, device=device)
        if self.elementwise_affine:
            self.weight = nn.Parameter(ones)
        else:
            self.register_parameter("weight", None)
            self.register_buffer("_ones", ones, persistent=False)

    @reference_kwargs(X="x")
    def forward(self, x, residual=None):
        w = self.weight if self.weight is not None else self._ones.to(x.dtype)
        y, res = _norm.rmsnorm(x, w, self.eps, residual)
        return y if residual is None else (y, res)


class TritonSwiGLU(nn.Module):
    """Gated MLP: down(silu(gate(x)) * up(x)) with gate|up as one GEMM and the fused gate kernel."""

    activation = "silu"

    def __init__(self, hidden_size: int, intermediate_size: int, dtype=None, device=None, *, bias: bool = False):
        """`bias=True` adds biases to the gate|up and the down projections (`TritonSwiGLU(hidden, inter, bias)` is
        the reference's positional form)."""
        super().__init__()
        if isinstance(dtype, bool):
            bias, dtype = dtype, None
        self.w_gate_up = nn.Parameter(torch.empty(2 * intermediate_size, hidden_size, dtype=dtype, device=device))
        self.w_down = nn.Parameter(torch.empty(hidden_size, intermediate_size, dtype=dtype, device=device))
        self.b_gate_up = nn.Parameter(torch.zeros(2 * intermediate_size, dtype=dtype, device=device)) if bias else None
        self.b_down = nn.Parameter(torch.zeros(hidden_size, dtype=dtype, device=device)) if bias else None
        nn.init.normal_(self.w_gate_up, std=0.02)
        nn.init.normal_(self.w_down, std=0.02)

    def forward(self, x):
        return _gemm.linear(_act.glu(_gemm.linear(x, self.w_gate_up, self.b_gate_up), self.activation), self.w_down,
                            self.b_down)


class TritonGeGLU(TritonSwiGLU):
    """`approx=True` (default): the tanh approximation of GELU; `approx=False`: the exact erf form."""
    activation = "gelu_tanh"

    def __init__(self, hidden_size: int, intermediate_size: int, dtype=None, device=None, *, bias: bool = False,
                 approx: bool = True):
        if isinstance(dtype, bool) and isinstance(device, bool):          # (hidden, inter, bias, approx)
            bias, approx, dtype, device = dtype, device, None, None
        super().__init__(hidden_size, intermediate_size, dtype, device, bias=bias)
        self.approx = bool(approx)
        self.activation = "gelu_tanh" if approx else "gelu"


RMSNorm, SwiGLU, GeGLU = TritonRMSNorm, TritonSwiGLU, TritonGeGLU


# ------------------------------------------------------------------------------------------------ attention
class AttentionMaskType(str, Enum):
    CAUSAL = "causal"
    FULL = "full"
    SLIDING_WINDOW = "sliding_window"
    DOCUMENT = "document"


class AttentionBackend(str, Enum):
    TCGEN05_FLASH = "tcgen05_flash"       # the framework kernel (bf16, head_dim 64 / 128)
    REFERENCE = "reference"               # fp32 PyTorch maths


class AttentionOutput(NamedTuple):
    output: torch.Tensor
    lse: torch.Tensor | None = None


@dataclass
class FlashAttentionConfig:
    causal: bool = True
    softmax_scale: float | None = None
    window_size: int | None = None
    softcap: float = 0.0
    dropout: float = 0.0                  # not supported by the kernel; must stay 0
    head_dim: int | None = None
    num_heads: int | None = None
    num_kv_heads: int | None = None       # fewer than num_heads: grouped-query / multi-query attention
    sliding_window: int | None = None     # the reference's name for window_size

    def __post_init__(self):
        if self.sliding_window is not None and self.window_size is None:
            self.window_size = self.sliding_window
        self.sliding_window = self.window_size
        if self.num_heads and self.num_kv_heads and self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be divisible by num_kv_heads")

    @property
    def scale(self) -> float:
        """softmax_scale, or 1 / sqrt(head_dim) (data_pipeline/trainer/kernels/flash_attention.py:98-100)."""
        if self.softmax_scale:
            return self.softmax_scale
        if not self.head_dim:
            raise ValueError("scale needs softmax_scale or head_dim")
        return 1.0 / math.sqrt(self.head_dim)

    @property
    def num_kv_groups(self) -> int:
        return 1 if not (self.num_heads and self.num_kv_heads) else self.num_heads // self.num_kv_heads

    @property
    def is_gqa(self) -> bool:
        return bool(self.num_heads and self.num_kv_heads and self.num_kv_heads < self.num_heads)

    @property
    def mask_type(self) -> "AttentionMaskType":
        return (AttentionMaskType.SLIDING_WINDOW if self.window_size else
                AttentionMaskType.CAUSAL if self.causal else AttentionMaskType.FULL)


@dataclass
class FlexAttentionConfig(FlashAttentionConfig):
    """`mask_type` / `backend` select the kernel switches of `FlexAttention`; the remaining fields are the reference's
    (data_pipeline/trainer/kernels/flex_attention.py:58-99) and are what the functions of `kernels/flex.py` read."""
    mask_type: AttentionMaskType = AttentionMaskType.CAUSAL
    backend: AttentionBackend | None = None
    num_attention_heads: int | None = None
    num_key_value_heads: int | None = None
    head_dim: int | None = None
    query_pre_attn_scalar: float = 1.0
    attn_logit_softcapping: float = 0.0
    sliding_window_size: int | None = None
    max_seq_length: int = 8192
    precision_mode: "PrecisionMode" = None
    use_flash_attention: bool = True
    use_triton_kernels: bool = False
    enable_kv_cache: bool = True
    page_size: int = 16
    block_size: int = 128
    dropout_p: float = 0.0
    deterministic: bool = True

    def __post_init__(self):
        super().__post_init__()
        if self.num_attention_heads and self.num_key_value_heads and \
                self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("num_attention_heads must be divisible by num_key_value_heads")
        if self.precision_mode is None:
            self.precision_mode = PrecisionMode.BF16
        if self.attn_logit_softcapping and not self.softcap:
            self.softcap = self.attn_logit_softcapping
        if self.sliding_window_size and not self.window_size:
            self.window_size = self.sliding_window_size

    @property
    def num_kv_groups(self) -> int:
        return (self.num_attention_heads or 1) // (self.num_key_value_heads or self.num_attention_heads or 1)

    @property
    def hidden_size(self) -> int:
        return (self.num_attention_heads or 0) * (self.head_dim or 0)

    @property
    def kv_hidden_size(self) -> int:
        return (self.num_key_value_heads or self.num_attention_heads or 0) * (self.head_dim or 0)


@dataclass
class BackendCapabilities:
    backend: AttentionBackend
    head_dims: tuple = (64, 128)
    sliding_window: bool = True
    softcap: bool = True
    varlen: bool = True
    gqa: bool = True

    @classmethod
    def detect(cls) -> "BackendCapabilities":
        return cls(AttentionBackend.TCGEN05_FLASH if supports_tcgen05() else AttentionBackend.REFERENCE)

    # ---- the reference's probes (data_pipeline/trainer/kernels/flex_attention.py:199-258).  The `has_*` names
    # describe CAPABILITIES of this framework's own kernels; no flash-attn, Triton or xformers package is on any path.
    @property
    def has_flex_attention(self) -> bool:
        """Block-mask attention (`kernels.flex`) is always present: tcgen05 kernels on sm_100, fp32 maths elsewhere."""
        return True

    @property
    def has_flash_attention_2(self) -> bool:
        return self.backend is AttentionBackend.TCGEN05_FLASH

    has_flash_attention_3 = has_flash_attention_2

    @property
    def has_triton(self) -> bool:
        return False

    @property
    def cuda_capability(self) -> tuple | None:
        return torch.cuda.get_device_capability() if torch.cuda.is_available() else None

    @property
    def supports_fp8(self) -> bool:
        cap = self.cuda_capability
        return cap is not None and cap >= (8, 9)

    @property
    def supports_bf16(self) -> bool:
        cap = self.cuda_capability
        return cap is not None and cap >= (8, 0)

    @property
    def flex_attention_fn(self):
        from .flex import flex_attention_forward
        return flex_attention_forward

    @property
    def create_block_mask_fn(self):
        from .flex import create_block_mask
        return create_block_mask

    def select_optimal_backend(self, config=None) -> AttentionBackend:
        """The tcgen05 flash kernels when the device has them and the head dimension is one they are built for
        (soft-capping, windows, GQA and packed documents are all switches of the same kernels); fp32 maths otherwise."""
        hd = getattr(config, "head_dim", None)
        ok = self.backend is AttentionBackend.TCGEN05_FLASH and (hd is None or hd in self.head_dims)
        return AttentionBackend.TCGEN05_FLASH if ok else AttentionBackend.REFERENCE


def is_flash_attn_available() -> bool:
    """True when the framework's own flash kernels can run (an sm_100 GPU); no external flash-attn package is used."""
    return supports_tcgen05()


def flash_attention(q=None, k=None, v=None, causal: bool | None = None, softmax_scale: float | None = None,
                    window_size: int | None = None, softcap: float = 0.0, cu_seqlens: torch.Tensor | None = None, *,
                    query=None, key=None, value=None, dropout_p: float = 0.0, scale: float | None = None,
                    sliding_window: int | None = None, return_softmax: bool = False):
    """q [B, S, Hq, D], k / v [B, S, Hkv, D] -> [B, S, Hq, D], causal unless told otherwise.  bf16 CUDA inputs run the
    tcgen05 flash kernels (forward and backward); anything else the fp32 reference.

    The reference's keyword form `flash_attention(query=, key=, value=, causal=False, scale=, sliding_window=)` uses ITS
    conventions: [B, H, S, D] tensors in and out, not causal unless asked, and `return_softmax=True` wraps the result
    in `AttentionOutput` (data_pipeline/trainer/kernels/flash_attention.py:795).  Dropout is not implemented."""
    if dropout_p:
        raise NotImplementedError("attention dropout is not supported by this framework")
    if query is not None:
        o = flash_attention(query.transpose(1, 2).contiguous(), key.transpose(1, 2).contiguous(),
                            value.transpose(1, 2).contiguous(), bool(causal), scale if scale is not None else softmax_scale,
                            sliding_window if sliding_window is not None else window_size, softcap).transpose(1, 2)
        return AttentionOutput(o) if return_softmax else o
    causal = True if causal is None else causal
    softmax_scale = softmax_scale if softmax_scale is not None else scale
    window_size = window_size if window_size is not None else sliding_window
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    if q.is_cuda and q.dtype == torch.bfloat16 and k.shape[1] == S:
        qkv = torch.cat((q.reshape(B, S, -1), k.reshape(B, S, -1), v.reshape(B, S, -1)), dim=-1)
        return _attn.attention_qkv(qkv, Hq, Hkv, D, causal, softmax_scale, window_size, softcap, cu_seqlens) \
            .view(B, S, Hq, D)
    doc = None
    if cu_seqlens is not None:
        idx = torch.arange(B * S, device=q.device)
        doc = torch.bucketize(idx, cu_seqlens[1:].to(idx.dtype), right=True).view(B, S)
    return _attn.attention_reference(q, k, v, causal, softmax_scale, window_size, softcap, doc).to(q.dtype)


def naive_attention(q=None, k=None, v=None, causal: bool = True, softmax_scale: float | None = None, *, query=None,
                    key=None, value=None, dropout_p: float = 0.0, scale: float | None = None, attn_mask=None):
    """fp32 attention maths.  Positional / q-k-v form: [B, S, H, D], causal by default.  The reference's keyword form
    (`query=, key=, value=`) uses ITS layout, [B, H, S, D], and takes an additive or boolean `attn_mask`
    (data_pipeline/trainer/kernels/flash_attention.py:895).  Dropout is not implemented (dropout_p must be 0)."""
    if dropout_p:
        raise NotImplementedError("attention dropout is not supported by this framework")
    if query is not None:
        if attn_mask is not None:
            return F.scaled_dot_product_attention(query.float(), key.float(), value.float(), attn_mask=attn_mask,
                                                  is_causal=False, scale=scale).to(query.dtype)
        o = _attn.attention_reference(query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2), causal, scale)
        return o.transpose(1, 2).to(query.dtype)
    return _attn.attention_reference(q, k, v, causal, softmax_scale if softmax_scale is not None else scale).to(q.dtype)


def _reference_flash_attention(query, key, value, causal: bool = False, dropout_p: float = 0.0, scale: float | None = None,
                               sliding_window: int | None = None, return_softmax: bool = False, **options):
    """`flash_attention` in the reference's positional order and conventions ([B, H, S, D], not causal by default);
    what `from data_pipeline.trainer.kernels import flash_attention` gives under `reference_paths`."""
    return flash_attention(query=query, key=key, value=value, causal=causal, dropout_p=dropout_p, scale=scale,
                           sliding_window=sliding_window, return_softmax=return_softmax, **options)


def _reference_naive_attention(query, key, value, causal: bool = False, dropout_p: float = 0.0, scale: float | None = None,
                               attn_mask=None):
    return naive_attention(query=query, key=key, value=value, causal=causal, dropout_p=dropout_p, scale=scale,
                           attn_mask=attn_mask)


flash_attention.__reference_form__ = _reference_flash_attention
naive_attention.__reference_form__ = _reference_naive_attention


@reference_kwargs({"dropout_p": (0, 0.0, None)}, Q="q", K="k", V="v")
def scaled_dot_product_attention(q, k, v, attn_mask=None, is_causal: bool = False, scale: float | None = None):
    """[B, H, S, D] layout of torch's function; an explicit mask takes torch's path, causal / full the flash kernels."""
    if attn_mask is not None:
        return F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask, is_causal=False, scale=scale)
    return flash_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal, scale).transpose(1, 2)


def _softcap_args(q, k, v, softcap, causal, softmax_scale, Q, K, V, causal_mask, config, query_scalar):
    """Common part of the two soft-capped entry points: the reference's form passes [B, H, S, D] tensors as Q / K / V,
    the mask object instead of a flag, and the soft-max scale either as `query_scalar` (scale = query_scalar^-0.5) or
    inside `config` (`query_pre_attn_scalar`, `attn_logit_softcapping`)."""
    ref_form = Q is not None
    if ref_form:
        q, k, v = Q.transpose(1, 2), K.transpose(1, 2), V.transpose(1, 2)
        causal = causal_mask is not None if causal_mask is not None or causal is None else causal
    if config is not None:
        softcap = softcap if softcap is not None else getattr(config, "attn_logit_softcapping", 0.0)
        query_scalar = query_scalar if query_scalar is not None else getattr(config, "query_pre_attn_scalar", None)
    if softmax_scale is None and query_scalar:
        softmax_scale = float(query_scalar) ** -0.5
    return q, k, v, float(softcap or 0.0), True if causal is None else bool(causal), softmax_scale, ref_form


def slow_attention_softcapping(q=None, k=None, v=None, softcap: float | None = None, causal: bool | None = None,
                               softmax_scale: float | None = None, *, Q=None, K=None, V=None, causal_mask=None,
                               config=None, bsz=None, q_len=None, query_scalar=None):
    """fp32 reference of soft-capped attention: scores -> softcap * tanh(scores / softcap).  [B, S, H, D] in and out;
    with the reference's `Q= K= V=` form [B, H, S, D] in and [B, S, H * D] out (`bsz` / `q_len` are implied)."""
    q, k, v, softcap, causal, softmax_scale, ref = _softcap_args(q, k, v, softcap, causal, softmax_scale, Q, K, V,
                                                                 causal_mask, config, query_scalar)
    o = _attn.attention_reference(q, k, v, causal, softmax_scale, None, softcap).to(q.dtype)
    return o.reshape(o.shape[0], o.shape[1], -1) if ref else o


def attention_softcapping_compiled(q=None, k=None, v=None, softcap: float | None = None, causal: bool | None = None,
                                   softmax_scale: float | None = None, *, Q=None, K=None, V=None, causal_mask=None,
                                   query_scalar=None, num_heads=None, num_kv_heads=None, head_dim=None):
    """Soft-capped attention on the flash kernel (the cap is applied to the scores inside the kernel).  Same two
    calling forms as `slow_attention_softcapping`; head counts are read from the tensors."""
    q, k, v, softcap, causal, softmax_scale, ref = _softcap_args(q, k, v, softcap, causal, softmax_scale, Q, K, V,
                                                                 causal_mask, None, query_scalar)
    o = flash_attention(q.contiguous(), k.contiguous(), v.contiguous(), causal, softmax_scale, None, softcap)
    return o.reshape(o.shape[0], o.shape[1], -1) if ref else o


@reference_kwargs(max_seq_len="seq_len")
def create_causal_mask(seq_len: int, device=None, dtype=torch.float32) -> torch.Tensor:
    if isinstance(device, torch.dtype):                      # (max_seq_len, dtype, device), the reference's order
        device, dtype = (dtype if not isinstance(dtype, torch.dtype) else None), device
    return torch.full((seq_len, seq_len), float("-inf"), device=device, dtype=dtype).triu(1)


@reference_kwargs(max_seq_len="seq_len", window_size="window")
def create_sliding_window_causal_mask(seq_len: int, window: int, device=None, dtype=torch.float32) -> torch.Tensor:
    if isinstance(device, torch.dtype):                      # (max_seq_len, window_size, dtype, device)
        device, dtype = (dtype if not isinstance(dtype, torch.dtype) else None), device
    i = torch.arange(seq_len, device=device)
    keep = (i[None, :] <= i[:, None]) & (i[:, None] - i[None, :] < window)
    return torch.zeros(seq_len, seq_len, device=device, dtype=dtype).masked_fill(~keep, float("-inf"))


def inference_attention_single_token(q=None, k_cache=None, v_cache=None, seq_lens: torch.Tensor | None = None,
                                     softmax_scale: float | None = None, *, Q=None, K=None, V=None, config=None
                                     ) -> torch.Tensor:
    """Decode step: q [B, Hq, D] against caches [B, S_max, Hkv, D] (valid prefix `seq_lens[b]`) -> [B, Hq, D].
    The reference's form: Q [B, Hq, 1, D], K / V [B, Hkv, S, D] and a config with `query_pre_attn_scalar` /
    `attn_logit_softcapping` -> [B, 1, Hq * D] (data_pipeline/trainer/kernels/flex_attention.py:1032)."""
    if Q is not None:
        qs = getattr(config, "query_pre_attn_scalar", None)
        cap = float(getattr(config, "attn_logit_softcapping", 0.0) or 0.0)
        scale = float(qs) ** -0.5 if qs and qs != 1.0 else None
        if cap:
            o = _attn.attention_reference(Q.transpose(1, 2), K.transpose(1, 2), V.transpose(1, 2), False, scale, None, cap)
            return o.reshape(Q.shape[0], 1, -1).to(Q.dtype)
        o = inference_attention_single_token(Q[:, :, 0], K.transpose(1, 2), V.transpose(1, 2), None, scale)
        return o.reshape(Q.shape[0], 1, -1)
    B, Hq, D = q.shape
    S, Hkv = k_cache.shape[1], k_cache.shape[2]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D)
    g = Hq // Hkv
    qf = q.float().view(B, Hkv, g, D)
    s = torch.einsum("bhgd,bshd->bhgs", qf, k_cache.float()) * scale
    if seq_lens is not None:
        pad = torch.arange(S, device=q.device)[None, :] >= seq_lens[:, None]
        s = s.masked_fill(pad[:, None, None, :], float("-inf"))
    o = torch.einsum("bhgs,bshd->bhgd", torch.softmax(s, -1), v_cache.float())
    return o.reshape(B, Hq, D).to(q.dtype)


# ---- the same three functions in the reference's POSITIONAL order ([B, H, S, D] tensors, mask object, config); served
# under the reference's import path (data_pipeline/trainer/kernels/flex_attention.py:731, 1032, 1397)
def _reference_slow_attention_softcapping(Q, K, V, causal_mask, config, bsz=None, q_len=None):
    return slow_attention_softcapping(Q=Q, K=K, V=V, causal_mask=causal_mask, config=config, bsz=bsz, q_len=q_len)


def _reference_attention_softcapping_compiled(Q, K, V, causal_mask, query_scalar, softcap, num_heads=None,
                                              num_kv_heads=None, head_dim=None):
    return attention_softcapping_compiled(Q=Q, K=K, V=V, causal_mask=causal_mask, query_scalar=query_scalar,
                                          softcap=softcap, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim)


def _reference_inference_attention_single_token(Q, K, V, config):
    return inference_attention_single_token(Q=Q, K=K, V=V, config=config)


slow_attention_softcapping.__reference_form__ = _reference_slow_attention_softcapping
attention_softcapping_compiled.__reference_form__ = _reference_attention_softcapping_compiled
inference_attention_single_token.__reference_form__ = _reference_inference_attention_single_token


class FlashAttention(nn.Module):
    """`FlashAttention(config)(q, k, v)`: [B, S, H, D] tensors.  The reference's `FlashAttention(head_dim, num_heads,
    num_kv_heads, causal=False, dropout, sliding_window)(query, key, value, attn_mask)` takes and returns [B, H, S, D]
    (data_pipeline/trainer/kernels/flash_attention.py:953); an explicit `attn_mask` goes through the fp32 path."""

    def __init__(self, config: "FlashAttentionConfig | int | None" = None, num_heads: int | None = None,
                 num_kv_heads: int | None = None, causal: bool | None = None, dropout: float = 0.0,
                 sliding_window: int | None = None, *, head_dim: int | None = None):
        super().__init__()
        self.heads_first = head_dim is not None or isinstance(config, int)
        if self.heads_first:
            head_dim = head_dim if head_dim is not None else config
            config = FlashAttentionConfig(causal=bool(causal), dropout=dropout, head_dim=head_dim, num_heads=num_heads,
                                          num_kv_heads=num_kv_heads or num_heads, sliding_window=sliding_window)
        self.config = config or FlashAttentionConfig()
        if self.config.dropout:
            raise ValueError("attention dropout is not supported")

    head_dim = property(lambda self: self.config.head_dim)
    num_heads = property(lambda self: self.config.num_heads)
    num_kv_heads = property(lambda self: self.config.num_kv_heads)
    causal = property(lambda self: self.config.causal)
    sliding_window = property(lambda self: self.config.window_size)

    def forward(self, q=None, k=None, v=None, cu_seqlens=None, *, query=None, key=None, value=None, attn_mask=None):
        c = self.config
        if query is not None or self.heads_first:
            query, key, value = (query if query is not None else q), (key if key is not None else k), \
                (value if value is not None else v)
            attn_mask = attn_mask if attn_mask is not None else cu_seqlens
            if attn_mask is not None:
                return naive_attention(query=query, key=key, value=value, attn_mask=attn_mask, scale=c.softmax_scale)
            return flash_attention(query=query, key=key, value=value, causal=c.causal, scale=c.softmax_scale,
                                   sliding_window=c.window_size, softcap=c.softcap)
        return flash_attention(q, k, v, c.causal, c.softmax_scale, c.window_size, c.softcap, cu_seqlens)


class FlexAttention(FlashAttention):
    """Mask-type front end: causal / full / sliding window / packed documents map onto the kernel's own switches."""

    def __init__(self, config: FlexAttentionConfig | None = None):
        config = config or FlexAttentionConfig()
        if config.mask_type is AttentionMaskType.FULL:
            config.causal = False
        if config.mask_type is AttentionMaskType.SLIDING_WINDOW and not config.window_size:
            raise ValueError("sliding-window attention needs window_size")
        super().__init__(config)

    def forward(self, q=None, k=None, v=None, cu_seqlens=None, *, Q=None, K=None, V=None, attention_mask=None,
                is_causal: bool | None = None, use_inference_mode: bool = False):
        """`attn(q, k, v)`: [B, S, H, D] in and out.  The reference's `attn(Q=, K=, V=, attention_mask=, is_causal=,
        use_inference_mode=)` takes [B, heads, S, D] and returns [B, q_len, heads * D]; scale, soft-cap and window come
        from the configuration (data_pipeline/trainer/kernels/flex_attention.py:1319)."""
        if Q is None:
            return super().forward(q, k, v, cu_seqlens)
        from . import flex as _flex
        c = self.config
        causal = c.causal if is_causal is None else bool(is_causal)
        if use_inference_mode and Q.shape[2] == 1 and attention_mask is None:
            return inference_attention_single_token(Q, K, V, c)
        if attention_mask is not None:
            return _flex.sdpa_attention_forward(Q, K, V, c, attn_mask=attention_mask, is_causal=causal)
        return _flex.flash_attention_forward(Q, K, V, c, causal=causal)


class MultiHeadFlashAttention(nn.Module):
    """Self-attention block: fused qkv projection, rotary embedding, flash attention, output projection."""

    def __init__(self, hidden_size: int | None = None, num_heads: int | None = None, num_kv_heads: int | None = None,
                 head_dim: int | None = None, causal: bool | None = None, rope_theta: float | None = 10000.0,
                 max_position: int = 8192, dtype=None, device=None, *, embed_dim: int | None = None,
                 dropout: float = 0.0, bias: bool | None = None, sliding_window: int | None = None):
        """`MultiHeadFlashAttention(hidden_size, num_heads, ...)`: causal, rotary positions, no biases.  The reference's
        keyword form (`embed_dim=, num_heads, num_kv_heads, dropout, bias=True, causal=False, sliding_window`) is a
        plain attention layer: no rotary embedding, biases on by default, `forward(query, key, value, key_cache,
        value_cache)` (data_pipeline/trainer/kernels/flash_attention.py MultiHeadFlashAttention)."""
        super().__init__()
        reference_form = embed_dim is not None
        if reference_form:
            hidden_size, rope_theta = embed_dim, None
            causal = False if causal is None else causal
            bias = True if bias is None else bias
        if dropout:
            raise ValueError("attention dropout is not supported")
        causal = True if causal is None else causal
        self.embed_dim = hidden_size
        self.h, self.kv = num_heads, num_kv_heads or num_heads
        self.d = head_dim or hidden_size // num_heads
        self.causal, self.rope_theta, self.max_position = causal, rope_theta, max_position
        self.sliding_window = sliding_window
        self.wqkv = nn.Parameter(torch.empty((self.h + 2 * self.kv) * self.d, hidden_size, dtype=dtype, device=device))
        self.wo = nn.Parameter(torch.empty(hidden_size, self.h * self.d, dtype=dtype, device=device))
        self.bqkv = nn.Parameter(torch.zeros((self.h + 2 * self.kv) * self.d, dtype=dtype, device=device)) if bias else None
        self.bo = nn.Parameter(torch.zeros(hidden_size, dtype=dtype, device=device)) if bias else None
        nn.init.normal_(self.wqkv, std=0.02)
        nn.init.normal_(self.wo, std=0.02)
        self._tables = None

    num_heads = property(lambda self: self.h)
    num_kv_heads = property(lambda self: self.kv)
    head_dim = property(lambda self: self.d)

    def _cross(self, query, key, value, key_cache, value_cache):
        """Separate query / key / value inputs and an optional [B, Hkv, N, D] cache in front of the new keys: q, k and v
        are projected with their slices of the fused weight."""
        nq, nk = self.h * self.d, self.kv * self.d
        bq, bk, bv = (None, None, None) if self.bqkv is None else self.bqkv.split((nq, nk, nk))
        wq, wk, wv = self.wqkv.split((nq, nk, nk))
        B, M, _ = query.shape
        q = _gemm.linear(query, wq, bq).view(B, M, self.h, self.d)
        k = _gemm.linear(key, wk, bk).view(B, key.shape[1], self.kv, self.d)
        v = _gemm.linear(value, wv, bv).view(B, value.shape[1], self.kv, self.d)
        if key_cache is not None and value_cache is not None:
            k = torch.cat((key_cache.transpose(1, 2), k), dim=1)
            v = torch.cat((value_cache.transpose(1, 2), v), dim=1)
        if k.shape[1] == M:
            o = flash_attention(q, k, v, self.causal, None, self.sliding_window)
        else:                                               # the queries are the LAST M positions of the keys
            N = k.shape[1]
            rep = self.h // self.kv
            kk, vv = k.repeat_interleave(rep, 2).transpose(1, 2), v.repeat_interleave(rep, 2).transpose(1, 2)
            mask = None
            if self.causal or self.sliding_window:
                qi = torch.arange(N - M, N, device=q.device)[:, None]
                ki = torch.arange(N, device=q.device)[None, :]
                mask = torch.ones(M, N, dtype=torch.bool, device=q.device)
                if self.causal:
                    mask &= ki <= qi
                if self.sliding_window:
                    mask &= ki > qi - self.sliding_window
            o = F.scaled_dot_product_attention(q.transpose(1, 2).float(), kk.float(), vv.float(), attn_mask=mask) \
                .transpose(1, 2).to(q.dtype)
        return _gemm.linear(o.reshape(B, M, nq), self.wo, self.bo)

    def forward(self, x=None, cu_seqlens=None, value=None, key_cache=None, value_cache=None, *, query=None, key=None):
        """`attn(x, cu_seqlens)`: self-attention.  `attn(query, key, value, key_cache, value_cache)` (key and value
        default to the query): attention of `query` over `key` / `value`, optionally behind a cache."""
        query = query if query is not None else x
        if key is None and torch.is_tensor(cu_seqlens) and cu_seqlens.is_floating_point():
            key, cu_seqlens = cu_seqlens, None               # positional (query, key, value)
        if key is not None or value is not None or key_cache is not None:
            key = key if key is not None else query
            return self._cross(query, key, value if value is not None else key, key_cache, value_cache)
        x = query
        B, S, _ = x.shape
        qkv = _gemm.linear(x, self.wqkv, self.bqkv)
        if self.rope_theta:
            if self._tables is None or self._tables[0].device != x.device or self._tables[0].shape[0] < S:
                self._tables = _rope.rope_tables(max(S, self.max_position), self.d, self.rope_theta, device=x.device)
            qkv = _rope.apply_rope_qkv(qkv, self.h + self.kv, self.d, *self._tables)
        o = _attn.attention_qkv(qkv, self.h, self.kv, self.d, self.causal, window=self.sliding_window,
                                cu_seqlens=cu_seqlens)
        return _gemm.linear(o, self.wo, self.bo)


# ------------------------------------------------------------------------------------------------ rotary embeddings
class RoPEScalingType(str, Enum):
    NONE = "none"
    LINEAR = "linear"
    NTK = "ntk"
    DYNAMIC_NTK = "dynamic_ntk"
    YARN = "yarn"
    LLAMA3 = "llama3"
    LONGROPE = "longrope"


@dataclass
class RoPEConfig:
    dim: int = 128
    max_position: int = 8192
    theta: float = 10000.0
    scaling_type: RoPEScalingType = RoPEScalingType.NONE
    scaling_factor: float = 1.0
    original_max_position: int = 8192
    interleaved: bool = False
    longrope_short_factor: Optional[List[float]] = None
    longrope_long_factor: Optional[List[float]] = None


@reference_kwargs({"dtype": ANY}, max_seq_len="end")
def precompute_freqs_cis(dim: int, end: int, theta: float = 10000.0, scaling_factor: float = 1.0, device=None):
    """(cos, sin) tables [end, dim/2] (linear position scaling when scaling_factor != 1)."""
    return _rope.rope_tables(end, dim, theta, device=device,
                             **({"scaling": "linear", "factor": scaling_factor} if scaling_factor != 1.0 else {}))


class RoPEFrequencyCache:
    """(cos, sin) tables per (config, device), grown on demand."""

    def __init__(self):
        self._cache: dict = {}

    def get(self, cfg: RoPEConfig, seq_len: int, device=None):
        key = (cfg.dim, cfg.theta, cfg.scaling_type, cfg.scaling_factor, cfg.original_max_position, str(device))
        cur = self._cache.get(key)
        if cur is None or cur[0].shape[0] < seq_len:
            n = max(seq_len, cfg.max_position)
            cur = _rope.rope_tables(n, cfg.dim, cfg.theta, device, scaling=cfg.scaling_type.value,
                                    factor=cfg.scaling_factor, original_max_pos=cfg.original_max_position,
                                    long_factor=cfg.longrope_long_factor, short_factor=cfg.longrope_short_factor)
            self._cache[key] = cur
        return cur

    # ---- class-level form (data_pipeline/trainer/kernels/rope_kernels.py:116-143): one shared cache, tables cut to
    # `seq_len` rows and cast to `dtype`
    _shared: "RoPEFrequencyCache | None" = None

    @classmethod
    def get_freqs(cls, config: RoPEConfig, seq_len: int, device=None, dtype: torch.dtype | None = None):
        if cls._shared is None:
            cls._shared = cls()
        cos, sin = cls._shared.get(config, seq_len, device)
        cos, sin = cos[:seq_len], sin[:seq_len]
        return (cos.to(dtype), sin.to(dtype)) if dtype is not None else (cos, sin)

    @classmethod
    def clear_cache(cls) -> None:
        if cls._shared is not None:
            cls._shared._cache.clear()


def _tables(cos, sin):
    cos, sin = cos.squeeze(), sin.squeeze()
    return cos.float().contiguous(), sin.float().contiguous()


@reference_kwargs(Q="q")
def fast_rope_embedding(q, k, cos, sin=None, positions=None, interleaved: bool = False):
    """q [B, S, Hq, D], k [B, S, Hkv, D], tables [max_pos, D/2] -> rotated (q, k).  The three-argument form
    `fast_rope_embedding(Q, cos, sin)` rotates one tensor and returns it."""
    if sin is None:                                   # (Q, cos, sin)
        c, s_ = _tables(k, cos)
        return _rope.apply_rope(q, c, s_, None, 0, interleaved)
    return _rope.apply_rope(q, cos, sin, positions, 0, interleaved), _rope.apply_rope(k, cos, sin, positions, 0, interleaved)


def apply_rope(q, k, cos, sin, interleaved: bool = False):
    """(q', k') for q [B, S, Hq, D], k [B, S, Hkv, D] and tables [max_pos, D/2]
    (data_pipeline/trainer/kernels/triton_kernels.py:984); the single-tensor op is `ops.rope.apply_rope`."""
    c, s_ = _tables(cos, sin)
    return _rope.apply_rope(q, c, s_, None, 0, interleaved), _rope.apply_rope(k, c, s_, None, 0, interleaved)


def inplace_rope_embedding(qkv=None, n_heads=None, n_kv_heads=None, head_dim=None, cos=None, sin=None, positions=None, *,
                           Q=None, K=None, position_offset: int = 0):
    """Rotates the q and k heads of a fused [B, S, (Hq + 2 Hkv) D] buffer (each k head once).  The reference's form
    `inplace_rope_embedding(Q, K, cos, sin, position_offset)` rotates two separate [B, S, H, D] tensors in place and
    returns them."""
    if Q is not None or torch.is_tensor(n_heads):
        if Q is None:                                 # positional: (Q, K, cos, sin, position_offset)
            Q, K = qkv, n_heads
            if isinstance(cos, int):
                position_offset = cos
            cos, sin = n_kv_heads, head_dim
        c, s_ = _tables(cos, sin)
        with torch.no_grad():
            Q.copy_(_rope.apply_rope(Q, c, s_, None, position_offset, False))
            K.copy_(_rope.apply_rope(K, c, s_, None, position_offset, False))
        return Q, K
    return _rope.apply_rope_qkv(qkv, n_heads + n_kv_heads, head_dim, cos, sin, positions)


class Fast_RoPE_Embedding(_FunctionPair):
    """`apply(Q [B, S, H, D], cos, sin)` -> rotated Q (data_pipeline/trainer/kernels/rope_kernels.py:1210)."""

    @staticmethod
    def apply(Q, cos, sin):
        return fast_rope_embedding(Q, cos, sin)

    @classmethod
    def forward(cls, ctx, Q, cos, sin):
        return super().forward(ctx, Q, cos, sin)

    @classmethod
    def backward(cls, ctx, dQ):
        return super().backward(ctx, dQ)


# ------------------------------------------------------------------------------------------------ fused LoRA
def torch_amp_custom_fwd(fn=None, **_kw):
    """The framework's autograd functions compute in their input dtype and need no autocast bracketing; the decorators
    exist so that code written against the reference's names imports and runs unchanged."""
    return fn if fn is not None else (lambda f: f)


torch_amp_custom_bwd = torch_amp_custom_fwd


def matmul_lora(x, W, *rest, A=None, B=None, s: float | None = None, W_quant=None, scaling: float | None = None):
    """x W^T + s (x A^T) B^T with the adapter product accumulated by the GEMM epilogue (A [r, in], B [out, r]).
    Positional tails: (A, B, s) or, in the reference's order, (W_quant, A, B, scaling) - told apart by their number;
    a quantisation state must be None here (quantised bases go through `quantization.FP8Linear` / `QuantState`)."""
    if len(rest) == 4:
        W_quant, A, B, scaling = rest
    elif rest:
        A, B, s = (list(rest) + [None, None])[:3] if len(rest) < 3 else rest
    if W_quant is not None:
        raise NotImplementedError("matmul_lora takes a dense base weight; dequantise first (quantization.fast_dequantize)")
    s = s if s is not None else (scaling if scaling is not None else 1.0)
    if A is None or B is None:
        return _gemm.linear(x, W)
    from ..lora import _LoRALinearFn
    return _LoRALinearFn.apply(x, W, ((float(s), 0, int(W.shape[0])),), A, B)


def get_lora_parameters(module):
    """(W, A, B, scaling) of a module that carries one adapter (`LoRALinear`-style attributes), else (W, None, None, 1)."""
    W = getattr(module, "weight", None)
    A, B = getattr(module, "lora_A", None), getattr(module, "lora_B", None)
    return W, A, B, float(getattr(module, "scaling", 1.0))


def _proj(x, module):
    W, A, B, s = get_lora_parameters(module)
    y = matmul_lora(x, W, A, B, s)
    b = getattr(module, "bias", None)
    return y if b is None else y + b


def apply_lora_qkv(x=None, Wq=None, Wk=None, Wv=None, Aq=None, Bq=None, Ak=None, Bk=None, Av=None, Bv=None, s: float = 1.0,
                   *, q_proj=None, k_proj=None, v_proj=None, X=None, inplace: bool = True):
    """(q, k, v) projections with their adapters.  Tensor form: (x, Wq, Wk, Wv, adapters..., s).  Module form of the
    reference: (q_proj, k_proj, v_proj, X) with modules that carry `weight`, `lora_A`, `lora_B`, `scaling`
    (data_pipeline/trainer/kernels/fast_lora_mlp.py:1293); `inplace` has no meaning here."""
    if isinstance(x, nn.Module) or q_proj is not None:
        q_proj, k_proj, v_proj, X = (x, Wq, Wk, Wv) if q_proj is None else (q_proj, k_proj, v_proj, X)
        return _proj(X, q_proj), _proj(X, k_proj), _proj(X, v_proj)
    return matmul_lora(x, Wq, Aq, Bq, s), matmul_lora(x, Wk, Ak, Bk, s), matmul_lora(x, Wv, Av, Bv, s)


def apply_lora_mlp_swiglu(x=None, Wg=None, Wu=None, Wd=None, Ag=None, Bg=None, Au=None, Bu=None, Ad=None, Bd=None,
                          s: float = 1.0, *, mlp_module=None, X=None, inplace: bool = True):
    """down(silu(gate(x)) * up(x)) with adapters on all three.  Module form of the reference: (mlp_module, X) with
    `gate_proj` / `up_proj` / `down_proj` children."""
    if isinstance(x, nn.Module) or mlp_module is not None:
        mlp_module, X = (x, Wg) if mlp_module is None else (mlp_module, X)
        h = _act.swiglu(_proj(X, mlp_module.gate_proj), _proj(X, mlp_module.up_proj))
        return _proj(h, mlp_module.down_proj)
    h = _act.swiglu(matmul_lora(x, Wg, Ag, Bg, s), matmul_lora(x, Wu, Au, Bu, s))
    return matmul_lora(h, Wd, Ad, Bd, s)


class _LoRABlock(_ExplicitBackward, nn.Module):
    def _adapter(self, name, out_f, in_f, r, dtype, device):
        A = nn.Parameter(torch.empty(r, in_f, dtype=dtype, device=device))
        B = nn.Parameter(torch.zeros(out_f, r, dtype=dtype, device=device))
        nn.init.kaiming_uniform_(A, a=math.sqrt(5))
        setattr(self, f"A_{name}", A)
        setattr(self, f"B_{name}", B)

    def _ab(self, name):
        return getattr(self, f"A_{name}"), getattr(self, f"B_{name}")


class LoRA_MLP(_LoRABlock):
    """Frozen gated MLP with trainable low-rank adapters on gate / up / down."""

    def __init__(self, hidden_size: int, intermediate_size: int, r: int = 16, alpha: float = 32.0, dtype=None,
                 device=None):
        super().__init__()
        self.scaling = alpha / r
        for n, (o, i) in {"gate": (intermediate_size, hidden_size), "up": (intermediate_size, hidden_size),
                          "down": (hidden_size, intermediate_size)}.items():
            w = nn.Parameter(torch.empty(o, i, dtype=dtype, device=device), requires_grad=False)
            nn.init.normal_(w, std=0.02)
            setattr(self, f"W_{n}", w)
            self._adapter(n, o, i, r, dtype, device)

    def forward(self, x):
        return apply_lora_mlp_swiglu(x, self.W_gate, self.W_up, self.W_down, *self._ab("gate"), *self._ab("up"),
                                     *self._ab("down"), s=self.scaling)


class LoRA_QKV(_LoRABlock):
    def __init__(self, hidden_size: int, q_out: int, kv_out: int, r: int = 16, alpha: float = 32.0, dtype=None,
                 device=None):
        super().__init__()
        self.scaling = alpha / r
        for n, o in {"q": q_out, "k": kv_out, "v": kv_out}.items():
            w = nn.Parameter(torch.empty(o, hidden_size, dtype=dtype, device=device), requires_grad=False)
            nn.init.normal_(w, std=0.02)
            setattr(self, f"W_{n}", w)
            self._adapter(n, o, hidden_size, r, dtype, device)

    def forward(self, x):
        return apply_lora_qkv(x, self.W_q, self.W_k, self.W_v, *self._ab("q"), *self._ab("k"), *self._ab("v"),
                              s=self.scaling)


def validate_lora_gradients(T: int = 64, hidden: int = 64, out: int = 96, r: int = 8, device=None, dtype=None,
                            atol: float | None = None, *, X=None, W=None, A=None, B=None, scaling: float = 1.0,
                            eps: float = 1e-4, rtol: float = 1e-3):
    """Gradients of `matmul_lora` (custom backward with accumulating GEMMs) against autograd on the plain formula.
    Without tensors: random operands of the given sizes, returns {dx, dA, dB: relative error, passed}.  With the
    reference's tensors (X, W, A, B, scaling - by position or name) the check runs on them and returns a bool."""
    if torch.is_tensor(T) or X is not None:
        X, W, A, B = (T, hidden, out, r) if X is None else (X, W, A, B)
        leaves = [t.detach().clone().requires_grad_(True) for t in (X, A, B)]
        matmul_lora(leaves[0], W, leaves[1], leaves[2], float(scaling)).float().pow(2).sum().backward()
        ref = [t.detach().float().clone().requires_grad_(True) for t in (X, A, B)]
        (ref[0] @ W.float().t() + scaling * (ref[0] @ ref[1].t()) @ ref[2].t()).pow(2).sum().backward()
        tol = atol if atol is not None else 1e-3
        return all(torch.allclose(a.grad.float(), b.grad, atol=tol, rtol=rtol) for a, b in zip(leaves, ref))
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    dtype = dtype or (torch.bfloat16 if device == "cuda" else torch.float32)
    g = torch.Generator().manual_seed(0)
    mk = lambda *s: (torch.randn(*s, generator=g) * 0.1).to(device, dtype)   # noqa: E731
    x, W, A, B = mk(T, hidden), mk(out, hidden), mk(r, hidden), mk(out, r)
    leaves = [t.clone().requires_grad_(True) for t in (x, A, B)]
    matmul_lora(leaves[0], W, leaves[1], leaves[2], 2.0).float().pow(2).sum().backward()
    ref = [t.float().clone().requires_grad_(True) for t in (x, A, B)]
    (ref[0] @ W.float().t() + 2.0 * (ref[0] @ ref[1].t()) @ ref[2].t()).pow(2).sum().backward()
    errs = {n: float((a.grad.float() - b.grad).abs().max() / b.grad.abs().max().clamp(min=1e-9))
            for n, a, b in zip(("dx", "dA", "dB"), leaves, ref)}
    tol = atol if atol is not None else (3e-2 if dtype == torch.bfloat16 else 1e-4)
    return dict(errs, passed=all(v < tol for v in errs.values()))


# ------------------------------------------------------------------------------------------------ MoE
@dataclass
class MoEKernelConfig:
    num_experts: int = 8
    top_k: int = 2
    segment_alignment: int = 128          # expert segments of the sorted layout start on tile boundaries
    activation: str = "silu"


def moe_grouped_gemm(x=None, expert_ids=None, weights=None, w_gate_up=None, w_down=None, activation: str = "silu", *,
                     X=None, W=None, topk=None, expert_offsets=None, gather_indices=None, topk_weights=None,
                     permute_x: bool = False, permute_y: bool = False, fuse_topk_weights: bool = False,
                     fwd_config=None, bwd_config=None):
    """Top-k expert FFN over tokens x [T, H]: device-side routing plan, permute into 128-aligned expert segments,
    grouped tcgen05 GEMMs, weighted combine (w_gate_up [E, 2I, H], w_down [E, H, I]).

    The reference's single grouped GEMM `moe_grouped_gemm(X, W, topk, expert_offsets, gather_indices, ...)` (one weight
    [E, N, K], rows grouped by `expert_offsets`) is `kernels.moe.moe_grouped_gemm_forward`; it is reached from here by
    those keywords, or positionally when the third argument is the integer `topk`."""
    if X is not None or isinstance(weights, int):
        from .moe import moe_grouped_gemm_forward
        if X is None:
            X, W, topk, expert_offsets = x, expert_ids, weights, w_gate_up
            gather_indices = gather_indices if gather_indices is not None else w_down
        return moe_grouped_gemm_forward(X, W, topk, expert_offsets, gather_indices, topk_weights, permute_x, permute_y,
                                        fuse_topk_weights, fwd_config)
    if _moe.available(x):
        return _moe.moe_ffn(x, expert_ids, weights, w_gate_up, w_down, activation)
    out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)       # per-expert loop (CPU / non-bf16 inputs)
    for e in range(w_gate_up.shape[0]):
        tok, slot = (expert_ids == e).nonzero(as_tuple=True)
        if tok.numel():
            h = _act.glu(x[tok].float() @ w_gate_up[e].float().t(), activation)
            out.index_add_(0, tok, (h @ w_down[e].float().t()) * weights[tok, slot].float().unsqueeze(1))
    return out.to(x.dtype)


# ------------------------------------------------------------------------------------------------ fp8
class FP8Format(str, Enum):
    E4M3 = "e4m3"
    E5M2 = "e5m2"


@dataclass
class FP8Config:
    format: FP8Format = FP8Format.E4M3
    block_size: int = 128
    amax_history_len: int = 16
    margin: int = 0
    forward_format: FP8Format = FP8Format.E4M3        # activations and weights: more mantissa
    backward_format: FP8Format = FP8Format.E5M2       # gradients: more range
    scale_update_interval: int = 1

    @property
    def forward_spec(self):
        from .compat import get_fp8_spec
        return get_fp8_spec(self.forward_format)

    @property
    def backward_spec(self):
        from .compat import get_fp8_spec
        return get_fp8_spec(self.backward_format)


def _fp8_dtype(fp8_format):
    if fp8_format is None or isinstance(fp8_format, torch.dtype):
        return fp8_format or torch.float8_e4m3fn
    return torch.float8_e5m2 if "5" in str(getattr(fp8_format, "value", fp8_format)) else torch.float8_e4m3fn


def _on_kernel(t, block=128, dtype=torch.float8_e4m3fn):
    return t.is_cuda and t.dtype == torch.bfloat16 and block == 128 and dtype == torch.float8_e4m3fn and t.dim() == 2 \
        and t.shape[1] % 128 == 0


@reference_kwargs(x="x2")
def row_quantize_fp8(x2, fp8_format=None):
    """(q, scale [rows]) with x ~ q * scale; e4m3 unless `fp8_format` says e5m2."""
    dt = _fp8_dtype(fp8_format)
    if _on_kernel(x2, 128, dt):
        return _fp8.quant_row(x2)
    from ..quantization import row_quantize_fp8 as _rq
    return _rq(x2, dt)


@reference_kwargs(y="q", scales="scale", out_dtype="dtype")
def row_dequantize_fp8(q, scale, dtype=torch.bfloat16):
    from ..quantization import row_dequantize_fp8 as _rd
    return _rd(q, scale, dtype)


@reference_kwargs(x="w")
def block_quantize_fp8(w, block_size: int = 128, fp8_format=None):
    """(q, scale [ceil(N / b), ceil(K / b)]) with w ~ q * scale per b x b block."""
    dt = _fp8_dtype(fp8_format)
    if _on_kernel(w, block_size, dt):
        return _fp8.quant_block(w)
    from ..quantization import block_quantize_fp8 as _bq
    return _bq(w, block_size, dt)


@reference_kwargs(y="q", scales="scale")
def block_dequantize_fp8(q, scale, block_size: int = 128, out_dtype=None):
    if q.is_cuda and block_size == 128 and out_dtype in (None, torch.float32):
        return _fp8.dequant(q, scale, "block")
    from ..quantization import block_dequantize_fp8 as _bd
    return _bd(q, scale, block_size, out_dtype or torch.bfloat16)


def _expand_scale(scale, shape):
    """Per-row [M], per-row-block [M, K/b] or per-block [M/b, K/b] scales broadcast to `shape` = (M, K)."""
    s = scale.float()
    if s.dim() == 1:
        return s[:, None].expand(shape)
    for d in (0, 1):
        if s.shape[d] != shape[d]:
            s = s.repeat_interleave(-(-shape[d] // s.shape[d]), dim=d).narrow(d, 0, shape[d])
    return s


def _fp8_matmul_prequantized(A, A_scale, B, B_scale, out_dtype):
    """The reference's operand form: A [M, K] and B [K, N] already in fp8 with their scales (any of the layouts that
    `_expand_scale` understands).  The product is formed on the dequantised values."""
    a = A.float() * _expand_scale(A_scale, A.shape)
    b = B.float() * _expand_scale(B_scale, B.shape)
    return (a @ b).to(out_dtype or torch.bfloat16)


def fp8_matmul_block_scaled(x2=None, w=None, *args, A=None, A_scale=None, B=None, B_scale=None, out_dtype=None,
                            block_size: int = 128):
    """x2 [M, K] bf16, w [N, K] bf16 -> x2 w^T through e4m3 operands (1x128 activation / 128x128 weight scales).
    With four tensors (A, A_scale, B [K, N], B_scale - positionally or by those names) the operands are taken as
    already quantised (data_pipeline/trainer/kernels/fp8_kernels.py:844)."""
    if args or A is not None:
        ops_ = [t for t in (x2, w) + args if t is not None] if A is None else [A, A_scale, B, B_scale]
        return _fp8_matmul_prequantized(*ops_[:4], out_dtype)
    aq, sa = _fp8.quant_act(x2)
    bq, sb = _fp8.quant_block(w)
    return _fp8.gemm_fp8(aq, sa, bq, sb, w.shape[0])


def fp8_matmul_row_scaled(x2=None, w=None, *args, A=None, A_scale=None, B=None, B_scale=None, out_dtype=None):
    """Per-row scaled operands; the product is formed on the dequantised bf16 values (tcgen05 bf16 GEMM).  Four tensors
    select the pre-quantised form as in `fp8_matmul_block_scaled` (B [K, N] with one scale per column or row)."""
    if args or A is not None:
        ops_ = [t for t in (x2, w) + args if t is not None] if A is None else [A, A_scale, B, B_scale]
        a, sa, b, sb = ops_[:4]
        # B is [K, N]: a row-wise quantised [N, K] weight, transposed, carries one scale per COLUMN here
        bfull = b.float() * (sb.float().reshape(1, -1) if sb.numel() == b.shape[1] else _expand_scale(sb, b.shape))
        return ((a.float() * _expand_scale(sa, a.shape)) @ bfull).to(out_dtype or torch.bfloat16)
    xq, xs = _fp8.quant_row(x2)
    wq, ws = _fp8.quant_row(w)
    return _gemm.matmul_nt(_fp8.dequant(xq, xs, "row").to(x2.dtype), _fp8.dequant(wq, ws, "row").to(w.dtype))


class FP8ScaleManager:
    """Delayed scaling: keeps an amax history per tensor name and turns it into the scale of the next step."""

    FMAX = {FP8Format.E4M3: 448.0, FP8Format.E5M2: 57344.0}

    def __init__(self, config: FP8Config | None = None, device=None):
        """`device`: where the per-tensor scale tensors of `get_meta` live (the tensor's own device when None)."""
        self.config = config or FP8Config()
        self.device = device
        self.history: dict[str, list[float]] = {}

    def update(self, name: str, tensor: torch.Tensor) -> float:
        h = self.history.setdefault(name, [])
        h.append(float(tensor.detach().abs().max()))
        del h[:-self.config.amax_history_len]
        return self.scale(name)

    def scale(self, name: str) -> float:
        h = self.history.get(name)
        amax = max(h) if h else 1.0
        return (self.FMAX[self.config.format] / (2 ** self.config.margin)) / max(amax, 1e-12)

    # ---- tensor-valued state per name (data_pipeline/trainer/kernels/fp8_kernels.py:170-196): the scale stays on the
    # tensor's device, so nothing is read back to the host in the training loop
    def get_meta(self, name: str, fp8_format: FP8Format = FP8Format.E4M3, device=None):
        from .compat import FP8TensorMeta, get_fp8_spec
        metas = self.__dict__.setdefault("_metas", {})
        if name not in metas:
            metas[name] = FP8TensorMeta(get_fp8_spec(fp8_format), device, self.config.amax_history_len)
        return metas[name]

    def update_and_get_scale(self, tensor: torch.Tensor, name: str, fp8_format: FP8Format = FP8Format.E4M3):
        """Record the tensor's amax and return (scale, 1 / scale) with scale = amax_history.max() / fmax * 2^margin, so
        that tensor / scale fills the format's range; the scale is refreshed every `scale_update_interval` steps."""
        meta = self.get_meta(name, fp8_format, tensor.device)
        meta.update_amax(tensor.detach().abs().max())
        if self.__dict__.get("_steps", 0) % max(1, self.config.scale_update_interval) == 0:
            meta.compute_scale(self.config.margin)
        return meta.scale, meta.scale_inv

    def step(self) -> None:
        self.__dict__["_steps"] = self.__dict__.get("_steps", 0) + 1


class FP8Linear(nn.Module):
    """Linear layer whose forward and input-gradient products run on the block-scaled fp8 kernel (bf16 CUDA inputs
    with in_features a multiple of 128); weight gradient and parameters stay bf16."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, dtype=torch.bfloat16, device=None, *,
                 block_size: int = 128):
        super().__init__()
        if isinstance(dtype, int) and not isinstance(dtype, torch.dtype):     # (in, out, bias, block_size, device, dtype)
            block_size, dtype = dtype, torch.bfloat16
        if block_size != 128:
            raise ValueError("the block-scaled fp8 GEMM uses 128 x 128 weight blocks")
        self.block_size = block_size
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None
        nn.init.normal_(self.weight, std=0.02)

    @reference_kwargs(X="x")
    def forward(self, x):
        y = _fp8.fp8_linear(x, self.weight) if _fp8.available(x) and self.weight.shape[0] % 8 == 0 \
            else _gemm.linear(x, self.weight)
        return y if self.bias is None else y + self.bias

    @property
    def in_features(self) -> int:
        return self.weight.shape[1]

    @property
    def out_features(self) -> int:
        return self.weight.shape[0]

    @classmethod
    def from_linear(cls, linear: nn.Linear, block_size: int = 128) -> "FP8Linear":
        """The same weights (and bias) in a layer whose products run in fp8.  The parameters stay in the source dtype
        and trainable: quantisation happens per call, on the current values."""
        if block_size != 128:
            raise ValueError("the block-scaled fp8 GEMM uses 128 x 128 weight blocks")
        m = cls(linear.in_features, linear.out_features, linear.bias is not None, linear.weight.dtype, linear.weight.device)
        m.quantize_weight(linear.weight.data)
        if linear.bias is not None:
            m.bias.data.copy_(linear.bias.data)
        return m

    def quantize_weight(self, weight: torch.Tensor):
        """Load `weight` and return its block-scaled image (e4m3 values, one fp32 scale per 128 x 128 block) - what the
        GEMM will see; useful to inspect the quantisation error."""
        if tuple(weight.shape) != tuple(self.weight.shape):
            raise ValueError(f"weight shape {tuple(weight.shape)} != {tuple(self.weight.shape)}")
        with torch.no_grad():
            self.weight.copy_(weight)
        from ..quantization import block_quantize_fp8 as _bq
        return _bq(self.weight.detach(), 128)

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, bias={self.bias is not None}"


# ------------------------------------------------------------------------------------------------ flex-style front end
from .flex import (BlockMask, CausalSlidingWindowMasker, SlidingWindowMasker, apply_softcap_inplace,  # noqa: E402,F401
                   apply_softcap_stable, attention_sliding_window_compiled, causal_masker, create_block_mask,
                   create_flex_attention_causal_mask, create_flex_attention_sliding_window_mask, expand_kv_for_gqa,
                   expand_kv_for_gqa_contiguous, flash_attention_forward, flex_attention_forward,
                   generate_combined_modifier, generate_scale_modifier, generate_tanh_softcap, get_causal_mask_slice,
                   get_flex_attention, get_sliding_window_masker, inference_attention_softcapping,
                   sdpa_attention_forward, slow_inference_attention_softcapping)

from .moe import (ExpertMLPLayer, MoEAutotuneConfig, MoEGroupedGEMMFunction, MoERouter, RouterConfig,  # noqa: E402,F401
                  SparseMoEBlock, benchmark_moe_kernel, create_moe_block, get_l2_cache_size, get_max_shared_memory,
                  get_num_sms, moe_forward, moe_grouped_gemm_backward_dw, moe_grouped_gemm_backward_dx,
                  moe_grouped_gemm_forward)

from .compat import (CUDAGraphConfig, CompiledFunctionWrapper, DynamicShapeConfig, FP8LinearFunction,  # noqa: E402,F401
                     FP8Spec, FP8TensorMeta, Fast_RoPE, FlashAttentionTritonFunction, FusedAddRMSLayerNormFunction,
                     FusedLoRAMLP, FusedLoRAQKV, FusedRMSNorm, FusedRoPEQKFunction, InductorConfig, LayerNorm,
                     LayerNormFunction, RMSLayerNormFunction, RoPEFunction, RotaryEmbedding, apply_lora_o, apply_rope_qk,
                     benchmark_attention, benchmark_rope, calculate_multi_row_settings, calculate_settings,
                     clear_compilation_cache, compilation_context, compile_function, compiled, compute_rope_frequencies,
                     convert_model_to_fp8, dequantize_weight, fp8_linear_forward, fused_add_layernorm,
                     get_attention_backend, get_compiler, get_cuda_capability, get_device_capability,
                     get_flash_attn_version, get_fp8_capability, get_fp8_spec, get_layernorm_info,
                     get_optimal_block_size, is_flash_attn_triton_available, rms_layernorm, supports_bf16,
                     swiglu_backward, swiglu_backward_triton, triton_flash_attention)


# ---- module-level flags and constants of the reference's kernel files.  Availability flags describe THIS framework:
# there is no Triton path, "flash attention" is the tcgen05 kernel of csrc/flash_attn.cu, not the flash-attn package.
from typing import Any as _Any, Callable as _Callable, TypeVar as _TypeVar, Union as _Union  # noqa: E402

FLASH_ATTN_VERSION = None                  # not the flash-attn package
TRITON_AVAILABLE = False
TORCH_COMPILE_OPTIONS: dict = {}           # nothing here is traced; kept for scripts that read it
HAS_FLEX_ATTENTION = True                  # block-mask attention (`kernels.flex`) is always present


def __getattr__(name: str):
    """`BACKEND_CAPS` and `FLASH_ATTN_AVAILABLE` probe the device, so they are computed on first use and not while
    the package is imported (an import must not create a CUDA context)."""
    if name == "BACKEND_CAPS":
        value = BackendCapabilities.detect()
    elif name == "FLASH_ATTN_AVAILABLE":
        value = supports_tcgen05()
    else:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    globals()[name] = value
    return value


FP8_E4M3_SPEC, FP8_E5M2_SPEC = get_fp8_spec(FP8Format.E4M3), get_fp8_spec(FP8Format.E5M2)
FP8_CONFIG = FP8Config()
LN_CONFIG = LayerNormConfig()
fast_layernorm = layernorm
ROPE_GROUP_SIZE, BLOCK_SIZE_DEFAULT, WARP_SIZE, MIN_BLOCK_SIZE = 4, 1024, 32, 128
ModelType = _TypeVar("ModelType", bound=nn.Module)
CompiledModel = _Union[nn.Module, _Callable[..., _Any]]
