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
from typing import NamedTuple

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
from ..losses import Fast_CrossEntropyLoss, FusedCrossEntropyFunction  # noqa: F401
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


def get_accelerator_arch(device: int = 0) -> AcceleratorArch:
    if not torch.cuda.is_available():
        return AcceleratorArch.CPU
    major = torch.cuda.get_device_capability(device)[0]
    return {10: AcceleratorArch.BLACKWELL, 9: AcceleratorArch.HOPPER, 8: AcceleratorArch.AMPERE}.get(
        major, AcceleratorArch.OTHER)


def supports_tma(device: int = 0) -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_capability(device)[0] >= 9


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


def fast_rms_layernorm(x, weight, eps: float = 1e-6, gemma: bool = False):
    return _norm.rmsnorm(x, weight, eps, None, 1.0 if gemma else 0.0)[0]


def fused_add_rms_layernorm(x, residual, weight, eps: float = 1e-6):
    """(norm(x + residual), x + residual): the sum is formed inside the norm kernel."""
    return _norm.rmsnorm(x, weight, eps, residual)


def fused_softmax(x, dim: int = -1):
    return _act.softmax(x, dim)


def fused_gelu(x, approximate: str = "tanh"):
    return _act.gelu(x, approximate)


def swiglu_forward(gate, up):
    return _act.swiglu(gate, up)


def geglu_forward(gate, up, approximate: str = "tanh"):
    return _act.glu(torch.cat((gate, up), dim=-1), "gelu_tanh" if approximate == "tanh" else "gelu")


def fast_cross_entropy_loss(logits, labels, ignore_index: int = -100, label_smoothing: float = 0.0,
                            reduction: str = "mean"):
    """logits [..., V], labels [...] -> scalar (mean over non-ignored tokens) or per-token losses (reduction="none")."""
    z, y = logits.reshape(-1, logits.shape[-1]), labels.reshape(-1)
    if z.is_cuda and z.dtype == torch.bfloat16:
        rows = _ce.cross_entropy_rows(z, y, ignore_index, label_smoothing)
    else:
        rows = F.cross_entropy(z.float(), y, ignore_index=ignore_index, label_smoothing=label_smoothing, reduction="none")
    if reduction == "none":
        return rows.view(labels.shape)
    s = rows.sum()
    return s / (y != ignore_index).sum().clamp(min=1) if reduction == "mean" else s


Fast_RMS_LayerNorm = _norm._RMSNormFn
Fast_SwiGLU = _act._GluFn
Fast_GeGLU = _act._GluFn


class TritonRMSNorm(nn.Module):
    """RMSNorm module on the fused row kernel (name kept from the reference; nothing here is Triton)."""

    def __init__(self, hidden_size: int, eps: float = 1e-6, dtype=None, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype, device=device))
        self.eps = eps

    def forward(self, x, residual=None):
        y, res = _norm.rmsnorm(x, self.weight, self.eps, residual)
        return y if residual is None else (y, res)


class TritonSwiGLU(nn.Module):
    """Gated MLP: down(silu(gate(x)) * up(x)) with gate|up as one GEMM and the fused gate kernel."""

    activation = "silu"

    def __init__(self, hidden_size: int, intermediate_size: int, dtype=None, device=None):
        super().__init__()
        self.w_gate_up = nn.Parameter(torch.empty(2 * intermediate_size, hidden_size, dtype=dtype, device=device))
        self.w_down = nn.Parameter(torch.empty(hidden_size, intermediate_size, dtype=dtype, device=device))
        nn.init.normal_(self.w_gate_up, std=0.02)
        nn.init.normal_(self.w_down, std=0.02)

    def forward(self, x):
        return _gemm.linear(_act.glu(_gemm.linear(x, self.w_gate_up), self.activation), self.w_down)


class TritonGeGLU(TritonSwiGLU):
    activation = "gelu_tanh"


RMSNorm, SwiGLU, GeGLU = TritonRMSNorm, TritonSwiGLU, TritonGeGLU
