"""CUDA flash attention binding (csrc/attention.cu) with autograd."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def supported(head_dim: int, window, softcap) -> bool:
    return head_dim in (64, 128) and not window and not softcap


def flash_attention_qkv(qkv, n_heads, n_kv_heads, head_dim, causal=True, scale=None, cu_seqlens=None):
    # interim library path until the tcgen05 kernels land
    B, S, _ = qkv.shape
    q, k, v = qkv.split((n_heads * head_dim, n_kv_heads * head_dim, n_kv_heads * head_dim), dim=-1)
    q = q.view(B, S, n_heads, head_dim).transpose(1, 2)
    k = k.view(B, S, n_kv_heads, head_dim).transpose(1, 2)
    v = v.view(B, S, n_kv_heads, head_dim).transpose(1, 2)
    if cu_seqlens is not None:
        raise NotImplementedError
    o = F.scaled_dot_product_attention(q, k, v, is_causal=causal, scale=scale, enable_gqa=n_heads != n_kv_heads)
    return o.transpose(1, 2).reshape(B, S, n_heads * head_dim)
