"""Attention front-end: causal / sliding-window / soft-capped / packed-document attention with GQA.

`attention_qkv` consumes the fused qkv projection output directly (no q/k/v split copies).  On CUDA bf16
inputs it runs the tcgen05 flash-attention kernels of csrc/attention.cu; everywhere else (CPU, fp32,
unsupported head sizes) it runs `attention_reference`, the fp32 PyTorch oracle the tests compare against.

Reference behaviour: data_pipeline/trainer/kernels/flash_attention.py:147-300 (online softmax, GQA by
h // groups, causal, sliding window, LSE output), :895 (naive oracle),
data_pipeline/trainer/kernels/flex_attention.py:271-408,1094 (soft-cap, window masks).
"""
from __future__ import annotations

import math

import torch


def attention_reference(q, k, v, causal=True, scale=None, window=None, softcap=0.0, doc_ids=None):
    """q [B,S,Hq,D], k/v [B,Sk,Hkv,D] -> [B,S,Hq,D]; fp32 math. doc_ids [B,S] restricts attention to the
    same document (packed sequences)."""
    B, S, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    g = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if softcap and softcap > 0:
        s = softcap * torch.tanh(s / softcap)
    qi = torch.arange(S, device=q.device).unsqueeze(1) + (Sk - S)
    ki = torch.arange(Sk, device=q.device).unsqueeze(0)
    mask = torch.ones(S, Sk, dtype=torch.bool, device=q.device)
    if causal:
        mask &= ki <= qi
    if window is not None and window > 0:
        mask &= ki > qi - window
    mask = mask.view(1, 1, S, Sk)
    if doc_ids is not None:
        same = doc_ids.unsqueeze(2) == doc_ids.unsqueeze(1)
        mask = mask & same.unsqueeze(1)
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p)
    o = torch.matmul(p, vf)
    return o.permute(0, 2, 1, 3).to(q.dtype)


def _split_qkv(qkv, n_heads, n_kv_heads, head_dim):
    B, S, _ = qkv.shape
    q, k, v = qkv.split((n_heads * head_dim, n_kv_heads * head_dim, n_kv_heads * head_dim), dim=-1)
    return (q.view(B, S, n_heads, head_dim), k.view(B, S, n_kv_heads, head_dim), v.view(B, S, n_kv_heads, head_dim))


def attention_qkv(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, causal: bool = True,
                  scale: float | None = None, window: int | None = None, softcap: float = 0.0,
                  cu_seqlens: torch.Tensor | None = None, doc_ids: torch.Tensor | None = None) -> torch.Tensor:
    """qkv [B, S, (Hq + 2 Hkv) * D] (RoPE already applied) -> [B, S, Hq * D].

    `cu_seqlens` (int32 [n_docs + 1], cumulative over the flattened B*S token axis) gives packed-document
    (block-diagonal causal) attention.
    """
    B, S, _ = qkv.shape
    if qkv.is_cuda and qkv.dtype == torch.bfloat16:
        from . import flash
        if flash.supported(head_dim, window, softcap):
            return flash.flash_attention_qkv(qkv, n_heads, n_kv_heads, head_dim, causal, scale, cu_seqlens,
                                             None, window, softcap)
    q, k, v = _split_qkv(qkv, n_heads, n_kv_heads, head_dim)
    if doc_ids is None and cu_seqlens is not None:
        idx = torch.arange(B * S, device=qkv.device)
        doc_ids = (torch.bucketize(idx, cu_seqlens[1:].to(idx.dtype), right=True)).view(B, S)
    o = attention_reference(q, k, v, causal, scale, window, softcap, doc_ids)
    return o.reshape(B, S, n_heads * head_dim)
