"""Mask / score-modifier front end of the attention kernels, in the [B, heads, S, D] layout and with the function names
of data_pipeline/trainer/kernels/flex_attention.py (:271-360 score modifiers, :357-413 maskers, :421-474 block masks,
:482-590 factories and GQA expansion, :599-650 soft-capping, :707-1040 and :1444-1500 forward variants).

The reference builds these on torch's flex_attention + torch.compile and falls back to SDPA or an eager loop.  Here
causal, sliding-window and soft-capped attention are switches of the framework's own tcgen05 flash kernels
(csrc/attention.cu), so a "block mask" is a small descriptor that says WHICH of those switches a mask function means;
only a mask that is neither causal nor a causal window is materialised and sent through the fp32 reference math.

Softmax scale: `query_pre_attn_scalar` follows Gemma-2 - when it is set (not None / 0 / 1) the scale is
1 / sqrt(query_pre_attn_scalar), otherwise 1 / sqrt(head_dim).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Callable

import torch
import torch.nn.functional as F

_SOFTCAP_EPS = 1e-6


# ------------------------------------------------------------------------------------------------ score modifiers
def generate_tanh_softcap(t: float) -> Callable:
    """score -> t * tanh(score / t) (Gemma-2 logit soft-capping) as a flex-style modifier (score, b, h, q_idx, kv_idx)."""
    inv = 1.0 / (t + _SOFTCAP_EPS)

    def tanh_softcap(score, b=None, h=None, q_idx=None, kv_idx=None):
        return t * torch.tanh(score * inv)
    tanh_softcap.softcap = t
    return tanh_softcap


def generate_scale_modifier(scale: float) -> Callable:
    def scale_mod(score, b=None, h=None, q_idx=None, kv_idx=None):
        return score * scale
    scale_mod.scale = scale
    return scale_mod


def generate_combined_modifier(scale: float, softcap: float) -> Callable:
    """Scale then soft-cap in one modifier."""
    inv = 1.0 / (softcap + _SOFTCAP_EPS)

    def combined(score, b=None, h=None, q_idx=None, kv_idx=None):
        return softcap * torch.tanh(score * scale * inv)
    combined.scale, combined.softcap = scale, softcap
    return combined


def apply_softcap_stable(scores: torch.Tensor, softcap: float) -> torch.Tensor:
    return softcap * torch.tanh(scores / softcap)


def apply_softcap_inplace(scores: torch.Tensor, softcap: float) -> torch.Tensor:
    return scores.mul_(1.0 / softcap).tanh_().mul_(softcap)


# ------------------------------------------------------------------------------------------------ mask functions
def causal_masker(b, h, q_idx, kv_idx):
    return q_idx >= kv_idx


class SlidingWindowMasker:
    """Causal window: a query sees itself and the `window_size - 1` keys before it.  Works on ints and on index tensors."""
    __slots__ = ("window_size",)

    def __init__(self, window_size: int):
        self.window_size = int(window_size)

    def __call__(self, b, h, q_idx, kv_idx):
        causal, near = q_idx >= kv_idx, (q_idx - kv_idx) < self.window_size
        return (causal & near) if isinstance(causal, torch.Tensor) else (causal and near)


class CausalSlidingWindowMasker:
    """Causal window whose width may differ per head ({head: window}, `default_window` for the others)."""
    __slots__ = ("window_sizes", "default_window")

    def __init__(self, window_sizes: dict | None = None, default_window: int = 4096):
        self.window_sizes, self.default_window = dict(window_sizes or {}), int(default_window)

    def window(self, h) -> int:
        return self.window_sizes.get(int(h), self.default_window)

    def __call__(self, b, h, q_idx, kv_idx):
        causal, near = q_idx >= kv_idx, (q_idx - kv_idx) < self.window(h)
        return (causal & near) if isinstance(causal, torch.Tensor) else (causal and near)


def get_sliding_window_masker(size: int) -> SlidingWindowMasker:
    return SlidingWindowMasker(size)


# ------------------------------------------------------------------------------------------------ block masks
@dataclass
class BlockMask:
    """What a mask function means to the kernels: `kind` is "causal", "sliding_window" (with `window`) or "dense"
    (anything else: `dense` holds the boolean [S, S] mask, True = attend).  `block_size` is kept for API parity; the
    kernels tile by their own sizes."""
    kind: str
    seq_len: int
    window: int | None = None
    dense: torch.Tensor | None = None
    block_size: int = 128

    def to_bool(self, device=None) -> torch.Tensor:
        i = torch.arange(self.seq_len, device=device)
        q, k = i[:, None], i[None, :]
        if self.kind == "causal":
            return q >= k
        if self.kind == "sliding_window":
            return (q >= k) & (q - k < self.window)
        return self.dense.to(device) if device is not None else self.dense


def _evaluate(mask_fn, seq_len: int, head: int = 0) -> torch.Tensor:
    i = torch.arange(seq_len)
    try:
        m = mask_fn(0, head, i[:, None], i[None, :])
        if isinstance(m, torch.Tensor) and m.shape == (seq_len, seq_len):
            return m.bool()
    except (RuntimeError, TypeError, ValueError):
        pass                                      # a function written for ints (`and`, `if`): evaluate it per pair
    return torch.tensor([[bool(mask_fn(0, head, q, k)) for k in range(seq_len)] for q in range(seq_len)])


def create_block_mask(mask_fn: Callable, seq_len: int, block_size: int = 128, batch_size: int = 1,
                      num_heads: int = 1) -> BlockMask:
    """Classify a flex-style mask function (b, h, q_idx, kv_idx) -> bool.  The known maskers are recognised by type;
    any other function is evaluated once over [seq_len, seq_len] and recognised by value when it happens to be causal."""
    if mask_fn is causal_masker:
        return BlockMask("causal", seq_len, block_size=block_size)
    if isinstance(mask_fn, SlidingWindowMasker):
        return BlockMask("sliding_window", seq_len, window=mask_fn.window_size, block_size=block_size)
    if isinstance(mask_fn, CausalSlidingWindowMasker) and len({mask_fn.window(h) for h in range(num_heads)}) == 1:
        return BlockMask("sliding_window", seq_len, window=mask_fn.window(0), block_size=block_size)
    if isinstance(mask_fn, CausalSlidingWindowMasker):
        dense = torch.stack([_evaluate(mask_fn, seq_len, h) for h in range(num_heads)])
        return BlockMask("dense", seq_len, dense=dense, block_size=block_size)
    dense = _evaluate(mask_fn, seq_len)
    if torch.equal(dense, torch.ones(seq_len, seq_len).tril().bool()):
        return BlockMask("causal", seq_len, block_size=block_size)
    return BlockMask("dense", seq_len, dense=dense, block_size=block_size)


def create_flex_attention_causal_mask(max_seq_length: int = 8192, block_size: int = 128) -> BlockMask:
    return create_block_mask(causal_masker, max_seq_length, block_size)


def create_flex_attention_sliding_window_mask(max_seq_length: int = 8192, sliding_window: int = 4096,
                                              block_size: int = 128) -> BlockMask:
    return create_block_mask(get_sliding_window_masker(sliding_window), max_seq_length, block_size)


def get_causal_mask_slice(causal_mask: torch.Tensor, q_len: int, kv_len: int) -> torch.Tensor:
    return causal_mask[:q_len, :kv_len]


# ------------------------------------------------------------------------------------------------ GQA
def expand_kv_for_gqa(K: torch.Tensor, V: torch.Tensor, num_kv_groups: int):
    """[B, Hkv, S, D] -> [B, Hkv * groups, S, D]; head h of the result is KV head h // groups."""
    if num_kv_groups == 1:
        return K, V
    B, Hkv, S, D = K.shape

    def ex(t):
        return t[:, :, None].expand(B, Hkv, num_kv_groups, S, D).reshape(B, Hkv * num_kv_groups, S, D)
    return ex(K), ex(V)


def expand_kv_for_gqa_contiguous(K, V, num_kv_groups: int):
    K, V = expand_kv_for_gqa(K, V, num_kv_groups)
    return K.contiguous(), V.contiguous()


# ------------------------------------------------------------------------------------------------ forward variants
def _softmax_scale(query_pre_attn_scalar, head_dim: int) -> float:
    qs = query_pre_attn_scalar
    return 1.0 / math.sqrt(qs) if qs not in (None, 0, 0.0, 1, 1.0) else 1.0 / math.sqrt(head_dim)


def _cfg(config, name, default=None):
    return getattr(config, name, default) if config is not None else default


def _merge_heads(o: torch.Tensor) -> torch.Tensor:          # [B, H, S, D] -> [B, S, H * D]
    B, H, S, D = o.shape
    return o.transpose(1, 2).reshape(B, S, H * D)


def _kernel_attention(Q, K, V, causal: bool, scale: float, window: int | None, softcap: float) -> torch.Tensor:
    from . import flash_attention
    o = flash_attention(Q.transpose(1, 2), K.transpose(1, 2), V.transpose(1, 2), causal, scale, window, softcap)
    return o.transpose(1, 2)


def _masked_attention(Q, K, V, mask_add: torch.Tensor | None, scale: float, softcap: float) -> torch.Tensor:
    """fp32 math with an additive mask [.., q_len, kv_len]; GQA by expansion.  The decode / odd-mask path."""
    K, V = expand_kv_for_gqa(K, V, Q.shape[1] // K.shape[1])
    s = torch.matmul(Q.float() * scale, K.float().transpose(-2, -1))
    if softcap and softcap > 0:
        s = apply_softcap_inplace(s, softcap)
    if mask_add is not None:
        s = s + mask_add.to(s.dtype)
    return torch.matmul(torch.softmax(s, dim=-1), V.float()).to(Q.dtype)


def get_flex_attention(query_scalar: float, softcap: float, enable_gqa: bool = True) -> Callable:
    """attention(query, key, value, block_mask=None) -> [B, H, S, D] with the scale and soft-cap baked in."""
    def attn(query, key, value, block_mask: BlockMask | None = None):
        scale = _softmax_scale(query_scalar, query.shape[-1])
        if not enable_gqa and key.shape[1] != query.shape[1]:
            raise ValueError("key / value heads differ from query heads and enable_gqa is off")
        if block_mask is None:                    # no mask: every query sees every key
            if query.shape[2] == key.shape[2]:
                return _kernel_attention(query, key, value, False, scale, None, softcap)
            return _masked_attention(query, key, value, None, scale, softcap)
        if block_mask.kind in ("causal", "sliding_window") and query.shape[2] == key.shape[2]:
            return _kernel_attention(query, key, value, True, scale, block_mask.window, softcap)
        S = key.shape[2]
        allow = block_mask.to_bool(query.device)[..., S - query.shape[2]:S, :S]
        add = torch.zeros(allow.shape, device=query.device).masked_fill(~allow, float("-inf"))
        return _masked_attention(query, key, value, add, scale, softcap)
    return attn


def flex_attention_forward(Q, K, V, block_mask: BlockMask | None, config: Any) -> torch.Tensor:
    """[B, H, S, D] inputs -> [B, S, H * D]; scale and soft-cap from the config, pattern from the block mask."""
    fn = get_flex_attention(_cfg(config, "query_pre_attn_scalar"), _cfg(config, "attn_logit_softcapping", 0.0) or 0.0)
    return _merge_heads(fn(Q, K, V, block_mask))


def flash_attention_forward(Q, K, V, config: Any, causal: bool = True) -> torch.Tensor:
    """Flash-kernel forward -> [B, S, H * D].  Unlike the flash-attn package the kernel soft-caps natively, so a config
    with `attn_logit_softcapping` is served here as well."""
    scale = _softmax_scale(_cfg(config, "query_pre_attn_scalar"), Q.shape[-1])
    o = _kernel_attention(Q, K, V, causal, scale, _cfg(config, "sliding_window_size"),
                          _cfg(config, "attn_logit_softcapping", 0.0) or 0.0)
    return _merge_heads(o)


def sdpa_attention_forward(Q, K, V, config: Any, attn_mask: torch.Tensor | None = None,
                           is_causal: bool = True) -> torch.Tensor:
    """An explicit mask goes through torch's SDPA (GQA by expansion); causal / full through the flash kernels."""
    scale = _softmax_scale(_cfg(config, "query_pre_attn_scalar"), Q.shape[-1])
    if attn_mask is None and Q.shape[2] == K.shape[2]:
        return _merge_heads(_kernel_attention(Q, K, V, is_causal, scale, None, 0.0))
    K, V = expand_kv_for_gqa(K, V, Q.shape[1] // K.shape[1])
    o = F.scaled_dot_product_attention(Q, K, V, attn_mask=attn_mask, is_causal=is_causal and attn_mask is None,
                                       scale=scale)
    return _merge_heads(o)


def attention_sliding_window_compiled(Q, K, V, causal_mask: torch.Tensor, query_scalar: float, softcap: float,
                                      num_heads: int, num_kv_heads: int, head_dim: int) -> torch.Tensor:
    """Soft-capped attention under an additive (sliding-window) causal mask -> [B, q_len, num_heads * head_dim]."""
    q_len, kv_len = Q.shape[2], K.shape[2]
    return _merge_heads(_masked_attention(Q, K, V, causal_mask[:q_len, :kv_len], _softmax_scale(query_scalar, head_dim),
                                          softcap))


def inference_attention_softcapping(Q, K, V, causal_mask: torch.Tensor, config: Any) -> torch.Tensor:
    """Eager soft-capped attention for generation steps (q_len small) -> [B, q_len, H * D]."""
    q_len, kv_len = Q.shape[2], K.shape[2]
    scale = _softmax_scale(_cfg(config, "query_pre_attn_scalar"), Q.shape[-1])
    return _merge_heads(_masked_attention(Q, K, V, causal_mask[:q_len, :kv_len], scale,
                                          _cfg(config, "attn_logit_softcapping", 0.0) or 0.0))


def slow_inference_attention_softcapping(Q, K, V, causal_mask: torch.Tensor, config: Any, bsz: int,
                                         q_len: int) -> torch.Tensor:
    """Same as `inference_attention_softcapping` for a HuggingFace-style model config (the batch size and query length
    are passed explicitly by that call site)."""
    return inference_attention_softcapping(Q, K, V, causal_mask, config).reshape(bsz, q_len, -1)
