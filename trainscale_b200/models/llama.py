"""Llama-style decoder owned by the framework (GQA, RoPE, SwiGLU, RMSNorm, tied or untied head).

The reference has no model code: it loads a HuggingFace `AutoModelForCausalLM` and monkey-patches layers
(data_pipeline/trainer/trainers/sota_trainer.py:1161-1212, data_pipeline/trainer/registry/__init__.py:1033-1324).
Here the decoder is built for the sm_100a kernels from the start:
  * q/k/v are ONE projection ([Hq+2Hkv]*D rows) and gate/up are ONE projection, so each block is four GEMMs;
  * RoPE rotates the q|k heads of the fused buffer in place, attention reads that buffer directly;
  * the residual add is fused into the following RMSNorm;
  * the loss head is the chunked fused lm_head + cross-entropy (logits are never materialised).
State dicts convert to and from the HuggingFace Llama naming (`to_hf_state_dict` / `load_hf_state_dict`).
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass, field
from typing import Any

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from ..ops import activation, attention, cross_entropy, fused_blocks, gemm, norm, rope
from ..utils import recompute as _recompute_switch


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    hidden_size: int = 256
    intermediate_size: int = 688
    num_hidden_layers: int = 4
    num_attention_heads: int = 4
    num_key_value_heads: int | None = None
    head_dim: int | None = None
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: dict | None = None
    rope_interleaved: bool = False
    max_position_embeddings: int = 8192
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    sliding_window: int | None = None
    attn_logit_softcap: float = 0.0
    final_logit_softcap: float = 0.0
    initializer_range: float = 0.02
    model_type: str = "llama"
    attention_bias: bool = False            # q / k / v projection biases (Qwen2 family)
    num_local_experts: int = 0              # > 0: every MLP is a top-k mixture of experts (Mixtral / Qwen-MoE family)
    num_experts_per_tok: int = 2
    norm_topk_prob: bool = True
    router_aux_loss_coef: float = 0.0       # load-balancing loss weight (0 = off)
    norm_weight_offset: float = 0.0         # Gemma stores (norm weight - 1): y = x_hat * (offset + w)
    scale_embeddings: bool = False          # Gemma multiplies the token embeddings by sqrt(hidden_size)

    def __post_init__(self):
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads

    def to_dict(self) -> dict:
        return asdict(self)

    def tensor_parallel_local(self, tp: int) -> "LlamaConfig":
        """The shapes ONE tensor-parallel rank holds: heads and FFN columns divided by `tp`, everything else equal.
        A decoder built from it has exactly the parameters `shard_llama_state_for_tp` would leave on a rank."""
        if self.num_attention_heads % tp or self.num_key_value_heads % tp or self.intermediate_size % tp:
            raise ValueError(f"heads ({self.num_attention_heads}/{self.num_key_value_heads}) and FFN width "
                             f"({self.intermediate_size}) must divide by the tensor-parallel size {tp}")
        d = self.to_dict()
        d.update(num_attention_heads=self.num_attention_heads // tp, num_key_value_heads=self.num_key_value_heads // tp,
                 intermediate_size=self.intermediate_size // tp, head_dim=self.head_dim)
        return LlamaConfig(**d)

    @classmethod
    def from_dict(cls, d: dict) -> "LlamaConfig":
        keys = {f for f in cls.__dataclass_fields__}
        return cls(**{k: v for k, v in d.items() if k in keys})

    def num_parameters(self, include_embeddings: bool = True) -> int:
        H, I, L, V = self.hidden_size, self.intermediate_size, self.num_hidden_layers, self.vocab_size
        D, Hq, Hkv = self.head_dim, self.num_attention_heads, self.num_key_value_heads
        E = self.num_local_experts
        mlp = 3 * H * I if E == 0 else E * (3 * H * I + H)
        per_layer = (Hq + 2 * Hkv) * D * H + Hq * D * H + mlp + 2 * H
        if self.attention_bias:
            per_layer += (Hq + 2 * Hkv) * D
        n = L * per_layer + H
        if include_embeddings:
            n += V * H * (1 if self.tie_word_embeddings else 2)
        return n

    def flops_per_token(self, seq_len: int, causal: bool = True) -> float:
        """Training FLOPs per token: 6 * matmul params + attention (12 * L * d_attn * S, halved if causal)."""
        H, I, L, V = self.hidden_size, self.intermediate_size, self.num_hidden_layers, self.vocab_size
        D, Hq, Hkv = self.head_dim, self.num_attention_heads, self.num_key_value_heads
        active = 3 * H * I * (self.num_experts_per_tok if self.num_local_experts else 1)     # experts a token visits
        mm = L * ((Hq + 2 * Hkv) * D * H + Hq * D * H + active) + V * H
        attn = 12 * L * Hq * D * seq_len * (0.5 if causal else 1.0)
        return 6.0 * mm + attn


PRESETS: dict[str, dict[str, Any]] = {
    "tiny": dict(vocab_size=32000, hidden_size=256, intermediate_size=688, num_hidden_layers=4,
                 num_attention_heads=4, num_key_value_heads=4, rms_norm_eps=1e-5, rope_theta=10000.0),
    "llama3-8b": dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                      num_attention_heads=32, num_key_value_heads=8, rms_norm_eps=1e-5, rope_theta=500000.0,
                      max_position_embeddings=131072),
    "llama3-70b": dict(vocab_size=128256, hidden_size=8192, intermediate_size=28672, num_hidden_layers=80,
                       num_attention_heads=64, num_key_value_heads=8, rms_norm_eps=1e-5, rope_theta=500000.0,
                       max_position_embeddings=131072),
    "llama3-1b": dict(vocab_size=128256, hidden_size=2048, intermediate_size=8192, num_hidden_layers=16,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=64, rope_theta=500000.0,
                      tie_word_embeddings=True, max_position_embeddings=131072),
    "mistral-7b": dict(vocab_size=32000, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                       num_attention_heads=32, num_key_value_heads=8, rope_theta=10000.0, sliding_window=4096,
                       model_type="mistral"),
    "qwen2-7b": dict(vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
                     num_attention_heads=28, num_key_value_heads=4, rope_theta=1000000.0, rms_norm_eps=1e-6,
                     model_type="qwen2", attention_bias=True),
    "mixtral-8x7b": dict(vocab_size=32000, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                         num_attention_heads=32, num_key_value_heads=8, rope_theta=1000000.0, model_type="mixtral",
                         num_local_experts=8, num_experts_per_tok=2, max_position_embeddings=32768),
    "moe-tiny": dict(vocab_size=32000, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                     num_attention_heads=4, num_key_value_heads=2, model_type="mixtral", num_local_experts=4,
                     num_experts_per_tok=2),
}


def preset_config(name: str, **overrides) -> LlamaConfig:
    d = dict(PRESETS[name])
    d.update(overrides)
    return LlamaConfig(**d)


_TP_FIRST, _TP_LAST = ("wqkv", "w_gate_up"), ("wo", "w_down")


def _lin(mod, x, name: str):
    """x @ W^T plus the low-rank adapter of that weight when one is attached.

    `mod.fp8`: the product runs on the fp8 tensor-core kernels (`mod.fp8_recipe`: "rowwise" = forward, dgrad and wgrad
    in fp8 with per-token / per-feature scales; "block" = 1 x 128 / 128 x 128 scales, wgrad in bf16).
    `mod.tp_ctx` (set by the tensor-parallel wrapper on the fused back-end, with sequence parallelism): `x` of the
    block's first projection is this rank's token shard and the all-gather runs inside the GEMM kernel; the block's
    last projection reduce-scatters its output over the token dimension from the GEMM epilogue."""
    w = getattr(mod, name)
    tp = getattr(mod, "tp_ctx", None)
    if tp is not None and x.is_cuda and x.dtype == torch.bfloat16 and mod.lora is None:
        y = _tp_fused_lin(x, w, name, tp)
        if y is not None:
            return y
    has_lora = mod.lora is not None and name in mod.lora
    if has_lora and not getattr(mod, "fp8", False) and hasattr(mod.lora[name], "linear"):
        return mod.lora[name].linear(x, w)
    if getattr(mod, "fp8", False) and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 128 == 0 \
            and w.shape[0] % 8 == 0:
        from ..ops import fp8 as fp8_ops
        y = fp8_ops.fp8_linear(x, w, recipe=getattr(mod, "fp8_recipe", "rowwise"),
                               grad_format=getattr(mod, "fp8_grad_format", "e4m3"))
    else:
        y = gemm.linear(x, w)
    if has_lora:
        y = y + mod.lora[name](x)
    return y


def _tp_fused_lin(x, w, name, tp):
    """First / last projection of a tensor-parallel block on the fused all-gather->GEMM / GEMM->reduce-scatter
    kernels (one sequence, token-sharded).  None when the shape does not fit their tiling: the caller's wrapper then
    gathers / scatters with library collectives around ordinary GEMMs."""
    from ..parallel import tp_fused
    if x.dim() != 3 or x.shape[0] != 1:
        return None
    if name in _TP_FIRST:
        S_loc, K = x.shape[1], x.shape[2]
        if S_loc % 128 != 0 or K % 64 != 0:
            return None
        return tp_fused.all_gather_linear(x.view(S_loc, K), w, tp).view(1, S_loc * tp.size, w.shape[0])
    if name in _TP_LAST:
        S, K = x.shape[1], x.shape[2]
        if S % (128 * tp.size) != 0 or K % 64 != 0:
            return None
        return tp_fused.linear_reduce(x.reshape(S, K), w, tp, scatter=True).view(1, S // tp.size, w.shape[0])
    return None


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, offset: float = 0.0):
        super().__init__()
        self.weight = nn.Parameter(torch.full((dim,), 1.0 - offset))
        self.eps, self.offset = eps, offset

    def forward(self, x, residual=None):
        return norm.rmsnorm(x, self.weight, self.eps, residual, self.offset)


class LlamaAttention(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        self.n_heads, self.n_kv, self.hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        self.wqkv = nn.Parameter(torch.empty((self.n_heads + 2 * self.n_kv) * self.hd, cfg.hidden_size))
        self.wo = nn.Parameter(torch.empty(cfg.hidden_size, self.n_heads * self.hd))
        self.bqkv = nn.Parameter(torch.zeros((self.n_heads + 2 * self.n_kv) * self.hd)) if cfg.attention_bias else None
        self.lora = None      # nn.ModuleDict of low-rank adapters keyed by weight name (see lora.py)
        self.cp_group = None  # context-parallel process group (ring attention) when set

    def forward(self, x, cos, sin, position_ids=None, cu_seqlens=None, doc_ids=None, kv_cache=None):
        qkv = _lin(self, x, "wqkv")
        if self.bqkv is not None:
            qkv = qkv + self.bqkv
        return self.attend(qkv, cos, sin, position_ids, cu_seqlens, doc_ids, kv_cache)

    def attend(self, qkv, cos, sin, position_ids=None, cu_seqlens=None, doc_ids=None, kv_cache=None):
        """Everything after the fused q|k|v projection: rotary embedding, attention, output projection."""
        offset = 0 if kv_cache is None else kv_cache.seq_len
        qkv = rope.apply_rope_qkv(qkv, self.n_heads + self.n_kv, self.hd, cos, sin, position_ids, qkv.shape[-2], offset,
                                  self.cfg.rope_interleaved, inplace=True)
        if kv_cache is not None:
            o = kv_cache.attend(qkv, self)
        elif self.cp_group is not None:
            if getattr(self, "cp_mode", "ring") == "ulysses":
                # contiguous token shards; all-to-all to head shards, ordinary attention over the whole sequence
                from ..parallel.cp import ulysses_attention
                B, S = qkv.shape[0], qkv.shape[1]
                q, k, v = qkv.split((self.n_heads * self.hd, self.n_kv * self.hd, self.n_kv * self.hd), dim=-1)
                o = ulysses_attention(q.reshape(B, S, self.n_heads, self.hd), k.reshape(B, S, self.n_kv, self.hd),
                                      v.reshape(B, S, self.n_kv, self.hd), self.cp_group, True, None,
                                      self.cfg.sliding_window, self.cfg.attn_logit_softcap).reshape(B, S, -1)
            else:
                from ..parallel.cp import attention_qkv_cp
                o = attention_qkv_cp(qkv, self.n_heads, self.n_kv, self.hd, self.cp_group)
        else:
            o = attention.attention_qkv(qkv, self.n_heads, self.n_kv, self.hd, True, None, self.cfg.sliding_window,
                                        self.cfg.attn_logit_softcap, cu_seqlens, doc_ids)
        return _lin(self, o, "wo")


class LlamaMLP(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.act = cfg.hidden_act
        self.w_gate_up = nn.Parameter(torch.empty(2 * cfg.intermediate_size, cfg.hidden_size))
        self.w_down = nn.Parameter(torch.empty(cfg.hidden_size, cfg.intermediate_size))
        self.lora = None

    def forward(self, x):
        return _lin(self, activation.glu(_lin(self, x, "w_gate_up"), self.act), "w_down")


class LlamaMoEMLP(nn.Module):
    """Top-k mixture of gated experts (Mixtral layout: router [E, H], experts' gate|up [E, 2I, H] and down [E, H, I]).
    Routing = softmax over all experts, top-k, optional renormalisation.  On bf16 CUDA tensors the router top-k, the
    device-side routing plan, the permute into 128-aligned expert segments, two grouped tcgen05 GEMMs and the weighted
    combine are the kernels of ops/moe.py; elsewhere a loop over the experts gives the same result."""

    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        E, H, I = cfg.num_local_experts, cfg.hidden_size, cfg.intermediate_size
        self.act, self.top_k, self.norm_topk = cfg.hidden_act, cfg.num_experts_per_tok, cfg.norm_topk_prob
        self.aux_coef = cfg.router_aux_loss_coef
        self.router = nn.Parameter(torch.empty(E, H))
        self.w_gate_up = nn.Parameter(torch.empty(E, 2 * I, H))
        self.w_down = nn.Parameter(torch.empty(E, H, I))
        self.lora = None
        self.aux_loss: torch.Tensor | None = None

    def forward(self, x):
        from ..ops import moe as moe_ops
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        logits = F.linear(x2, self.router)                       # [T, E]: a few experts wide, not worth a tiled GEMM
        w, ids, probs = moe_ops.topk_softmax(logits, self.top_k, self.norm_topk)     # kernel on CUDA, torch ops on CPU
        if moe_ops.available(x2):
            y = moe_ops.moe_ffn(x2, ids, w.to(x2.dtype), self.w_gate_up, self.w_down, self.act)
        else:
            y = moe_ops.moe_ffn_reference(x2, ids, w, self.w_gate_up, self.w_down, self.act)
        if self.aux_coef > 0 and self.training:
            # Switch-style balance term: E * sum_e (fraction of routed slots on e) * (mean router probability of e)
            E = self.router.shape[0]
            frac = torch.zeros(E, device=x.device).index_add_(0, ids.reshape(-1).long(),
                                                              torch.ones(ids.numel(), device=x.device)) / ids.numel()
            self.aux_loss = E * (frac * probs.mean(0)).sum()
        return y.view(shape)


class LlamaDecoderLayer(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.norm_weight_offset)
        self.self_attn = LlamaAttention(cfg)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.norm_weight_offset)
        self.mlp = LlamaMoEMLP(cfg) if cfg.num_local_experts > 0 else LlamaMLP(cfg)
        self.op_selective = False   # keep only GEMM-side tensors; norm / GLU outputs are rebuilt in backward

    def forward(self, x, residual, cos, sin, position_ids=None, cu_seqlens=None, doc_ids=None, kv_cache=None):
        if self.op_selective and self.training and kv_cache is None and self.self_attn.lora is None \
                and self.mlp.lora is None and not getattr(self.mlp, "fp8", False) and self.self_attn.bqkv is None \
                and isinstance(self.mlp, LlamaMLP) and self.input_layernorm.offset == 0.0:
            n1, n2 = self.input_layernorm, self.post_attention_layernorm
            qkv, residual = fused_blocks.norm_linear(x, residual, n1.weight, self.self_attn.wqkv, n1.eps)
            a = self.self_attn.attend(qkv, cos, sin, position_ids, cu_seqlens, doc_ids, None)
            gu, residual = fused_blocks.norm_linear(a, residual, n2.weight, self.mlp.w_gate_up, n2.eps)
            return fused_blocks.glu_linear(gu, self.mlp.w_down, self.mlp.act), residual
        h, residual = self.input_layernorm(x, residual)
        a = self.self_attn(h, cos, sin, position_ids, cu_seqlens, doc_ids, kv_cache)
        h, residual = self.post_attention_layernorm(a, residual)
        return self.mlp(h), residual


@dataclass
class CausalLMOutput:
    loss: torch.Tensor | None = None
    logits: torch.Tensor | None = None
    hidden_states: torch.Tensor | None = None
    num_tokens: torch.Tensor | None = None


class LlamaModel(nn.Module):
    def __init__(self, cfg: LlamaConfig, layer_range: range | None = None):
        """`layer_range`: build only these decoder layers (one pipeline stage's); the others are placeholders."""
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList(LlamaDecoderLayer(cfg) if (layer_range is None or i in layer_range) else nn.Identity()
                                    for i in range(cfg.num_hidden_layers))
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.norm_weight_offset)
        self.gradient_checkpointing = False
        self.checkpoint_every = 1
        self._rope_cache: dict = {}

    def rope_tables(self, device, needed: int):
        key = (str(device),)
        cached = self._rope_cache.get(key)
        if cached is None or cached[0].shape[0] < needed:
            n = max(needed, min(self.cfg.max_position_embeddings, 8192))
            sc = dict(self.cfg.rope_scaling or {})
            kind = sc.pop("rope_type", sc.pop("type", "none"))
            kw = {}
            if kind != "none":
                kw = dict(scaling=kind, factor=sc.get("factor", 1.0),
                          original_max_pos=sc.get("original_max_position_embeddings", 8192),
                          low_freq_factor=sc.get("low_freq_factor", 1.0),
                          high_freq_factor=sc.get("high_freq_factor", 4.0))
                if str(kind).lower() == "longrope":
                    kw.update(long_factor=sc.get("long_factor"), short_factor=sc.get("short_factor"))
            cached = rope.rope_tables(n, self.cfg.head_dim, self.cfg.rope_theta, device, **kw)
            self._rope_cache[key] = cached
        return cached

    def forward(self, input_ids, position_ids=None, cu_seqlens=None, doc_ids=None, kv_caches=None,
                inputs_embeds=None):
        x = self.embed_tokens(input_ids) if inputs_embeds is None else inputs_embeds
        if self.cfg.scale_embeddings and inputs_embeds is None:
            x = x * torch.tensor(self.cfg.hidden_size ** 0.5, dtype=x.dtype)
        S = x.shape[1]
        past = 0 if not kv_caches else kv_caches[0].seq_len
        need = S + past
        if position_ids is not None:
            need = max(need, self.cfg.max_position_embeddings if self.cfg.max_position_embeddings <= 1 << 17 else need)
        cos, sin = self.rope_tables(x.device, need)
        residual = None
        sp = getattr(self, "sp_ctx", None)
        if sp is not None:
            # sequence parallelism: the residual stream between blocks holds S / tp tokens per rank
            from ..parallel import tp as TP
            if x.shape[0] != 1:
                raise ValueError("sequence-parallel training expects one sequence per micro-batch")
            x = TP.scatter_to_sequence_parallel_region(x.view(S, -1), sp).view(1, S // sp.size, -1)
        for i, layer in enumerate(self.layers):
            cache = None if kv_caches is None else kv_caches[i]
            ck = getattr(self, "checkpoint_layers", None)
            recompute = (i in ck) if ck is not None else (i % self.checkpoint_every == 0)
            if _recompute_switch.wanted(self.gradient_checkpointing and recompute, self.training):
                x, residual = checkpoint(layer, x, residual, cos, sin, position_ids, cu_seqlens, doc_ids, None,
                                         use_reentrant=False)
            else:
                x, residual = layer(x, residual, cos, sin, position_ids, cu_seqlens, doc_ids, cache)
        x, _ = self.norm(x, residual)
        if sp is not None:
            from ..parallel import tp as TP
            # every rank then computes the full loss on the gathered tokens: the backward of the gather sums the
            # tp copies of the gradient, so it is divided by tp here
            x = TP.all_gather_from_sequence_parallel_region(x.view(S // sp.size, -1), sp).view(1, S, -1)
            x = _ScaleGrad.apply(x, 1.0 / sp.size)
        return x


class _ScaleGrad(torch.autograd.Function):
    """Identity whose backward multiplies the gradient by a constant."""

    @staticmethod
    def forward(ctx, x, scale):
        ctx.scale = scale
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return g * ctx.scale, None


class LlamaForCausalLM(nn.Module):
    """Decoder + loss head. `forward(input_ids, labels=...)` shifts labels by one (labels are NOT pre-shifted,
    as in data_pipeline/trainer/trainers/sota_trainer.py:2044-2055) and returns the mean loss over
    non-ignored tokens."""

    def __init__(self, cfg: LlamaConfig, layer_range: range | None = None, init: bool = True):
        super().__init__()
        self.config = cfg
        self.model = LlamaModel(cfg, layer_range)
        self.lm_head = None if cfg.tie_word_embeddings else nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size))
        self.loss_chunk_tokens = cross_entropy.DEFAULT_CHUNK_TOKENS
        if init:
            self.reset_parameters()

    # ---------------------------------------------------------------- init / introspection
    @torch.no_grad()
    def reset_parameters(self, seed: int | None = None, on_device: bool = False):
        """Normal(0, initializer_range) weights (output projections scaled by 1/sqrt(2L)), unit norm weights.  With a
        seed the values come from a CPU generator, so every device and every rank builds the same model; `on_device`
        draws them with the parameters' own device generator instead (seconds instead of minutes for tens of billions
        of parameters; the values then depend on the device type, not only on the seed)."""
        gen = None
        if seed is not None and not on_device:
            gen = torch.Generator(device="cpu").manual_seed(seed)
        dgen: dict = {}
        std = self.config.initializer_range
        for name, p in self.named_parameters():
            if name.endswith("bqkv"):
                p.zero_()
            elif p.dim() == 1:
                p.fill_(1.0 - self.config.norm_weight_offset)
            else:
                s = std
                if name.endswith("wo") or name.endswith("w_down"):
                    s = std / math.sqrt(2 * self.config.num_hidden_layers)
                if gen is not None:
                    p.copy_(torch.randn(p.shape, generator=gen) * s)
                elif seed is not None:
                    g = dgen.get(p.device)
                    if g is None:
                        g = dgen[p.device] = torch.Generator(device=p.device).manual_seed(seed)
                    p.normal_(0.0, s, generator=g)
                else:
                    p.normal_(0.0, s)

    @property
    def head_weight(self) -> torch.Tensor:
        return self.model.embed_tokens.weight if self.lm_head is None else self.lm_head

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def gradient_checkpointing_enable(self, every: int = 1):
        self.model.gradient_checkpointing = True
        self.model.checkpoint_every = max(1, every)

    def enable_fp8(self, enabled: bool = True, recipe: str = "rowwise", grad_format: str = "e4m3"):
        """fp8 GEMMs for the attention and MLP projections (the head and the embedding stay bf16).  recipe "rowwise":
        forward, dgrad and wgrad in fp8 with per-token / per-feature scales (gradients in `grad_format`, e4m3 or e5m2);
        "block": 1 x 128 / 128 x 128 block scales, forward and dgrad in fp8."""
        for layer in self.model.layers:
            if isinstance(layer, nn.Identity):        # another pipeline stage's layer (not built on this rank)
                continue
            for blk in (layer.self_attn, layer.mlp):
                blk = getattr(blk, "inner", blk)      # under tensor parallelism the block sits inside its wrapper
                blk.fp8, blk.fp8_recipe, blk.fp8_grad_format = enabled, recipe, grad_format

    def op_selective_recompute(self, enabled: bool = True):
        """Operator-level selective recomputation: no layer is re-run, but norm and GLU outputs are rebuilt in
        backward instead of stored (see ops/fused_blocks.py)."""
        for layer in self.model.layers:
            if not isinstance(layer, nn.Identity):
                layer.op_selective = enabled

    def gradient_checkpointing_disable(self):
        self.model.gradient_checkpointing = False

    # ---------------------------------------------------------------- forward
    def forward(self, input_ids=None, attention_mask=None, labels=None, position_ids=None, cu_seqlens=None,
                doc_ids=None, kv_caches=None, return_logits: bool | None = None, loss_scale: float = 1.0,
                label_smoothing: float = 0.0, ignore_index: int = -100, shift_labels: bool = True,
                inputs_embeds=None, loss_denominator=None, **_unused) -> CausalLMOutput:
        h = self.model(input_ids, position_ids, cu_seqlens, doc_ids, kv_caches, inputs_embeds)
        out = CausalLMOutput(hidden_states=h)
        if labels is not None:
            if attention_mask is not None:
                labels = labels.masked_fill(attention_mask == 0, ignore_index)
            if shift_labels:
                tgt = torch.full_like(labels, ignore_index)
                tgt[..., :-1] = labels[..., 1:]
                if doc_ids is not None:   # never predict across a packed-document boundary
                    tgt[..., :-1] = tgt[..., :-1].masked_fill(doc_ids[..., 1:] != doc_ids[..., :-1], ignore_index)
            else:
                tgt = labels
            loss, count = cross_entropy.fused_linear_cross_entropy(
                h, self.head_weight, tgt, ignore_index, label_smoothing, 1.0, self.config.final_logit_softcap,
                self.loss_chunk_tokens, "mean", loss_scale, loss_denominator)
            if self.config.num_local_experts > 0 and self.config.router_aux_loss_coef > 0 and self.training:
                aux = [l.mlp.aux_loss for l in self.model.layers if getattr(l.mlp, "aux_loss", None) is not None]
                if aux:
                    loss = loss + self.config.router_aux_loss_coef * loss_scale * torch.stack(aux).mean()
            out.loss, out.num_tokens = loss, count
        if return_logits or (return_logits is None and labels is None):
            out.logits = self.logits(h)
        return out

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        z = gemm.linear(hidden, self.head_weight)
        cap = self.config.final_logit_softcap
        return cap * torch.tanh(z / cap) if cap and cap > 0 else z

    # ---------------------------------------------------------------- HF interop
    @torch.no_grad()
    def to_hf_state_dict(self, tp=None, first: bool = True, last: bool = True,
                         keep: bool = True) -> dict[str, torch.Tensor]:
        """Weights in HuggingFace Llama naming (layout of transformers' LlamaForCausalLM checkpoints).

        `tp`: a tensor-parallel context; every projection is then gathered over its group to full width (a
        collective: all ranks of the group call this), one tensor at a time, landing on the host.  `keep=False`
        takes part in the gathers and returns an empty dict (ranks that do not write).
        Layers replaced by `nn.Identity` (other pipeline stages) are skipped; `first` / `last` say whether this
        stage owns the embedding and the final norm + head."""
        import torch.distributed as dist
        cfg = self.config
        D, Hq, Hkv, I = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size
        ws = tp.size if tp is not None and tp.active else 1
        sd: dict[str, torch.Tensor] = {}

        def full(t, dim):
            t = t.detach()
            if ws == 1:
                return t
            parts = [torch.empty_like(t) for _ in range(ws)]
            dist.all_gather(parts, t.contiguous(), group=tp.group)
            return torch.cat(parts, dim).cpu() if keep else None

        def put(name, t):
            if keep:
                sd[name] = t

        if first:
            put("model.embed_tokens.weight", self.model.embed_tokens.weight.detach())
        if last:
            put("model.norm.weight", self.model.norm.weight.detach())
        for i, l in enumerate(self.model.layers):
            if isinstance(l, nn.Identity):
                continue
            p = f"model.layers.{i}."
            attn, mlp = getattr(l.self_attn, "inner", l.self_attn), getattr(l.mlp, "inner", l.mlp)
            q, k, v = attn.wqkv.detach().split((Hq // ws * D, Hkv // ws * D, Hkv // ws * D), dim=0)
            items = [("self_attn.q_proj", q, 0), ("self_attn.k_proj", k, 0), ("self_attn.v_proj", v, 0),
                     ("self_attn.o_proj", attn.wo, 1)]
            if hasattr(mlp, "full_expert_weights"):        # expert-parallel block: gather the experts (collective)
                gu, dn = mlp.full_expert_weights()
                put(p + "mlp.gate.weight", mlp.router.detach())
                put(p + "mlp.experts.gate_up_proj", gu)
                put(p + "mlp.experts.down_proj", dn)
            elif isinstance(mlp, LlamaMoEMLP):
                if ws > 1:
                    raise NotImplementedError("mixture-of-experts layers are sharded by expert parallelism, not tp")
                put(p + "mlp.gate.weight", mlp.router.detach())
                put(p + "mlp.experts.gate_up_proj", mlp.w_gate_up.detach())
                put(p + "mlp.experts.down_proj", mlp.w_down.detach())
            else:
                g, u = mlp.w_gate_up.detach().split((I // ws, I // ws), dim=0)
                items += [("mlp.gate_proj", g, 0), ("mlp.up_proj", u, 0), ("mlp.down_proj", mlp.w_down, 1)]
            for name, t, dim in items:
                put(p + name + ".weight", full(t, dim))
            if attn.bqkv is not None:
                bq, bk, bv = attn.bqkv.detach().split((Hq // ws * D, Hkv // ws * D, Hkv // ws * D), dim=0)
                for name, t in (("q_proj", bq), ("k_proj", bk), ("v_proj", bv)):
                    put(p + f"self_attn.{name}.bias", full(t, 0))
            put(p + "input_layernorm.weight", l.input_layernorm.weight.detach())
            put(p + "post_attention_layernorm.weight", l.post_attention_layernorm.weight.detach())
        if self.lm_head is not None and last:
            put("lm_head.weight", self.lm_head.detach())
        return sd

    @torch.no_grad()
    def load_hf_state_dict(self, sd: dict[str, torch.Tensor], strict: bool = True, tp=None) -> list[str]:
        """Inverse of `to_hf_state_dict`.  With a tensor-parallel context each rank copies its slice of every
        projection (head groups of q/k/v, column blocks of gate/up, input blocks of o/down); `nn.Identity` layers
        (other pipeline stages) are skipped."""
        missing = []
        ws = tp.size if tp is not None and tp.active else 1
        r = tp.rank if ws > 1 else 0

        def get(name, dim=None):
            if name not in sd:
                missing.append(name)
                return None
            t = sd[name]
            if dim is not None and ws > 1:
                n = t.shape[dim] // ws
                t = t.narrow(dim, r * n, n)
            return t

        def put(dst, parts):
            if any(p is None for p in parts):
                return
            dst.copy_(torch.cat([p.to(dst.dtype) for p in parts], dim=0) if len(parts) > 1 else parts[0])

        put(self.model.embed_tokens.weight, [get("model.embed_tokens.weight")])
        put(self.model.norm.weight, [get("model.norm.weight")])
        for i, l in enumerate(self.model.layers):
            if isinstance(l, nn.Identity):
                continue
            p = f"model.layers.{i}."
            attn, mlp = getattr(l.self_attn, "inner", l.self_attn), getattr(l.mlp, "inner", l.mlp)
            put(attn.wqkv, [get(p + f"self_attn.{n}_proj.weight", 0) for n in "qkv"])
            put(attn.wo, [get(p + "self_attn.o_proj.weight", 1)])
            if attn.bqkv is not None:
                put(attn.bqkv, [get(p + f"self_attn.{n}_proj.bias", 0) for n in "qkv"])
            if hasattr(mlp, "full_expert_weights"):
                # expert-parallel block: this rank's experts are a contiguous slice of the stacked expert tensors
                El, r_ep = mlp.w_gate_up.shape[0], mlp.dispatcher.rank
                put(mlp.router, [get(p + "mlp.gate.weight")])
                gu, dn = get(p + "mlp.experts.gate_up_proj"), get(p + "mlp.experts.down_proj")
                put(mlp.w_gate_up, [None if gu is None else gu[r_ep * El:(r_ep + 1) * El]])
                put(mlp.w_down, [None if dn is None else dn[r_ep * El:(r_ep + 1) * El]])
            elif isinstance(mlp, LlamaMoEMLP):
                put(mlp.router, [get(p + "mlp.gate.weight")])
                if p + "mlp.experts.gate_up_proj" in sd or p + "mlp.experts.0.w1.weight" not in sd:
                    put(mlp.w_gate_up, [get(p + "mlp.experts.gate_up_proj")])
                    put(mlp.w_down, [get(p + "mlp.experts.down_proj")])
                else:       # per-expert layout of older Mixtral checkpoints: w1 = gate, w3 = up, w2 = down
                    for e in range(mlp.router.shape[0]):
                        put(mlp.w_gate_up[e], [get(p + f"mlp.experts.{e}.w1.weight"), get(p + f"mlp.experts.{e}.w3.weight")])
                        put(mlp.w_down[e], [get(p + f"mlp.experts.{e}.w2.weight")])
            else:
                put(mlp.w_gate_up, [get(p + "mlp.gate_proj.weight", 0), get(p + "mlp.up_proj.weight", 0)])
                put(mlp.w_down, [get(p + "mlp.down_proj.weight", 1)])
            put(l.input_layernorm.weight, [get(p + "input_layernorm.weight")])
            put(l.post_attention_layernorm.weight, [get(p + "post_attention_layernorm.weight")])
        if self.lm_head is not None:
            put(self.lm_head, [get("lm_head.weight")])
        if strict and missing:
            raise KeyError(f"missing keys in state dict: {missing[:8]}{'...' if len(missing) > 8 else ''}")
        return missing

    def hf_config_dict(self) -> dict:
        c = self.config
        arch, mt = ("MixtralForCausalLM", "mixtral") if c.num_local_experts > 0 else \
            ("Qwen2ForCausalLM", "qwen2") if c.attention_bias else \
            ("GemmaForCausalLM", "gemma") if c.norm_weight_offset == 1.0 and c.scale_embeddings else \
            ("LlamaForCausalLM", "llama")
        extra = {"num_local_experts": c.num_local_experts, "num_experts_per_tok": c.num_experts_per_tok,
                 "router_aux_loss_coef": c.router_aux_loss_coef} if c.num_local_experts > 0 else {}
        return {**extra, "architectures": [arch], "model_type": mt, "vocab_size": c.vocab_size,
                "hidden_size": c.hidden_size, "intermediate_size": c.intermediate_size,
                "num_hidden_layers": c.num_hidden_layers, "num_attention_heads": c.num_attention_heads,
                "num_key_value_heads": c.num_key_value_heads, "head_dim": c.head_dim, "rms_norm_eps": c.rms_norm_eps,
                "rope_theta": c.rope_theta, "rope_scaling": c.rope_scaling,
                "max_position_embeddings": c.max_position_embeddings, "tie_word_embeddings": c.tie_word_embeddings,
                "hidden_act": c.hidden_act, "torch_dtype": "bfloat16"}


def build_model(cfg: LlamaConfig | str | dict, dtype=torch.bfloat16, device=None, seed: int | None = None,
                layer_range: range | None = None, init_on_device: bool = False) -> LlamaForCausalLM:
    """Random-init decoder.  `layer_range`: only these layers are built (a pipeline stage); `init_on_device`: draw the
    weights with the device's generator (see `reset_parameters`)."""
    if isinstance(cfg, str):
        cfg = preset_config(cfg)
    elif isinstance(cfg, dict):
        cfg = LlamaConfig.from_dict(cfg)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        if device is not None:
            with torch.device(device):
                m = LlamaForCausalLM(cfg, layer_range, init=seed is None)
        else:
            m = LlamaForCausalLM(cfg, layer_range, init=seed is None)
    finally:
        torch.set_default_dtype(prev)
    if seed is not None:
        m.reset_parameters(seed, on_device=init_on_device)
    return m
