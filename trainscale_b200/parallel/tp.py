"""Tensor parallelism (Megatron column / row split) with optional sequence parallelism, for the framework decoder.

Covers data_pipeline/trainer/distributed/tensor_parallel.py:487-2282: the conjugate communication ops as
autograd functions (copy / reduce / scatter / gather over the hidden dim, all-gather / reduce-scatter over the
sequence dim), `ColumnParallelLinear`, `RowParallelLinear`, `VocabParallelEmbedding`,
`vocab_parallel_cross_entropy` (max / sum-exp / target-logit all-reduces), sequence-parallel norm gradient
all-reduce (data_pipeline/trainer/distributed/finalize_grads.py:148) and `shard_model_for_tensor_parallel`, which
here slices the trained weights (q/k/v by head, gate/up by column block) instead of re-initialising them.

Two communication back-ends: `nccl` (torch.distributed collectives: the measured baseline path) and `fused`
(csrc/tp_gemm.cu: all-gather fused into the consuming GEMM, reduce-scatter / all-reduce fused into the producing
GEMM's epilogue over peer memory).
"""
from __future__ import annotations

import contextlib
import math
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..ops import gemm
from ..utils.explicit_backward import ExplicitBackward as _ExplicitBackward
from ..utils.refargs import ANY, reference_kwargs


@dataclass
class TPContext:
    group: object | None
    size: int = 1
    rank: int = 0
    sequence_parallel: bool = False
    comm: str = "nccl"          # nccl | fused
    heap: object | None = None  # SymmetricHeap for the fused path

    @classmethod
    def from_group(cls, group, sequence_parallel=False, comm="nccl", heap=None) -> "TPContext":
        if group is None or not dist.is_initialized():
            return cls(None)
        return cls(group, dist.get_world_size(group), dist.get_rank(group), sequence_parallel, comm, heap)

    @property
    def active(self) -> bool:
        return self.size > 1


# ------------------------------------------------------------------------------------------------ raw collectives
def _all_reduce(x, ctx, op=dist.ReduceOp.SUM):
    if ctx.active:
        x = x.contiguous()
        dist.all_reduce(x, op=op, group=ctx.group)
    return x


def _all_gather_dim(x, ctx, dim):
    if not ctx.active:
        return x
    x = x.contiguous()
    if dim == 0 or x.dim() == 1:
        out = torch.empty((x.shape[0] * ctx.size, *x.shape[1:]), dtype=x.dtype, device=x.device)
        if x.is_cuda:
            dist.all_gather_into_tensor(out, x, group=ctx.group)
        else:
            parts = list(out.chunk(ctx.size, 0))
            dist.all_gather(parts, x, group=ctx.group)
        return out
    parts = [torch.empty_like(x) for _ in range(ctx.size)]
    dist.all_gather(parts, x, group=ctx.group)
    return torch.cat(parts, dim=dim)


def _reduce_scatter_dim0(x, ctx):
    if not ctx.active:
        return x
    x = x.contiguous()
    out = torch.empty((x.shape[0] // ctx.size, *x.shape[1:]), dtype=x.dtype, device=x.device)
    if x.is_cuda:
        dist.reduce_scatter_tensor(out, x, group=ctx.group)
    else:   # gloo: all-reduce then slice
        dist.all_reduce(x, group=ctx.group)
        out.copy_(x.chunk(ctx.size, 0)[ctx.rank])
    return out


def _split_dim(x, ctx, dim):
    return x.chunk(ctx.size, dim=dim)[ctx.rank].contiguous() if ctx.active else x


# ------------------------------------------------------------------------------------------------ autograd comm ops
class _CopyToTP(torch.autograd.Function):           # f: identity fwd, all-reduce bwd
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return x

    @staticmethod
    def backward(ctx, g):
        return _all_reduce(g, ctx.tp), None


class _ReduceFromTP(torch.autograd.Function):       # g: all-reduce fwd, identity bwd
    @staticmethod
    def forward(ctx, x, tp):
        return _all_reduce(x, tp)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _ScatterToTP(torch.autograd.Function):        # split last dim fwd, all-gather bwd
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return _split_dim(x, tp, -1)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_dim(g, ctx.tp, -1), None


class _GatherFromTP(torch.autograd.Function):       # all-gather last dim fwd, split bwd
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return _all_gather_dim(x, tp, -1)

    @staticmethod
    def backward(ctx, g):
        return _split_dim(g, ctx.tp, -1), None


class _GatherSeq(torch.autograd.Function):          # SP: all-gather tokens fwd, reduce-scatter bwd
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return _all_gather_dim(x, tp, 0)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_dim0(g, ctx.tp), None


class _ReduceScatterSeq(torch.autograd.Function):   # SP: reduce-scatter tokens fwd, all-gather bwd
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return _reduce_scatter_dim0(x, tp)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_dim(g, ctx.tp, 0), None


class _ScatterSeq(torch.autograd.Function):         # SP entry: split tokens fwd, all-gather bwd
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return _split_dim(x, tp, 0)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_dim(g, ctx.tp, 0), None


def _default_tp() -> TPContext:
    """Context of the registered tensor-parallel group (`tensor_parallel_context` / `ProcessGroupManager.initialize`);
    an inactive one when there is none.  Lets the region functions be called the reference's way, without a context."""
    m = ProcessGroupManager.get()
    g = m.tp_group if m.initialized else None
    return TPContext.from_group(g) if g is not None else TPContext(None)


def _region(fn_cls, dim):
    # the collective's dimension is fixed per function: last dim for the tensor-parallel pair, tokens (0) for the
    # sequence-parallel ones; the reference's `dim` argument is accepted when it names that dimension
    @reference_kwargs({"dim": (dim, None), "async_op": (False, None)}, input_="x")
    def region(x, tp=None):
        if isinstance(tp, (bool, int)):
            # the reference's second positional argument: `dim` (must name this function's dimension) or `async_op`
            if isinstance(tp, bool):
                if tp:
                    raise NotImplementedError("async_op=True is not supported by the region functions")
            elif dim is None or tp not in (dim, dim % max(x.dim(), 1), dim - x.dim() if dim >= 0 else dim + x.dim()):
                raise NotImplementedError(f"this region function works on dimension {dim}, not {tp}")
            tp = None
        tp = tp if tp is not None else _default_tp()
        return fn_cls.apply(x, tp) if tp.active else x
    return region


copy_to_tensor_parallel_region = _region(_CopyToTP, None)
reduce_from_tensor_parallel_region = _region(_ReduceFromTP, None)
scatter_to_tensor_parallel_region = _region(_ScatterToTP, -1)
gather_from_tensor_parallel_region = _region(_GatherFromTP, -1)
all_gather_from_sequence_parallel_region = _region(_GatherSeq, 0)
reduce_scatter_to_sequence_parallel_region = _region(_ReduceScatterSeq, 0)
scatter_to_sequence_parallel_region = _region(_ScatterSeq, 0)
for _n in ("copy_to_tensor_parallel_region", "reduce_from_tensor_parallel_region", "scatter_to_tensor_parallel_region",
           "gather_from_tensor_parallel_region", "all_gather_from_sequence_parallel_region",
           "reduce_scatter_to_sequence_parallel_region", "scatter_to_sequence_parallel_region"):
    globals()[_n].__name__ = globals()[_n].__qualname__ = _n


# ------------------------------------------------------------------------------------------------ layers
def _tp_ctor(third: str, **renames):
    """Constructor adapter of the tensor-parallel layers.  This framework passes the parallel context explicitly as
    the third argument (`Layer(in, out, tp, ...)`); the reference keeps it in process-global state and its third
    positional parameter is something else (`third`).  With this adapter a layer can be built either way: when no
    `TPContext` is given, the context of the registered tensor-parallel group is used (`tensor_parallel_context`), and
    the reference's options are honoured: `sequence_parallel` (a switch of the context), `init_method(weight)` (run on
    every weight of the layer after construction), `skip_bias_add` (refused: the bias is always added here), plus
    per-class keyword `renames`."""
    import dataclasses
    import functools
    import inspect

    def deco(init):
        sig = inspect.signature(init)

        @functools.wraps(init)
        def wrapper(self, *args, init_method=None, skip_bias_add=False, sequence_parallel=None, **kw):
            if skip_bias_add:
                raise NotImplementedError("skip_bias_add is not supported: the bias is added inside the layer")
            for ref, ours in renames.items():
                if ref in kw:
                    kw[ours] = kw.pop(ref)
            args = list(args)
            given = kw.get("tp") if "tp" in kw else (args[2] if len(args) >= 3 and isinstance(args[2], TPContext) else None)
            if given is None:
                if len(args) > 3:
                    raise TypeError("without a TPContext, pass the options after the third argument by keyword")
                if len(args) == 3:
                    kw[third] = args.pop()
                given = _default_tp()
                kw["tp"] = given
            if sequence_parallel is not None and bool(sequence_parallel) != given.sequence_parallel:
                new = dataclasses.replace(given, sequence_parallel=bool(sequence_parallel))
                if "tp" in kw:
                    kw["tp"] = new
                else:
                    args[2] = new
            init(self, *args, **kw)
            if init_method is not None:
                with torch.no_grad():
                    for n, p in self.named_parameters():
                        if n.endswith("weight") and p.dim() > 1:
                            init_method(p)

        params = [p.replace(default=None) if p.name == "tp" else p for p in sig.parameters.values()]
        # keep a valid ordering: parameters after `tp` need defaults too for inspection purposes only
        fixed, seen_default = [], False
        for p in params:
            if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD):
                if p.default is not p.empty:
                    seen_default = True
                elif seen_default:
                    p = p.replace(default=None)
            fixed.append(p)
        tail = [p for p in fixed if p.kind is inspect.Parameter.VAR_KEYWORD]
        head = [p for p in fixed if p.kind is not inspect.Parameter.VAR_KEYWORD]
        extra = [inspect.Parameter(n, inspect.Parameter.KEYWORD_ONLY, default=None)
                 for n in ("init_method", "skip_bias_add", "sequence_parallel", *renames) if n not in sig.parameters]
        wrapper.__signature__ = sig.replace(parameters=head + extra + tail)
        return wrapper
    return deco


class ColumnParallelLinear(nn.Module):
    """y_local = x W_local^T with W split along the output dim. With SP the input tokens are all-gathered first
    (fused into the GEMM on the `fused` back-end)."""

    @_tp_ctor("bias")
    def __init__(self, in_features: int, out_features: int, tp: TPContext, bias: bool = False, gather_output=False,
                 dtype=None, device=None):
        super().__init__()
        assert out_features % tp.size == 0, "out_features must divide by the TP size"
        self.tp, self.gather_output = tp, gather_output
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features // tp.size, in_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_features // tp.size, dtype=dtype, device=device)) if bias else None
        nn.init.normal_(self.weight, std=0.02)


    @reference_kwargs(input_="x")
    def forward(self, x):
        tp = self.tp
        if tp.active and tp.sequence_parallel:
            if tp.comm == "fused" and x.is_cuda:
                from . import tp_fused
                y = tp_fused.all_gather_linear(x, self.weight, tp)
            else:
                y = gemm.linear(all_gather_from_sequence_parallel_region(x, tp), self.weight)
        else:
            y = gemm.linear(copy_to_tensor_parallel_region(x, tp), self.weight)
        if self.bias is not None:
            y = y + self.bias
        return gather_from_tensor_parallel_region(y, tp) if self.gather_output else y


class RowParallelLinear(nn.Module):
    """y = sum_r x_r W_r^T with W split along the input dim; the partial sums are all-reduced, or reduce-scattered
    over tokens with SP (fused into the GEMM epilogue on the `fused` back-end)."""

    @_tp_ctor("bias")
    def __init__(self, in_features: int, out_features: int, tp: TPContext, bias: bool = False, input_is_parallel=True,
                 dtype=None, device=None):
        super().__init__()
        assert in_features % tp.size == 0, "in_features must divide by the TP size"
        self.tp, self.input_is_parallel = tp, input_is_parallel
        self.weight = nn.Parameter(torch.empty(out_features, in_features // tp.size, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None
        nn.init.normal_(self.weight, std=0.02)


    @reference_kwargs(input_="x")
    def forward(self, x):
        tp = self.tp
        if not self.input_is_parallel:
            x = scatter_to_tensor_parallel_region(x, tp)
        if tp.active and tp.comm == "fused" and x.is_cuda:
            from . import tp_fused
            y = tp_fused.linear_reduce(x, self.weight, tp, scatter=tp.sequence_parallel)
        else:
            y = gemm.linear(x, self.weight)
            y = reduce_scatter_to_sequence_parallel_region(y, tp) if tp.sequence_parallel else \
                reduce_from_tensor_parallel_region(y, tp)
        return y if self.bias is None else y + self.bias


class VocabParallelEmbedding(nn.Module):
    @_tp_ctor("padding_idx")
    def __init__(self, num_embeddings: int, embedding_dim: int, tp: TPContext, dtype=None, device=None,
                 padding_idx: int | None = None):
        """`padding_idx`: that token's row is zero and receives no gradient (on the rank that owns it)."""
        super().__init__()
        self.tp = tp
        self.num_embeddings = num_embeddings
        per = math.ceil(num_embeddings / tp.size)
        self.start, self.end = tp.rank * per, min(num_embeddings, (tp.rank + 1) * per)
        self.weight = nn.Parameter(torch.empty(per, embedding_dim, dtype=dtype, device=device))
        nn.init.normal_(self.weight, std=0.02)
        self.padding_idx = padding_idx
        self._local_pad = padding_idx - self.start if padding_idx is not None and self.start <= padding_idx < self.end \
            else None
        if self._local_pad is not None:
            with torch.no_grad():
                self.weight[self._local_pad].zero_()

    @reference_kwargs(input_="ids")
    def forward(self, ids):
        if not self.tp.active:
            return F.embedding(ids, self.weight, padding_idx=self._local_pad)
        mask = (ids < self.start) | (ids >= self.end)
        local = (ids - self.start).masked_fill(mask, 0)
        out = F.embedding(local, self.weight, padding_idx=self._local_pad).masked_fill(mask.unsqueeze(-1), 0.0)
        return reduce_from_tensor_parallel_region(out, self.tp)


class _VocabParallelCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits_local, labels, tp, vocab_start, ignore_index):
        z = logits_local.float()
        m = z.max(dim=-1).values
        m = _all_reduce(m, tp, dist.ReduceOp.MAX)
        z = z - m.unsqueeze(-1)
        ez = z.exp()
        s = _all_reduce(ez.sum(-1), tp)
        vend = vocab_start + z.shape[-1]
        mine = (labels >= vocab_start) & (labels < vend)
        idx = (labels - vocab_start).masked_fill(~mine, 0)
        tgt = z.gather(-1, idx.unsqueeze(-1)).squeeze(-1).masked_fill(~mine, 0.0)
        tgt = _all_reduce(tgt, tp)
        valid = labels != ignore_index
        loss = (s.log() - tgt).masked_fill(~valid, 0.0)
        ctx.save_for_backward(ez / s.unsqueeze(-1), idx, mine & valid, valid)
        return loss

    @staticmethod
    def backward(ctx, g):
        p, idx, mine, valid = ctx.saved_tensors
        grad = p.clone()
        grad.scatter_add_(-1, idx.unsqueeze(-1), -mine.unsqueeze(-1).to(grad.dtype))
        grad = grad * (g * valid).unsqueeze(-1)
        return grad, None, None, None, None


@reference_kwargs(logits="logits_local", targets="labels")
def vocab_parallel_cross_entropy(logits_local: torch.Tensor, labels: torch.Tensor, tp: TPContext | None = None,
                                 vocab_start: int | None = None, ignore_index: int = -100,
                                 label_smoothing: float = 0.0) -> torch.Tensor:
    """Per-token loss for logits split along the vocabulary; three small all-reduces (max, sum-exp, target logit).
    Without `tp` the registered tensor-parallel group is used and `vocab_start` defaults to rank x local vocabulary
    (the reference's call form `vocab_parallel_cross_entropy(logits, targets, label_smoothing)`).  Label smoothing
    mixes in the mean negative log-probability over the WHOLE vocabulary (one more all-reduce)."""
    tp = tp if tp is not None else _default_tp()
    if vocab_start is None:
        vocab_start = tp.rank * logits_local.shape[-1]
    loss = _VocabParallelCE.apply(logits_local, labels, tp, vocab_start, ignore_index)
    if label_smoothing:
        z = logits_local.float()
        m = _all_reduce(z.max(-1).values.detach().clone(), tp, dist.ReduceOp.MAX)
        lse = torch.log(_reduce_sum_differentiable(torch.exp(z - m[..., None]).sum(-1), tp)) + m
        mean_logit = _reduce_sum_differentiable(z.sum(-1), tp) / (z.shape[-1] * tp.size)
        smooth = (lse - mean_logit) * (labels != ignore_index)
        loss = (1.0 - label_smoothing) * loss + label_smoothing * smooth
    return loss


def _reduce_sum_differentiable(x, tp):
    """Sum over the tensor-parallel group whose backward passes the gradient through unchanged."""
    return _ReduceFromTP.apply(x, tp) if tp.active else x


class VocabParallelCrossEntropyLoss(_ExplicitBackward, nn.Module):
    def __init__(self, tp: TPContext, vocab_start: int, ignore_index: int = -100, reduction: str = "mean"):
        super().__init__()
        self.tp, self.vocab_start, self.ignore_index, self.reduction = tp, vocab_start, ignore_index, reduction

    def forward(self, logits_local, labels):
        loss = vocab_parallel_cross_entropy(logits_local, labels, self.tp, self.vocab_start, self.ignore_index)
        if self.reduction == "mean":
            return loss.sum() / (labels != self.ignore_index).sum().clamp(min=1)
        return loss.sum() if self.reduction == "sum" else loss


# ------------------------------------------------------------------------------------------------ model sharding
def shard_llama_state_for_tp(model, tp_size: int, tp_rank: int) -> None:
    """In place: keep this rank's slice of every projection of a framework decoder. q/k/v rows are taken per head
    group, gate/up per column block, o / down per input block; norms and embeddings stay replicated."""
    cfg = model.config
    D, Hq, Hkv, I = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size
    assert Hq % tp_size == 0 and Hkv % tp_size == 0 and I % tp_size == 0, "heads / ffn must divide by the TP size"
    hq, hkv, i_loc = Hq // tp_size, Hkv // tp_size, I // tp_size
    if getattr(cfg, "num_local_experts", 0) > 0:
        raise NotImplementedError("mixture-of-experts layers are distributed by expert parallelism (parallel/ep.py)")
    with torch.no_grad():
        for layer in model.model.layers:
            a, m = layer.self_attn, layer.mlp
            if getattr(a, "bqkv", None) is not None:
                bq, bk, bv = a.bqkv.data.split((Hq * D, Hkv * D, Hkv * D), dim=0)
                a.bqkv = nn.Parameter(torch.cat((bq[tp_rank * hq * D:(tp_rank + 1) * hq * D],
                                                 bk[tp_rank * hkv * D:(tp_rank + 1) * hkv * D],
                                                 bv[tp_rank * hkv * D:(tp_rank + 1) * hkv * D])).contiguous())
            q, k, v = a.wqkv.data.split((Hq * D, Hkv * D, Hkv * D), dim=0)
            a.wqkv = nn.Parameter(torch.cat((q[tp_rank * hq * D:(tp_rank + 1) * hq * D],
                                             k[tp_rank * hkv * D:(tp_rank + 1) * hkv * D],
                                             v[tp_rank * hkv * D:(tp_rank + 1) * hkv * D])).contiguous())
            a.wo = nn.Parameter(a.wo.data[:, tp_rank * hq * D:(tp_rank + 1) * hq * D].contiguous())
            a.n_heads, a.n_kv = hq, hkv
            g, u = m.w_gate_up.data.split((I, I), dim=0)
            m.w_gate_up = nn.Parameter(torch.cat((g[tp_rank * i_loc:(tp_rank + 1) * i_loc],
                                                  u[tp_rank * i_loc:(tp_rank + 1) * i_loc])).contiguous())
            m.w_down = nn.Parameter(m.w_down.data[:, tp_rank * i_loc:(tp_rank + 1) * i_loc].contiguous())


class _TPBlockIO(nn.Module):
    """Wraps a sub-module whose first GEMM is column-parallel and last GEMM is row-parallel."""

    def __init__(self, inner: nn.Module, tp: TPContext):
        super().__init__()
        self.inner, self.tp = inner, tp
        # fused back-end + sequence parallelism: the block's first projection gathers the token shards inside its GEMM
        # kernel and its last projection reduce-scatters from the GEMM epilogue (models/llama.py `_lin`)
        self.fused_sp = tp.sequence_parallel and tp.comm == "fused" and tp.heap is not None and \
            not getattr(inner, "fp8", False)
        if self.fused_sp:
            inner.tp_ctx = tp

    def _fits_fused(self, x) -> bool:
        B, S, H = x.shape
        return x.is_cuda and x.dtype == torch.bfloat16 and B == 1 and S % 128 == 0 and H % 64 == 0 and \
            getattr(self.inner, "lora", None) is None and not getattr(self.inner, "fp8", False)

    def forward(self, x, *args, **kw):
        tp = self.tp
        if tp.sequence_parallel:
            if self.fused_sp:
                if self._fits_fused(x) and kw.get("kv_cache") is None:
                    self.inner.tp_ctx = tp
                    return self.inner(x, *args, **kw)
                self.inner.tp_ctx = None       # this call goes through the library collectives below
            B, S, H = x.shape   # tokens are sharded along S; gather them (B must be 1 per shard row-block)
            xg = all_gather_from_sequence_parallel_region(x.reshape(B * S, H), tp).view(B, S * tp.size, H) if B == 1 else \
                all_gather_from_sequence_parallel_region(x.transpose(0, 1).contiguous(), tp).transpose(0, 1)
            y = self.inner(xg, *args, **kw)
            if B == 1:
                return reduce_scatter_to_sequence_parallel_region(y.reshape(-1, H), tp).view(B, S, H)
            return reduce_scatter_to_sequence_parallel_region(y.transpose(0, 1).contiguous(), tp).transpose(0, 1)
        return reduce_from_tensor_parallel_region(self.inner(copy_to_tensor_parallel_region(x, tp), *args, **kw), tp)


def shard_model_for_tensor_parallel(model, tp: "TPContext | TensorParallelConfig | None" = None, *, config=None):
    """Slice the weights for this TP rank and wrap attention / MLP with the conjugate communication ops.
    `tp` may also be a `TensorParallelConfig` (`config=` in the reference's spelling): the context is then built
    from the registered tensor-parallel group with that config's sequence-parallel switch.
    With sequence parallelism the caller feeds / receives token-sharded hidden states between blocks and must
    all-reduce the norm-weight gradients over the TP group (`allreduce_sequence_parallel_grads`)."""
    tp = tp if tp is not None else config
    if not isinstance(tp, TPContext):
        base = _default_tp()
        tp = TPContext(base.group, base.size, base.rank, bool(getattr(tp, "sequence_parallel_enabled", False)))
    if not tp.active:
        return model
    if getattr(model, "tp_presharded", 0) == tp.size:
        # built with this rank's slice only (random init): the replicated parameters must still agree inside the group
        with torch.no_grad():
            for n, p in model.named_parameters():
                if p.dim() == 1 or "embed_tokens" in n or "lm_head" in n:
                    dist.broadcast(p.data, src=dist.get_global_rank(tp.group, 0), group=tp.group)
    else:
        shard_llama_state_for_tp(model, tp.size, tp.rank)
    for layer in model.model.layers:
        if isinstance(layer, nn.Identity):      # another pipeline stage's layer
            continue
        layer.self_attn = _TPBlockIO(layer.self_attn, tp)
        layer.mlp = _TPBlockIO(layer.mlp, tp)
    model.tp = tp
    return model


def allreduce_sequence_parallel_grads(model, tp: TPContext) -> None:
    """Norm weights see only this rank's tokens under SP: sum their gradients over the TP group."""
    if not (tp.active and tp.sequence_parallel):
        return
    grads = []
    for n, p in model.named_parameters():
        if p.dim() == 1:
            g = getattr(p, "main_grad", None) if p.grad is None else p.grad
            if g is not None:
                grads.append(g)
    if grads:
        flat = torch.cat([g.reshape(-1).float() for g in grads])
        dist.all_reduce(flat, group=tp.group)
        off = 0
        for g in grads:
            g.copy_(flat[off:off + g.numel()].view_as(g))
            off += g.numel()


# ------------------------------------------------------------------------------------------------ generic building blocks
class ProcessGroupManager:
    """Process groups of a [data, pipeline, tensor] layout (tensor ranks adjacent, so that they share a node's
    NVLink); sequence parallelism uses the tensor group.  One instance per process
    (data_pipeline/trainer/distributed/tensor_parallel.py:133-480 keeps the same registry)."""

    _instance: "ProcessGroupManager | None" = None

    def __init__(self):
        self.tp_size = self.pp_size = self.dp_size = 1
        self.tp_group = self.pp_group = self.dp_group = None
        self.tp_rank = self.pp_rank = self.dp_rank = 0
        self.initialized = False

    @classmethod
    def get(cls) -> "ProcessGroupManager":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def initialize(self, tensor_parallel_size: "int | TensorParallelConfig" = 1, pipeline_parallel_size: int = 1, *,
                   config=None, rank: int | None = None, world_size: int | None = None, backend: str | None = None
                   ) -> "ProcessGroupManager":
        """Collective over the whole job.  `initialize(config, rank, world_size, backend)` is the reference's form: the
        sizes come from the `TensorParallelConfig`; rank / world size / backend are those of the running process group
        (they are checked against it when given, never used to create one)."""
        cfg = config if config is not None else (tensor_parallel_size if not isinstance(tensor_parallel_size, int) else None)
        if cfg is not None:
            self.config = cfg
            if isinstance(pipeline_parallel_size, int) and rank is None and config is None and pipeline_parallel_size != 1:
                rank, pipeline_parallel_size = pipeline_parallel_size, 1          # positional (config, rank, ...)
            tensor_parallel_size = int(getattr(cfg, "tensor_parallel_size", 1))
            pipeline_parallel_size = int(getattr(cfg, "pipeline_parallel_size", pipeline_parallel_size))
        if dist.is_available() and dist.is_initialized():
            if world_size is not None and int(world_size) != dist.get_world_size():
                raise ValueError(f"world_size={world_size} but the process group has {dist.get_world_size()} ranks")
            if rank is not None and int(rank) != dist.get_rank():
                raise ValueError(f"rank={rank} but this process is rank {dist.get_rank()}")
        from .dist_kernels import create_process_groups
        self.tp_size, self.pp_size = tensor_parallel_size, pipeline_parallel_size
        if dist.is_available() and dist.is_initialized():
            world, rank = dist.get_world_size(), dist.get_rank()
            g = create_process_groups(tensor_parallel_size, pipeline_parallel_size)
            self.tp_group, self.pp_group, self.dp_group = g["tensor"], g["pipeline"], g["data"]
            self.dp_size = world // (tensor_parallel_size * pipeline_parallel_size)
            self.tp_rank = rank % tensor_parallel_size
            self.pp_rank = (rank // tensor_parallel_size) % pipeline_parallel_size
            self.dp_rank = rank // (tensor_parallel_size * pipeline_parallel_size)
        elif tensor_parallel_size * pipeline_parallel_size != 1:
            raise RuntimeError("model parallelism needs an initialised process group")
        self.initialized = True
        return self

    @property
    def sp_group(self):
        return self.tp_group

    def tp_context(self, sequence_parallel: bool = False, comm: str = "nccl", heap=None) -> TPContext:
        if self.tp_group is None:
            return TPContext(None, 1, 0, sequence_parallel, comm, heap)
        return TPContext.from_group(self.tp_group, sequence_parallel, comm, heap)

    def destroy(self) -> None:
        type(self)._instance = None

    # ---- accessors by mode name (data_pipeline/trainer/distributed/tensor_parallel.py:133-395): "tensor" |
    # "sequence" (the tensor group) | "pipeline" | "data"
    config = None

    @classmethod
    def get_instance(cls) -> "ProcessGroupManager":
        return cls.get()

    def is_initialized(self) -> bool:
        return self.initialized

    @staticmethod
    def _mode(mode) -> str:
        m = str(getattr(mode, "name", mode)).lower()
        return {"tensor": "tp", "tp": "tp", "sequence": "tp", "sp": "tp", "pipeline": "pp", "pp": "pp", "data": "dp",
                "dp": "dp"}[m]

    def get_group(self, mode="tensor"):
        return getattr(self, self._mode(mode) + "_group")

    def get_rank(self, mode="tensor") -> int:
        return getattr(self, self._mode(mode) + "_rank")

    def get_world_size(self, mode="tensor") -> int:
        return getattr(self, self._mode(mode) + "_size")

    def get_stream(self, mode="tensor"):
        """A side stream per mode for library collectives that should overlap compute (None without CUDA)."""
        if not torch.cuda.is_available():
            return None
        streams = self.__dict__.setdefault("_streams", {})
        key = self._mode(mode)
        if key not in streams:
            streams[key] = torch.cuda.Stream()
        return streams[key]

    def acquire_buffer(self, shape=None, dtype=torch.float32, device=None, *, numel: int | None = None) -> torch.Tensor:
        """A pooled scratch tensor of `shape` (or flat, of `numel` elements; `acquire_buffer(dtype, numel)` is the
        reference's order)."""
        if isinstance(shape, torch.dtype):
            shape, dtype = (dtype if isinstance(dtype, int) else numel), shape
        if shape is None:
            shape = numel
        shape = (int(shape),) if isinstance(shape, int) else tuple(shape)
        from .dist_utils import TensorPool
        pools = self.__dict__.setdefault("_pools", {})
        dev = torch.device(device) if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        if dev not in pools:
            pools[dev] = TensorPool(dev)
        return pools[dev].acquire(shape, dtype)

    @reference_kwargs(buffer="tensor")
    def release_buffer(self, tensor: torch.Tensor) -> None:
        for pool in self.__dict__.get("_pools", {}).values():
            pool.release(tensor)


class ParallelEmbedding(nn.Module):
    """Embedding table split along the HIDDEN dimension: every rank looks up all tokens in its slice of columns and the
    slices are all-gathered (no masking needed, unlike the vocabulary split)."""

    @_tp_ctor("padding_idx")
    def __init__(self, num_embeddings: int, embedding_dim: int, tp: TPContext, gather_output: bool = True,
                 dtype=None, device=None, padding_idx: int | None = None):
        super().__init__()
        assert embedding_dim % tp.size == 0, "embedding_dim must divide by the TP size"
        self.tp, self.gather_output, self.padding_idx = tp, gather_output, padding_idx
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.weight = nn.Parameter(torch.empty(num_embeddings, embedding_dim // tp.size, dtype=dtype, device=device))
        nn.init.normal_(self.weight, std=0.02)
        if padding_idx is not None:
            with torch.no_grad():
                self.weight[padding_idx].zero_()

    @reference_kwargs(input_="ids")
    def forward(self, ids):
        out = F.embedding(ids, self.weight, padding_idx=self.padding_idx)
        return gather_from_tensor_parallel_region(out, self.tp) if self.gather_output else out


class SequenceParallelLayerNorm(nn.Module):
    """RMSNorm / LayerNorm applied to this rank's tokens under sequence parallelism.  The weights are replicated but
    each rank sees only 1/tp of the tokens, so their gradients must be summed over the group: the parameters carry
    `sequence_parallel = True` and `allreduce_sequence_parallel_grads` picks them up."""

    def __init__(self, hidden_size: int | None = None, eps: float = 1e-5, rms: bool | None = None, bias: bool | None = None,
                 dtype=None, device=None, *, normalized_shape=None, elementwise_affine: bool = True,
                 sequence_parallel: bool = True):
        """`SequenceParallelLayerNorm(hidden_size)` is an RMSNorm (this framework's decoders use nothing else).  Built with
        the reference's `normalized_shape=` it is a LayerNorm with bias, as there
        (data_pipeline/trainer/distributed/tensor_parallel.py, SequenceParallelLayerNorm); `rms` / `bias` override either.
        `sequence_parallel=False` leaves the parameters unmarked (their gradients are then not summed over the group)."""
        if not elementwise_affine:
            raise NotImplementedError("a norm without weights has nothing to synchronise: use torch's functional norm")
        ref_form = normalized_shape is not None
        if ref_form:
            hidden_size = normalized_shape if isinstance(normalized_shape, int) else tuple(normalized_shape)[-1]
        rms = (not ref_form) if rms is None else rms
        bias = ref_form if bias is None else bias
        super().__init__()
        self.eps, self.rms = eps, rms
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(hidden_size, dtype=dtype, device=device)) if (bias and not rms) else None
        for p in self.parameters():
            p.sequence_parallel = bool(sequence_parallel)

    @reference_kwargs(input_="x")
    def forward(self, x):
        from ..ops import norm as N
        if self.rms:
            return N.rmsnorm(x, self.weight, self.eps)[0]
        return N.layernorm(x, self.weight, self.bias, self.eps)


class ParallelMLP(nn.Module):
    """Column-parallel up (gate|up for gated activations) -> activation -> row-parallel down: one collective per
    direction (all-reduce, or all-gather + reduce-scatter of tokens with sequence parallelism)."""

    @_tp_ctor("activation", use_gated="gated")
    def __init__(self, hidden_size: int, intermediate_size: int, tp: TPContext, gated: bool = True,
                 activation: str = "silu", bias: bool = False, dtype=None, device=None, dropout_prob: float = 0.0):
        super().__init__()
        self.dropout = nn.Dropout(dropout_prob) if dropout_prob else None
        self.tp, self.gated, self.activation = tp, gated, activation
        self.up = ColumnParallelLinear(hidden_size, intermediate_size, tp, bias, dtype=dtype, device=device)
        self.gate = ColumnParallelLinear(hidden_size, intermediate_size, tp, bias, dtype=dtype, device=device) \
            if gated else None
        self.down = RowParallelLinear(intermediate_size, hidden_size, tp, bias, dtype=dtype, device=device)

    def _act(self, x):
        return {"silu": F.silu, "gelu": F.gelu, "relu": F.relu}[self.activation](x)

    @reference_kwargs(hidden_states="x")
    def forward(self, x):
        h = self._act(self.gate(x)) * self.up(x) if self.gated else self._act(self.up(x))
        y = self.down(h)
        return self.dropout(y) if getattr(self, "dropout", None) is not None else y


class ParallelSelfAttention(nn.Module):
    """Heads split over the tensor group: column-parallel q / k / v (grouped-query: kv heads split too), local causal
    attention over this rank's heads, row-parallel output projection."""

    @_tp_ctor("num_kv_heads", num_attention_heads="num_heads", num_key_value_heads="num_kv_heads")
    def __init__(self, hidden_size: int, num_heads: int, tp: TPContext, num_kv_heads: int | None = None,
                 head_dim: int | None = None, causal: bool = True, rope_theta: float | None = 10000.0, bias: bool = False,
                 dtype=None, device=None, attention_dropout: float = 0.0):
        if attention_dropout:
            raise NotImplementedError("attention dropout is not supported by the attention kernels")
        super().__init__()
        kv = num_kv_heads or num_heads
        assert num_heads % tp.size == 0 and kv % tp.size == 0, "heads must divide by the TP size"
        self.tp, self.causal = tp, causal
        self.head_dim = head_dim or hidden_size // num_heads
        self.h_loc, self.kv_loc = num_heads // tp.size, kv // tp.size
        self.rope_theta = rope_theta
        D = self.head_dim
        self.q_proj = ColumnParallelLinear(hidden_size, num_heads * D, tp, bias, dtype=dtype, device=device)
        self.k_proj = ColumnParallelLinear(hidden_size, kv * D, tp, bias, dtype=dtype, device=device)
        self.v_proj = ColumnParallelLinear(hidden_size, kv * D, tp, bias, dtype=dtype, device=device)
        self.o_proj = RowParallelLinear(num_heads * D, hidden_size, tp, bias, dtype=dtype, device=device)

    def _rope(self, x, S):
        D = self.head_dim
        inv = 1.0 / (self.rope_theta ** (torch.arange(0, D, 2, device=x.device, dtype=torch.float32) / D))
        ang = torch.arange(S, device=x.device, dtype=torch.float32)[:, None] * inv[None]
        cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
        x1, x2 = x.float()[..., : D // 2], x.float()[..., D // 2:]
        return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), -1).to(x.dtype)

    @reference_kwargs({"attention_mask": (None,), "position_embeddings": (None,)}, hidden_states="x")
    def forward(self, x):
        """x: [B, S, H] (with sequence parallelism [B, S/tp, H]; B must be 1 there, tokens are the sharded axis).
        Masking is causal (or none) as configured and rotary positions are computed inside: an explicit
        `attention_mask` / `position_embeddings` is refused."""
        tp = self.tp
        sp = tp.active and tp.sequence_parallel
        B = x.shape[0]
        if sp:
            assert B == 1, "sequence parallelism shards the tokens of one sequence"
            x = x.reshape(-1, x.shape[-1])
        q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
        S = q.shape[0] if sp else q.shape[1]
        q = q.view(B, S, self.h_loc, self.head_dim)
        k = k.view(B, S, self.kv_loc, self.head_dim)
        v = v.view(B, S, self.kv_loc, self.head_dim)
        if self.rope_theta:
            q, k = self._rope(q, S), self._rope(k, S)
        from ..ops import attention as A
        qkv = torch.cat((q.reshape(B, S, -1), k.reshape(B, S, -1), v.reshape(B, S, -1)), dim=-1)
        o = A.attention_qkv(qkv, self.h_loc, self.kv_loc, self.head_dim, causal=self.causal)
        o = o.reshape(B, S, self.h_loc * self.head_dim)
        y = self.o_proj(o.reshape(-1, o.shape[-1]) if sp else o)
        return y.view(B, -1, y.shape[-1]) if sp else y


# ------------------------------------------------------------------------------------------------ reference surface
from typing import NamedTuple  # noqa: E402


class CommStats(NamedTuple):
    """One collective as a profiling record (data_pipeline/trainer/distributed/tensor_parallel.py:121)."""
    bytes_sent: int
    bytes_received: int
    latency_ns: int
    operation: str


@dataclass(frozen=True)
class TensorParallelConfig:
    """Switches of a tensor-parallel run (data_pipeline/trainer/distributed/tensor_parallel.py:88-118).  Here
    `async_communication` / `use_ring_allreduce` / `memory_efficient_linear` describe the library path; the fused
    path (`comm="fused"` on the TP context) overlaps transfer and GEMM inside one kernel instead."""
    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    sequence_parallel_enabled: bool = True
    async_communication: bool = True
    gradient_accumulation_fusion: bool = True
    use_ring_allreduce: bool = True
    fp8_communication: bool = False
    memory_efficient_linear: bool = True
    cache_line_aligned: bool = True

    def __post_init__(self):
        if self.tensor_parallel_size < 1 or self.pipeline_parallel_size < 1:
            raise ValueError("tensor / pipeline parallel sizes must be >= 1")
        if self.tensor_parallel_size & (self.tensor_parallel_size - 1):
            raise ValueError("tensor_parallel_size must be a power of two")


def _mgr() -> ProcessGroupManager:
    return ProcessGroupManager.get()


def get_tensor_parallel_rank() -> int:
    return _mgr().tp_rank if _mgr().initialized else 0


def get_tensor_parallel_world_size() -> int:
    return _mgr().tp_size if _mgr().initialized else 1


def get_tensor_parallel_group():
    return _mgr().tp_group


def get_sequence_parallel_rank() -> int:
    return get_tensor_parallel_rank()          # sequence parallelism shares the tensor group


def get_sequence_parallel_world_size() -> int:
    return get_tensor_parallel_world_size()


def is_sequence_parallel_enabled() -> bool:
    cfg = getattr(_mgr(), "config", None)
    return bool(cfg is not None and cfg.sequence_parallel_enabled and _mgr().tp_size > 1)


@contextlib.contextmanager
def tensor_parallel_context(config: TensorParallelConfig):
    """Initialise the process-group registry for `config` (collective when a process group exists) and yield it; on
    exit the registry is forgotten, the torch process groups stay alive with the job."""
    mgr = ProcessGroupManager.get()
    mgr.config = config
    if dist.is_available() and dist.is_initialized():
        mgr.initialize(config.tensor_parallel_size, config.pipeline_parallel_size)
    elif config.tensor_parallel_size * config.pipeline_parallel_size == 1:
        mgr.initialize(1, 1)
    try:
        yield mgr
    finally:
        mgr.destroy()


def compute_parameter_count(model: nn.Module, include_parallel_factor: bool = True) -> dict:
    """Local / trainable / tensor-parallel / replicated parameter counts of a tensor-parallel model and, with
    `include_parallel_factor`, the size of the whole model (parallel parameters x TP size + replicated ones)."""
    tp = get_tensor_parallel_world_size() if include_parallel_factor else 1
    parallel = replicated = 0
    for m in model.modules():
        own = sum(p.numel() for p in m.parameters(recurse=False))
        if isinstance(m, (ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding)) or \
                getattr(m, "_is_tensor_parallel", False):
            size = getattr(getattr(m, "tp", None), "size", None)
            tp = max(tp, size) if include_parallel_factor and size else tp
            parallel += own
        else:
            replicated += own
    local = parallel + replicated
    return {"local_params": local, "local_trainable": sum(p.numel() for p in model.parameters() if p.requires_grad),
            "parallel_params": parallel, "replicated_params": replicated, "tp_world_size": tp,
            "total_params": parallel * tp + replicated}


class FusedColumnParallelLinearWithGELU(nn.Module):
    """Column-parallel projection followed by GELU (the first half of a classic transformer MLP); the activation runs
    on the fused elementwise kernel over the local columns, so no gathered pre-activation exists."""

    def __init__(self, in_features: int, out_features: int, tp: TPContext | None = None, *, bias: bool = True,
                 gather_output: bool = False, sequence_parallel: bool = False, approximate: str = "tanh", dtype=None,
                 device=None, init_method=None):
        super().__init__()
        tp = tp if tp is not None else _mgr().tp_context(sequence_parallel)
        self.linear = ColumnParallelLinear(in_features, out_features, tp, bias=bias, gather_output=False, dtype=dtype,
                                           device=device)
        if init_method is not None:
            with torch.no_grad():
                init_method(self.linear.weight)
        self.gather_output, self.approximate = gather_output, approximate


    @reference_kwargs(input_="x")
    def forward(self, x):
        from ..ops import activation
        y = activation.gelu(self.linear(x), self.approximate)
        return gather_from_tensor_parallel_region(y, self.linear.tp) if self.gather_output else y


class FusedRowParallelLinearWithDropout(nn.Module):
    """Row-parallel projection, reduction over the group, bias, then dropout - in that order, so that the bias is added
    once and every rank draws the dropout mask on the reduced tensor."""

    def __init__(self, in_features: int, out_features: int, tp: TPContext | None = None, *, bias: bool = True,
                 input_is_parallel: bool = True, sequence_parallel: bool = False, dropout_prob: float = 0.0, dtype=None,
                 device=None, init_method=None):
        super().__init__()
        tp = tp if tp is not None else _mgr().tp_context(sequence_parallel)
        self.linear = RowParallelLinear(in_features, out_features, tp, bias=bias, input_is_parallel=input_is_parallel,
                                        dtype=dtype, device=device, init_method=init_method)
        self.dropout_prob = dropout_prob


    @reference_kwargs(input_="x")
    def forward(self, x):
        y = self.linear(x)
        return torch.nn.functional.dropout(y, self.dropout_prob, self.training) if self.dropout_prob > 0 else y


# ---- NCCL settings suggested for tensor parallelism inside one NVLink / NVSwitch node (name from
# data_pipeline/trainer/distributed/tensor_parallel.py; the values are this framework's: peer-to-peer over NVLink,
# in-switch reduction on, asynchronous error handling so that a lost rank ends the collective instead of hanging it)
CACHE_LINE_BYTES, MAX_ASYNC_OPS = 64, 8
NCCL_ENV_VARS = {"NCCL_P2P_LEVEL": "NVL", "NCCL_NVLS_ENABLE": "1", "NCCL_ASYNC_ERROR_HANDLING": "1",
                 "TORCH_NCCL_ASYNC_ERROR_HANDLING": "1", "NCCL_BUFFSIZE": "8388608"}
