"""Chunked fused lm_head + cross-entropy / token log-prob: the [tokens, vocab] logits never exist in full.

For each chunk of tokens: logits = h W^T on the tcgen05 GEMM (bf16), one row kernel computes loss + lse and
overwrites the logits with d(loss)/d(logits), and two more GEMMs turn that into d(hidden) and an fp32
accumulation of d(W).  The gradient is produced during forward (the loss head is the last op), so backward
only scales it.

Reference behaviour: materialised-logit CE kernels data_pipeline/trainer/kernels/triton_kernels.py:122-467,
data_pipeline/trainer/loss/sota_losses.py:140-300,620-744 (chunked CE: mean over non-ignored tokens, count
clamped to >= 1), data_pipeline/trainer/rl_training.py:138-191 (chunked log-softmax for RL).
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib
from .gemm import matmul_nn, matmul_nt, matmul_tn

DEFAULT_CHUNK_TOKENS = 4096


def _ce_rows(logits, labels, loss, lse, ignore_index, label_smoothing, logit_scale, softcap, gscale_ptr, gscale_mul,
             row_gscale, write_grad):
    lib = _lib.load("elementwise")
    rows, V = logits.shape
    rc = lib.ts_cross_entropy(_lib.ptr(logits), _lib.ptr(labels), _lib.ptr(loss), _lib.ptr(lse),
                              ctypes.c_longlong(rows), V, ctypes.c_longlong(logits.stride(0)), ignore_index,
                              ctypes.c_float(label_smoothing), ctypes.c_float(logit_scale), ctypes.c_float(softcap),
                              _lib.ptr(gscale_ptr), ctypes.c_float(gscale_mul), _lib.ptr(row_gscale), int(write_grad),
                              _lib.stream_ptr())
    _lib.check(rc, "ts_cross_entropy")


def cross_entropy_logits(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100,
                         label_smoothing: float = 0.0, logit_scale: float = 1.0, softcap: float = 0.0):
    """Per-row loss and lse for materialised bf16 logits [rows, V] (no gradient). CUDA only."""
    rows = logits.shape[0]
    loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
    _ce_rows(logits, labels, loss, lse, ignore_index, label_smoothing, logit_scale, softcap, None, 1.0, None, False)
    return loss, lse


class _FocalLossFn(torch.autograd.Function):
    """Focal loss -(1 - p)^gamma log p on materialised bf16 logits.  Forward: one pass of the cross-entropy kernel gives
    the per-row ce = -log p.  Backward: d loss / d ce = (1 - p)^gamma + gamma p (1 - p)^(gamma - 1) ce goes in as the
    kernel's per-row gradient scale, and the kernel writes (softmax - onehot) * scale over a copy of the logits."""

    @staticmethod
    def forward(ctx, logits, labels, gamma, ignore_index):
        rows = logits.shape[0]
        loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
        lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
        lg = logits if logits.stride(-1) == 1 and logits.stride(0) % 8 == 0 else logits.contiguous()
        if lg.stride(0) % 8 != 0 or lg.data_ptr() % 16 != 0:
            pad = torch.zeros(rows, _pad_ld(lg.shape[1]), dtype=lg.dtype, device=lg.device)
            pad[:, :lg.shape[1]] = lg
            lg = pad[:, :logits.shape[1]]
        _ce_rows(lg, labels, loss, lse, ignore_index, 0.0, 1.0, 0.0, None, 1.0, None, False)
        p = torch.exp(-loss)
        valid = labels != ignore_index
        focal = torch.where(valid, (1 - p).clamp(min=0) ** gamma * loss, torch.zeros_like(loss))
        ctx.save_for_backward(lg, labels, loss, p, valid)
        ctx.gamma, ctx.ignore_index = gamma, ignore_index
        return focal

    @staticmethod
    def backward(ctx, dfocal):
        lg, labels, ce, p, valid = ctx.saved_tensors
        g = ctx.gamma
        one_m = (1 - p).clamp(min=0)
        dce = one_m ** g + (g * p * one_m ** (g - 1) * ce if g != 0 else 0.0)
        scale = torch.where(valid, dce * dfocal.float(), torch.zeros_like(ce)).contiguous()
        grad = _clone_keep_pitch(lg)
        loss = torch.empty_like(ce)
        lse = torch.empty_like(ce)
        _ce_rows(grad, labels, loss, lse, ctx.ignore_index, 0.0, 1.0, 0.0, None, 1.0, scale, True)
        return grad, None, None, None


class FusedCrossEntropyFunction(torch.autograd.Function):
    """Cross-entropy on materialised bf16 CUDA logits [rows, V] with the row kernel on both sides: forward = one pass
    (per-row loss + lse), backward = one pass writing (softmax - target) * per-row scale over a copy of the logits.
    Returns the per-row losses (0 for ignored rows); reduce them outside."""

    @staticmethod
    def forward(ctx, logits, labels, ignore_index=-100, label_smoothing=0.0):
        rows = logits.shape[0]
        lg = logits if logits.stride(-1) == 1 else logits.contiguous()
        if lg.stride(0) % 8 != 0 or lg.data_ptr() % 16 != 0:
            pad = torch.zeros(rows, _pad_ld(lg.shape[1]), dtype=lg.dtype, device=lg.device)
            pad[:, :lg.shape[1]] = lg
            lg = pad[:, :logits.shape[1]]
        labels = labels.reshape(-1).to(torch.int64)
        loss = torch.empty(rows, dtype=torch.float32, device=lg.device)
        lse = torch.empty(rows, dtype=torch.float32, device=lg.device)
        _ce_rows(lg, labels, loss, lse, ignore_index, label_smoothing, 1.0, 0.0, None, 1.0, None, False)
        ctx.save_for_backward(lg, labels)
        ctx.ignore_index, ctx.label_smoothing = ignore_index, label_smoothing
        return loss

    @staticmethod
    def backward(ctx, dloss):
        lg, labels = ctx.saved_tensors
        grad = _clone_keep_pitch(lg)
        tmp_loss = torch.empty(lg.shape[0], dtype=torch.float32, device=lg.device)
        tmp_lse = torch.empty_like(tmp_loss)
        _ce_rows(grad, labels, tmp_loss, tmp_lse, ctx.ignore_index, ctx.label_smoothing, 1.0, 0.0, None, 1.0,
                 dloss.float().contiguous(), True)
        return grad, None, None, None


def cross_entropy_rows(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100,
                       label_smoothing: float = 0.0) -> torch.Tensor:
    """Differentiable per-row cross-entropy of bf16 CUDA logits on the row kernel."""
    return FusedCrossEntropyFunction.apply(logits, labels, int(ignore_index), float(label_smoothing))


def focal_loss_rows(logits: torch.Tensor, labels: torch.Tensor, gamma: float = 2.0, ignore_index: int = -100):
    """Per-row focal loss of bf16 CUDA logits [rows, V] on the cross-entropy kernel (rows with ignore_index give 0)."""
    return _FocalLossFn.apply(logits, labels, float(gamma), int(ignore_index))


def _clone_keep_pitch(lg: torch.Tensor) -> torch.Tensor:
    """Copy of a [rows, V] view with the SAME row pitch (a plain clone of a padded view packs the rows, and an odd V
    then breaks the kernel's 16-byte row alignment)."""
    out = torch.empty_strided(lg.shape, lg.stride(), dtype=lg.dtype, device=lg.device)
    out.copy_(lg)
    return out


def _pad_ld(V: int) -> int:
    return (V + 7) // 8 * 8


class _FusedLinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, ignore_index, label_smoothing, logit_scale, softcap, chunk_tokens,
                reduction, loss_scale, denominator=None):
        T, H = hidden.shape
        V = weight.shape[0]
        dev = hidden.device
        labels = labels.reshape(-1).to(torch.int64)
        valid = (labels != ignore_index)
        count = valid.sum().clamp(min=1).to(torch.float32)
        if reduction == "mean":
            den = count if denominator is None else denominator.to(torch.float32).clamp(min=1e-6)
            gscale = (1.0 / den).reshape(1)
        else:
            gscale = torch.ones(1, dtype=torch.float32, device=dev)
        need_dh = hidden.requires_grad
        need_dw = weight.requires_grad
        write_grad = need_dh or need_dw
        dh = torch.empty_like(hidden) if need_dh else None
        main_grad = getattr(weight, "main_grad", None) if need_dw else None
        dw = None
        if need_dw:
            if main_grad is not None:
                dw = main_grad.view(V, H)
                dw_acc = bool(getattr(weight, "grad_added", False))
                weight.grad_added = True
            else:
                dw = torch.empty(V, H, dtype=torch.float32, device=dev)
                dw_acc = False
        ld = _pad_ld(V)
        chunk = min(chunk_tokens, T)
        buf = torch.empty(chunk, ld, dtype=torch.bfloat16, device=dev)
        loss_rows = torch.empty(T, dtype=torch.float32, device=dev)
        for s in range(0, T, chunk):
            e = min(s + chunk, T)
            n = e - s
            logits = buf[:n, :V]
            matmul_nt(hidden[s:e], weight, out=logits)
            _ce_rows(logits, labels[s:e], loss_rows[s:e], None, ignore_index, label_smoothing, logit_scale, softcap,
                     gscale, loss_scale, None, write_grad)
            if need_dh:
                matmul_nn(logits, weight, out=dh[s:e])
            if need_dw:
                matmul_tn(logits, hidden[s:e], out=dw, accumulate=(dw_acc or s > 0))
        total = loss_rows.sum()
        loss = total * gscale[0] if reduction == "mean" else total
        ctx.save_for_backward(dh, None if main_grad is not None else dw)
        ctx.direct = main_grad is not None
        ctx.w_dtype = weight.dtype
        ctx.mark_non_differentiable(count)
        return loss * loss_scale, count

    @staticmethod
    def backward(ctx, g, _gcount):
        dh, dw = ctx.saved_tensors
        gh = None if dh is None else dh * g.to(dh.dtype)
        gw = None
        if dw is not None:
            gw = (dw * g).to(ctx.w_dtype)
        return gh, gw, None, None, None, None, None, None, None, None, None


def fused_linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                               ignore_index: int = -100, label_smoothing: float = 0.0, logit_scale: float = 1.0,
                               softcap: float = 0.0, chunk_tokens: int = DEFAULT_CHUNK_TOKENS,
                               reduction: str = "mean", loss_scale: float = 1.0,
                               denominator: torch.Tensor | None = None):
    """loss (and valid-token count) of CE(hidden @ weight.T, labels) without materialising the logits.

    `labels` must already be aligned with `hidden` rows (the causal shift is the caller's job).
    `loss_scale` (e.g. 1/grad-accumulation) is folded into both the returned loss and the gradients.
    `denominator` (a one-element device tensor): with reduction "mean", divide the summed loss by it instead of by
    this call's own count of valid labels - a rank that holds a slice of a longer sequence passes its share of the
    global count, and nothing is read back to the host.
    When `weight.main_grad` exists the weight gradient is accumulated straight into it.
    """
    h2 = hidden.reshape(-1, hidden.shape[-1])
    if h2.is_cuda and h2.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
        if not h2.is_contiguous():
            h2 = h2.contiguous()
        return _FusedLinearCE.apply(h2, weight, labels, ignore_index, label_smoothing, logit_scale, softcap,
                                    chunk_tokens, reduction, loss_scale, denominator)
    return linear_cross_entropy_reference(h2, weight, labels, ignore_index, label_smoothing, logit_scale, softcap,
                                          reduction, loss_scale, denominator)


def linear_cross_entropy_reference(hidden, weight, labels, ignore_index=-100, label_smoothing=0.0, logit_scale=1.0,
                                   softcap=0.0, reduction="mean", loss_scale=1.0, denominator=None):
    """Plain PyTorch fp32 math with the same semantics (CPU path and test oracle)."""
    logits = (hidden.float() @ weight.float().t()) * logit_scale
    if softcap > 0:
        logits = softcap * torch.tanh(logits / softcap)
    labels = labels.reshape(-1)
    count = (labels != ignore_index).sum().clamp(min=1).float()
    loss = F.cross_entropy(logits, labels, ignore_index=ignore_index, label_smoothing=label_smoothing,
                           reduction="sum")
    if reduction == "mean":
        loss = loss / (count if denominator is None else denominator.to(loss.dtype).clamp(min=1e-6).reshape(()))
    return loss * loss_scale, count


class _FusedLinearLogProb(torch.autograd.Function):
    """Per-token log p(label) from hidden states; logits recomputed chunk by chunk in backward."""

    @staticmethod
    def forward(ctx, hidden, weight, labels, ignore_index, chunk_tokens):
        T, H = hidden.shape
        V = weight.shape[0]
        lib = _lib.load("elementwise")
        labels = labels.reshape(-1).to(torch.int64)
        chunk = min(chunk_tokens, T)
        buf = torch.empty(chunk, _pad_ld(V), dtype=torch.bfloat16, device=hidden.device)
        logp = torch.empty(T, dtype=torch.float32, device=hidden.device)
        for s in range(0, T, chunk):
            e = min(s + chunk, T)
            logits = buf[: e - s, :V]
            matmul_nt(hidden[s:e], weight, out=logits)
            rc = lib.ts_token_logprob(_lib.ptr(logits), _lib.ptr(labels[s:e]), _lib.ptr(logp[s:e]), None,
                                      ctypes.c_longlong(e - s), V, ctypes.c_longlong(logits.stride(0)), ignore_index,
                                      _lib.stream_ptr())
            _lib.check(rc, "ts_token_logprob")
        ctx.save_for_backward(hidden, weight, labels)
        ctx.ignore_index = ignore_index
        ctx.chunk = chunk
        return logp

    @staticmethod
    def backward(ctx, g):
        hidden, weight, labels = ctx.saved_tensors
        T, H = hidden.shape
        V = weight.shape[0]
        dev = hidden.device
        need_dw = ctx.needs_input_grad[1]
        dh = torch.empty_like(hidden)
        main_grad = getattr(weight, "main_grad", None) if need_dw else None
        dw = None
        acc0 = False
        if need_dw:
            if main_grad is not None:
                dw = main_grad.view(V, H)
                acc0 = bool(getattr(weight, "grad_added", False))
                weight.grad_added = True
            else:
                dw = torch.empty(V, H, dtype=torch.float32, device=dev)
        buf = torch.empty(ctx.chunk, _pad_ld(V), dtype=torch.bfloat16, device=dev)
        scratch = torch.empty(ctx.chunk, dtype=torch.float32, device=dev)
        neg_g = (-g.float()).contiguous()
        for s in range(0, T, ctx.chunk):
            e = min(s + ctx.chunk, T)
            logits = buf[: e - s, :V]
            matmul_nt(hidden[s:e], weight, out=logits)
            # (softmax - onehot) * (-g)  ==  g * d logp / d logits
            _ce_rows(logits, labels[s:e], scratch[: e - s], None, ctx.ignore_index, 0.0, 1.0, 0.0, None, 1.0,
                     neg_g[s:e], True)
            matmul_nn(logits, weight, out=dh[s:e])
            if need_dw:
                matmul_tn(logits, hidden[s:e], out=dw, accumulate=(acc0 or s > 0))
        gw = None
        if need_dw and main_grad is None:
            gw = dw.to(weight.dtype)
        return dh, gw, None, None, None


def fused_linear_token_logprobs(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                                ignore_index: int = -100, chunk_tokens: int = DEFAULT_CHUNK_TOKENS) -> torch.Tensor:
    """log p(labels[t] | hidden[t]) per token (0 where ignored), shape = labels.shape."""
    h2 = hidden.reshape(-1, hidden.shape[-1])
    if h2.is_cuda and h2.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
        if not h2.is_contiguous():
            h2 = h2.contiguous()
        return _FusedLinearLogProb.apply(h2, weight, labels, ignore_index, chunk_tokens).view(labels.shape)
    logits = h2.float() @ weight.float().t()
    lab = labels.reshape(-1)
    lp = torch.log_softmax(logits, dim=-1).gather(1, lab.clamp(min=0).unsqueeze(1)).squeeze(1)
    return torch.where(lab == ignore_index, torch.zeros_like(lp), lp).view(labels.shape)
