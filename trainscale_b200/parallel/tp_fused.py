"""Autograd wrappers of the fused tensor-parallel GEMMs (csrc/tp_gemm.cu).

`all_gather_linear`  y[M, N_local] = all_gather_rows(x_shard) @ W_local^T   - the gather runs inside the GEMM
`linear_reduce`      y_shard[M/W, N] = reduce_scatter_rows(x @ W_local^T)    - the reduction runs in the epilogue
Their backward passes are each other's fused form (dgrad of a gathered input is a GEMM -> reduce-scatter, dgrad of
a reduce-scattered output is an all-gather -> GEMM), and the weight gradients reuse the gathered operand.
"""
from __future__ import annotations

import os

import ctypes

import torch

from ..ops import _lib
from ..ops.gemm import matmul_tn

_ll, _u = ctypes.c_longlong, ctypes.c_uint
CALLS = {"gather_gemm": 0, "gemm_reduce": 0}     # launches of the fused kernels (tests check that they ran)


class _Buffers:
    """Symmetric staging / accumulation buffers and flag words, cached per shape on the heap object."""

    def __init__(self, heap):
        self.heap = heap
        self.cache: dict = {}

    def get(self, kind: str, rows: int, cols: int, n_mblocks: int):
        key = (kind, rows, cols)
        b = self.cache.get(key)
        if b is None:
            dt = torch.float32 if kind == "acc" else torch.bfloat16     # "src", "acc16": bf16
            t = self.heap.alloc(rows * cols, dt).view(rows, cols)
            buf, _ = self.heap.lookup(t)
            flags = torch.zeros(2 + n_mblocks, dtype=torch.int32, device=t.device)
            b = {"t": t, "buf": buf, "flags": flags, "epoch": 0}
            self.cache[key] = b
        b["epoch"] += 1
        return b


def _buffers(tp) -> _Buffers:
    if not hasattr(tp.heap, "_tp_buffers"):
        tp.heap._tp_buffers = _Buffers(tp.heap)
    return tp.heap._tp_buffers


def _launch(mode, tp, b, A, B, C, a_full, M, N, K, lda, ldb, ldc, b_mn):
    lib = _lib.load("tp_gemm")
    buf = b["buf"]
    src = buf.peer_ptrs if mode == 1 else None
    dst = buf.peer_ptrs if mode in (2, 3, 4) else None
    rc = lib.ts_tp_gemm(mode, _lib.ptr(A), _lib.ptr(B), _lib.ptr(C), _lib.ptr(a_full), M, N, K, lda, ldb, ldc, int(b_mn),
                        src, dst, buf.pad_ptrs, tp.rank, tp.size, _lib.ptr(b["flags"]), _u(b["epoch"]), _u(0),
                        _ll(tp.heap.wait_cycles), _lib.ptr(tp.heap.status), _lib.stream_ptr())
    _lib.check(rc, "ts_tp_gemm")


def _gather_gemm(x_shard, w, tp, b_mn):
    """(y [M, N], a_full [M, K]); w is [N, K] (b_mn False) or [K, N] (b_mn True)."""
    CALLS["gather_gemm"] += 1
    Ms, K = x_shard.shape
    M = Ms * tp.size
    N = w.shape[1] if b_mn else w.shape[0]
    b = _buffers(tp).get("src", Ms, K, M // 128)
    b["t"].copy_(x_shard)
    a_full = torch.empty(M, K, dtype=x_shard.dtype, device=x_shard.device)
    a_full[tp.rank * Ms:(tp.rank + 1) * Ms].copy_(x_shard)
    y = torch.empty(M, N, dtype=x_shard.dtype, device=x_shard.device)
    _launch(1, tp, b, None, w, y, a_full, M, N, K, K, w.stride(0), N, b_mn)
    return y, a_full


# GEMM -> reduce-scatter accumulates the ranks' partial sums either in fp32 buffers (16-byte reds of 4 values, then a
# cast pass) or directly in the bf16 output format (every addition rounds to bf16, as a bf16 ring reduce-scatter does).
# Measured at W=2, M=8192, N=K=4096: bulk tensor reductions 0.221 ms, packed-bf16 reds 0.282 ms, plain pushes into
# per-source slots 0.350 ms, fp32 reds 0.439 ms (cuBLAS + NCCL reduce-scatter: 0.279 ms).
ACC_BF16 = os.environ.get("TS_TP_ACC_FP32", "0") != "1"
# "push": no atomics at all - every rank stores its partial sums of a peer's rows into its own slot of that peer's
# staging buffer with plain 16-byte stores (NVLink carries them far better than 16-byte reductions) and the owner adds
# the W slots in fp32 after the kernel.  "red": reductions into one shared buffer (ACC_BF16 picks the format).
# "tma": shared bf16 buffer, output slices added by bulk tensor reductions (`cp.reduce.async.bulk.tensor`).
REDUCE_MODE = os.environ.get("TS_TP_REDUCE", "tma")


def _gemm_reduce(x, w, tp, b_mn):
    """y_shard [M/W, N] (bf16) = reduce_scatter(x @ w^T)."""
    CALLS["gemm_reduce"] += 1
    M, K = x.shape
    N = w.shape[1] if b_mn else w.shape[0]
    Ms = M // tp.size
    if REDUCE_MODE == "tma" and x.dtype == torch.bfloat16 and Ms % 256 == 0 and N >= 256 and N % 8 == 0:
        # 128 x 64 output slices are added into the owner's bf16 buffer by bulk tensor reductions of the copy engine
        b = _buffers(tp).get("acc16", Ms, N, M // 128)
        lib = _lib.load("tp_gemm")
        buf = b["buf"]
        rc = lib.ts_tp_gemm(5, _lib.ptr(x), _lib.ptr(w), None, None, M, N, K, x.stride(0), w.stride(0), N, int(b_mn),
                            None, buf.peer_ptrs, buf.pad_ptrs, tp.rank, tp.size, _lib.ptr(b["flags"]), _u(b["epoch"]),
                            _u(0), _ll(tp.heap.wait_cycles), _lib.ptr(tp.heap.status), _lib.stream_ptr())
        if rc != -13:
            _lib.check(rc, "ts_tp_gemm")
            out = b["t"].clone()
            b["t"].zero_()        # re-armed before the next call's entry barrier tells the peers so
            return out
    if REDUCE_MODE == "push" and x.dtype == torch.bfloat16:
        # per-source staging slots on the owner, plain stores only; the slots are summed after the kernel
        b = _buffers(tp).get("push", tp.size * Ms, N, M // 128)
        out = torch.empty(Ms, N, dtype=x.dtype, device=x.device)     # receives this rank's own partial sums
        _launch(4, tp, b, x, w, out, None, M, N, K, x.stride(0), w.stride(0), N, b_mn)
        lib = _lib.load("tp_gemm")
        rc = lib.ts_sum_slots(_lib.ptr(out), _lib.ptr(b["t"]), _lib.ptr(out), _ll(Ms * N), tp.size, tp.rank,
                              _lib.stream_ptr())
        _lib.check(rc, "ts_sum_slots")
        return out
    if ACC_BF16 and x.dtype == torch.bfloat16:
        b = _buffers(tp).get("acc16", Ms, N, M // 128)
        out = torch.empty(Ms, N, dtype=x.dtype, device=x.device)     # receives this rank's own partial sums
        _launch(3, tp, b, x, w, out, None, M, N, K, x.stride(0), w.stride(0), N, b_mn)
        lib = _lib.load("tp_gemm")
        # out += what the peers reduced into the shared buffer; the buffer is re-armed (zeroed) in the same pass,
        # before the next call's entry barrier tells the peers so
        rc = lib.ts_add_and_clear(_lib.ptr(out), _lib.ptr(b["t"]), _lib.ptr(out), _ll(Ms * N), _lib.stream_ptr())
        _lib.check(rc, "ts_add_and_clear")
        return out
    b = _buffers(tp).get("acc", Ms, N, M // 128)
    _launch(2, tp, b, x, w, None, None, M, N, K, x.stride(0), w.stride(0), N, b_mn)
    out = torch.empty(Ms, N, dtype=x.dtype, device=x.device)
    lib = _lib.load("tp_gemm")
    rc = lib.ts_cast_and_clear(_lib.ptr(b["t"]), _lib.ptr(out), _ll(Ms * N), _lib.stream_ptr())
    _lib.check(rc, "ts_cast_and_clear")
    return out


class _AllGatherLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, w, tp):
        y, a_full = _gather_gemm(x_shard.contiguous(), w, tp, False)
        ctx.save_for_backward(a_full, w)
        ctx.tp = tp
        return y

    @staticmethod
    def backward(ctx, dy):
        a_full, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = _gemm_reduce(dy, w, ctx.tp, True)           # [M, N] . [N, K] -> reduce-scatter rows
        main_grad = getattr(w, "main_grad", None)
        if main_grad is not None:
            matmul_tn(dy, a_full, out=main_grad.view(w.shape), accumulate=getattr(w, "grad_added", False))
            w.grad_added = True
            dw = None
        else:
            dw = matmul_tn(dy, a_full)
        return dx, dw, None


class _LinearReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, tp):
        x = x.contiguous()
        ctx.save_for_backward(x, w)
        ctx.tp = tp
        return _gemm_reduce(x, w, tp, False)

    @staticmethod
    def backward(ctx, dy_shard):
        x, w = ctx.saved_tensors
        dx, dy_full = _gather_gemm(dy_shard.contiguous(), w, ctx.tp, True)   # gather(dy)[M, N] . W[N, K]
        main_grad = getattr(w, "main_grad", None)
        if main_grad is not None:
            matmul_tn(dy_full, x, out=main_grad.view(w.shape), accumulate=getattr(w, "grad_added", False))
            w.grad_added = True
            dw = None
        else:
            dw = matmul_tn(dy_full, x)
        return dx, dw, None


def all_gather_linear(x_shard: torch.Tensor, w: torch.Tensor, tp) -> torch.Tensor:
    shp = x_shard.shape
    y = _AllGatherLinear.apply(x_shard.reshape(-1, shp[-1]), w, tp)
    return y


def linear_reduce(x: torch.Tensor, w: torch.Tensor, tp, scatter: bool = True) -> torch.Tensor:
    y = _LinearReduce.apply(x.reshape(-1, x.shape[-1]), w, tp)
    if not scatter:
        from .tp import _all_gather_dim
        y = _all_gather_dim(y, tp, 0)
    return y


def gather_weight_linear(x: torch.Tensor, w_shard: torch.Tensor, tp) -> torch.Tensor:
    """y[M, N] = x[M, K] @ gather_rows(w_shard over the group)[N, K]^T with the weight all-gather running inside the
    GEMM kernel (the parameter gather of a ZeRO-3 / FSDP forward): peers' row blocks are pulled over NVLink by copier
    warps while the tensor cores already work on the tiles of this rank's own rows.  Forward only.
    Falls back to all_gather + GEMM for shapes the paired-CTA kernel does not take."""
    import torch.distributed as dist
    from ..ops.gemm import matmul_nt
    M, K = x.shape
    Ns = w_shard.shape[0]
    N = Ns * tp.size
    lib = _lib.load("tp_gemm")
    if x.is_cuda and x.dtype == torch.bfloat16 and Ns % 256 == 0 and M % 256 == 0 and K % 32 == 0:
        b = _buffers(tp).get("wsrc", Ns, K, N // 128)
        b["t"].copy_(w_shard)
        w_full = torch.empty(N, K, dtype=x.dtype, device=x.device)
        w_full[tp.rank * Ns:(tp.rank + 1) * Ns].copy_(w_shard)
        y = torch.empty(M, N, dtype=x.dtype, device=x.device)
        buf = b["buf"]
        xc = x if x.is_contiguous() else x.contiguous()
        rc = lib.ts_weight_gather_gemm(_lib.ptr(xc), _lib.ptr(y), _lib.ptr(w_full), M, N, K, xc.stride(0), N,
                                       buf.peer_ptrs, buf.pad_ptrs, tp.rank, tp.size, _lib.ptr(b["flags"]),
                                       _u(b["epoch"]), _u(0), _ll(tp.heap.wait_cycles), _lib.ptr(tp.heap.status),
                                       _lib.stream_ptr())
        if rc != -13:
            _lib.check(rc, "ts_weight_gather_gemm")
            return y
    full = torch.empty(N, K, dtype=w_shard.dtype, device=w_shard.device)
    dist.all_gather_into_tensor(full, w_shard.contiguous(), group=tp.group)
    return matmul_nt(x, full)
