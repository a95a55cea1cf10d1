"""Kernel micro-benchmarks: `python -m trainscale_b200.benchmark_suite [--only NAME] [--small] [--json out.json]`.

Same cases as data_pipeline/trainer/kernels/benchmark_suite.py:97-340 (RMSNorm, GELU/SwiGLU, RoPE, cross-entropy,
flash attention) plus the GEMM and optimizer kernels, each timed with CUDA events after warm-up (L2 flushed between
iterations) against a PyTorch baseline, and reported as achieved bandwidth / FLOP rate and as a fraction of the
measured peaks (MEASURED_PEAKS.json next to the repository root when present).
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path
from typing import NamedTuple

import torch
import torch.nn.functional as F

ROOT = Path(__file__).resolve().parent.parent


def peaks() -> dict:
    try:
        return json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "fallback": True}


class Timer:
    def __init__(self, flush_mb: int = 256):
        self.flush = torch.empty(flush_mb * 2 ** 20, dtype=torch.int8, device="cuda")

    def __call__(self, fn, iters: int = 10, warmup: int = 3, graph: bool = False) -> float:
        """Mean device time of `fn` in ms.  `graph`: replay `fn` from a CUDA graph, so that the time between the two
        events is the kernels' own (for kernels of a few tens of microseconds the host-side launch path is longer
        than the kernel, and an event pair around a plain call measures the host)."""
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        run = fn
        if graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            run = g.replay
            run()
            torch.cuda.synchronize()
        total = 0.0
        for _ in range(iters):
            self.flush.zero_()           # evict L2 (126 MB)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            run()
            b.record()
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        return total / iters


def bench_rmsnorm(t, small, shapes=None):
    from .ops import norm
    out = []
    shapes = shapes or ([(4, 2048, 4096)] if small else [(4, 2048, 4096), (4, 4096, 8192), (32, 2048, 4096), (32, 4096, 8192)])
    for B, S, D in shapes:
        x = torch.randn(B * S, D, device="cuda", dtype=torch.bfloat16)
        w = torch.ones(D, device="cuda", dtype=torch.bfloat16)
        ms = t(lambda: norm.rmsnorm(x, w), graph=True)
        base = t(lambda: F.rms_norm(x, (D,), w, 1e-5), graph=True)
        out.append(dict(name=f"rmsnorm B={B},S={S},D={D}", ms=ms, baseline_ms=base, gbs=2 * x.numel() * 2 / ms / 1e6))
    return out


def bench_swiglu(t, small, sizes=None):
    from .ops import activation
    out = []
    for rows, I in (sizes or ([(2048, 11008)] if small else [(2048, 11008), (8192, 14336)])):
        gu = torch.randn(rows, 2 * I, device="cuda", dtype=torch.bfloat16)
        ms = t(lambda: activation.glu(gu), graph=True)
        base = t(lambda: F.silu(gu[:, :I]) * gu[:, I:], graph=True)
        out.append(dict(name=f"swiglu rows={rows},I={I}", ms=ms, baseline_ms=base, gbs=3 * rows * I * 2 / ms / 1e6))
    return out


def bench_rope(t, small, seq_lens=None, dim: int = 128):
    from .ops import rope
    out = []
    for S in (seq_lens or ([4096] if small else [4096, 8192, 16384])):
        Hq, Hkv, D = 32, 8, dim
        cos, sin = rope.rope_tables(S, D, 500000.0, "cuda")
        qkv = torch.randn(1, S, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
        # the decoder's form: q|k rotated where the projection wrote them (no copy)
        ms = t(lambda: rope.apply_rope_qkv(qkv, Hq + Hkv, D, cos, sin, inplace=True), graph=True)
        base = t(lambda: qkv.clone(), graph=True)
        # bytes: the q and k heads are read and written in place (v is not touched), plus the cos / sin rows
        out.append(dict(name=f"rope S={S}", ms=ms, baseline_ms=base,
                        gbs=(2 * S * (Hq + Hkv) * D * 2 + 2 * S * D * 2) / ms / 1e6))
    return out


def bench_cross_entropy(t, small, vocab_size: int = 128256, token_counts=None):
    from .ops import cross_entropy as ce
    out = []
    V = vocab_size
    for T in (token_counts or ([4096] if small else [4096, 16384])):
        logits = torch.randn(T, V, device="cuda", dtype=torch.bfloat16)
        labels = torch.randint(0, V, (T,), device="cuda")
        ms = t(lambda: ce.cross_entropy_logits(logits, labels), iters=5)
        base = t(lambda: F.cross_entropy(logits.float(), labels), iters=5)
        out.append(dict(name=f"cross_entropy T={T},V={V}", ms=ms, baseline_ms=base, gbs=logits.numel() * 2 / ms / 1e6))
    return out


def bench_gemm(t, small):
    from .ops import gemm
    out = []
    shapes = [(4096, 4096, 4096)] if small else [(8192, 4096, 4096), (8192, 6144, 4096), (8192, 28672, 4096),
                                                 (8192, 4096, 14336), (8192, 128256, 4096)]
    for M, N, K in shapes:
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms = t(lambda: gemm.matmul_nt(a, b, out=c))
        base = t(lambda: torch.matmul(a, b.t(), out=c))
        out.append(dict(name=f"gemm {M}x{N}x{K}", ms=ms, baseline_ms=base, tflops=2 * M * N * K / ms / 1e9))
    return out


def bench_attention(t, small, seq_lens=None, head_dim: int = 128):
    from .ops import flash
    out = []
    for S in (seq_lens or ([2048] if small else [4096, 8192, 16384])):
        Hq, Hkv, D = 32, 8, head_dim
        qkv = torch.randn(1, S, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        ms = t(lambda: flash.flash_forward_only(qkv.detach(), Hq, Hkv, D, True))
        q, k, v = [x.transpose(1, 2) for x in qkv.detach().view(1, S, Hq + 2 * Hkv, D).split((Hq, Hkv, Hkv), 2)]
        base = t(lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True))
        fl = 4 * S * S * D * Hq / 2
        out.append(dict(name=f"flash_fwd S={S}", ms=ms, baseline_ms=base, tflops=fl / ms / 1e9))
        o = flash.flash_attention_qkv(qkv, Hq, Hkv, D, True)
        g = torch.randn_like(o)
        ms = t(lambda: o.backward(g, retain_graph=True), iters=5)
        out.append(dict(name=f"flash_bwd S={S}", ms=ms, baseline_ms=None, tflops=2.5 * fl / ms / 1e9))
    return out


def bench_adamw(t, small):
    from .ops import optim
    n = (1 << 26) if small else (1 << 28)
    p, m, v = (torch.zeros(n, device="cuda") for _ in range(3))
    g = torch.randn(n, device="cuda").to(torch.bfloat16)
    low = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ms = t(lambda: optim.adamw_flat_(p, m, v, g, low, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=3),
           iters=5)
    return [dict(name=f"adamw_flat n={n}", ms=ms, baseline_ms=None, gbs=n * 28 / ms / 1e6)]


def bench_fp8(t, small, shapes=None):
    from .ops import fp8
    out = []
    for M, N, K in (shapes or ([(4096, 4096, 4096)] if small else [(8192, 4096, 4096), (8192, 28672, 4096), (8192, 4096, 14336)])):
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = (torch.randn(N, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
        xq, xs = fp8.quant_act(x)
        wq, ws = fp8.quant_block(w)
        ms = t(lambda: fp8.gemm_fp8(xq, xs, wq, ws, N))
        out.append(dict(name=f"fp8_gemm {M}x{N}x{K}", ms=ms, baseline_ms=None, tflops=2 * M * N * K / ms / 1e9))
        ms = t(lambda: fp8.quant_act(x), graph=True)
        out.append(dict(name=f"fp8_quant_act {M}x{K}", ms=ms, baseline_ms=None, gbs=M * K * 3 / ms / 1e6))
    return out


def bench_fp8_rowwise(t, small):
    """Row-scaled fp8 GEMM (forward / dgrad / wgrad layouts) against this framework's bf16 GEMM on the same shapes,
    the quantisation kernels, and the whole fp8 linear layer (quantise + 3 GEMMs) against the bf16 one."""
    from .ops import fp8, gemm
    out = []
    shapes = [(4096, 4096, 4096)] if small else [(8192, 8192, 8192), (8192, 28672, 8192), (8192, 4096, 14336),
                                                 (8192, 28672, 4096)]
    for M, N, K in shapes:
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = (torch.randn(N, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
        dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
        y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        xq, sx = fp8.quant_rowwise(x)
        wq, sw = fp8.quant_rowwise(w)
        ms = t(lambda: fp8.gemm_rowwise(xq, sx, wq, sw, M, N, K, out=y))
        base = t(lambda: gemm.matmul_nt(x, w, out=y))
        out.append(dict(name=f"fp8_rowwise_gemm fwd {M}x{N}x{K}", ms=ms, baseline_ms=base,
                        tflops=2 * M * N * K / ms / 1e9))
        dq, sd = fp8.quant_rowwise(dy)
        wc, swc = fp8.quant_colwise(w)
        dx = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
        ms = t(lambda: fp8.gemm_rowwise(dq, sd, wc, swc, M, K, N, b_mn=True, out=dx))
        base = t(lambda: gemm.matmul_nn(dy, w, out=dx))
        out.append(dict(name=f"fp8_rowwise_gemm dgrad {M}x{K}x{N}", ms=ms, baseline_ms=base,
                        tflops=2 * M * N * K / ms / 1e9))
        dc, sdc = fp8.quant_colwise(dy)
        xc, sxc = fp8.quant_colwise(x)
        dw = torch.empty(N, K, device="cuda", dtype=torch.bfloat16)
        ms = t(lambda: fp8.gemm_rowwise(dc, sdc, xc, sxc, N, K, M, a_mn=True, b_mn=True, out=dw))
        base = t(lambda: gemm.matmul_tn(dy, x, out=dw))
        out.append(dict(name=f"fp8_rowwise_gemm wgrad {N}x{K}x{M}", ms=ms, baseline_ms=base,
                        tflops=2 * M * N * K / ms / 1e9))
        ms = t(lambda: fp8.quant_rowwise(dy), graph=True)
        out.append(dict(name=f"fp8_quant_rowwise {M}x{N}", ms=ms, baseline_ms=None, gbs=M * N * 3 / ms / 1e6))
        ms = t(lambda: fp8.quant_colwise(dy), graph=True)
        out.append(dict(name=f"fp8_quant_colwise {M}x{N}", ms=ms, baseline_ms=None, gbs=M * N * 5 / ms / 1e6))
        xg, wg = x.clone().requires_grad_(True), w.clone().requires_grad_(True)

        def layer(fn):
            xg.grad = wg.grad = None
            fn(xg, wg).backward(dy)
        ms = t(lambda: layer(lambda a, b: fp8.fp8_linear(a, b, recipe="rowwise")))
        base = t(lambda: layer(gemm.linear))
        out.append(dict(name=f"fp8_rowwise_linear fwd+bwd {M}x{N}x{K}", ms=ms, baseline_ms=base,
                        tflops=6 * M * N * K / ms / 1e9))
    return out


def bench_comm(t, small):
    """The fused collective kernels of csrc/comm.cu on symmetric memory.  Under torchrun (one rank per GPU) the peer
    traffic crosses NVLink and the rates are per-GPU NVLink rates; in a single process the only "peer" is this GPU, so
    the same kernels run against local HBM (what an ncu capture of one GPU can show).  Bytes counted: reduce-scatter
    reads W shards of the gradient dtype and writes one fp32 shard; AdamW + broadcast reads 4 fp32 streams, writes 3 and
    stores W bf16 copies; the gather moves W - 1 remote shards (W = 1: one local copy)."""
    import torch.distributed as dist

    from .parallel import fused_comm
    from .parallel.symm import SymmetricHeap
    own = False
    if not dist.is_initialized():
        import os
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29555")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", torch.cuda.current_device()))
        own = True
    W, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    heap = SymmetricHeap.try_create(None, dev)
    out = []
    if heap is None:
        return out
    n = (1 << 26 if small else 1 << 28) // W * W            # bf16 elements of one layer-sized gradient buffer
    shard = n // W
    grad = heap.alloc(n, torch.bfloat16)
    grad.normal_()
    param = heap.alloc(n, torch.bfloat16)
    red = torch.empty(shard, dtype=torch.float32, device=dev)
    ss, nf = torch.zeros(1, device=dev), torch.zeros(1, device=dev)
    master, m, v = (torch.zeros(shard, dtype=torch.float32, device=dev) for _ in range(3))
    full = torch.empty(n, dtype=torch.bfloat16, device=dev)
    store = heap.alloc(shard, torch.bfloat16)

    def timed(fn):
        ms = t(fn, iters=5)
        x = torch.tensor([ms], device=dev)
        if W > 1:
            dist.all_reduce(x, op=dist.ReduceOp.MAX)       # multi-GPU numbers are the maximum over ranks
        return float(x)
    ms = timed(lambda: fused_comm.reduce_scatter_fp32(heap, grad, red, rank * shard, 1.0 / W, ss, nf))
    out.append(dict(name=f"symm_reduce_scatter W={W} n={n}", ms=ms, baseline_ms=None,
                    gbs=(W * shard * 2 + shard * 4) / ms / 1e6, nvlink_gbs=((W - 1) * shard * 2) / ms / 1e6))
    ms = timed(lambda: fused_comm.adamw_bcast(heap, param, rank * shard, master, m, v, red, lr=1e-4, beta1=0.9,
                                              beta2=0.95, eps=1e-8, weight_decay=0.0, step=1))
    out.append(dict(name=f"symm_adamw_bcast W={W} n={n}", ms=ms, baseline_ms=None,
                    gbs=(shard * 4 * 7 + W * shard * 2) / ms / 1e6, nvlink_gbs=((W - 1) * shard * 2) / ms / 1e6))
    for eng in ("ce", "sm"):
        ms = timed(lambda: fused_comm.gather_pull(heap, store, full, engine=eng))
        out.append(dict(name=f"gather_pull[{eng}] W={W} n={n}", ms=ms, baseline_ms=None,
                        gbs=2 * n * 2 / ms / 1e6, nvlink_gbs=((W - 1) * shard * 2) / ms / 1e6))
    if W > 1:
        ms = timed(lambda: dist.reduce_scatter_tensor(full[:shard], grad, op=dist.ReduceOp.AVG))
        out.append(dict(name=f"nccl reduce_scatter W={W} n={n}", ms=ms, baseline_ms=None,
                        gbs=(W * shard * 2 + shard * 2) / ms / 1e6, nvlink_gbs=((W - 1) * shard * 2) / ms / 1e6))
        ms = timed(lambda: dist.all_gather_into_tensor(full, store))
        out.append(dict(name=f"nccl all_gather W={W} n={n}", ms=ms, baseline_ms=None, gbs=2 * n * 2 / ms / 1e6,
                        nvlink_gbs=((W - 1) * shard * 2) / ms / 1e6))
    torch.cuda.synchronize()
    heap.check_status()
    if own:
        dist.destroy_process_group()
    return out


def bench_ep(t, small):
    """One expert-parallel mixture-of-experts block, forward + backward, per rank: tokens dispatched and combined by the
    peer-memory kernels of csrc/ep_comm.cu (`parallel/ep_peer.py`: no host synchronisation, grouped GEMMs) against the
    same block on the library all-to-all (`baseline`: host-side split sizes, one GEMM pair per expert).  Run under
    torchrun with one rank per GPU; in a single process the "peers" are this GPU.  TFLOP/s counts the three expert
    GEMMs of the rank's own tokens, forward + backward (3x forward)."""
    import copy

    import torch.distributed as dist

    from .models.llama import LlamaMoEMLP, preset_config
    from .parallel.ep import ExpertParallelDecoderMoE, make_peer_dispatcher
    own = False
    if not dist.is_initialized():
        import os
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29556")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", torch.cuda.current_device()))
        own = True
    W, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    out = []
    T, H, I, E, k = (2048, 2048, 1024, 8, 2) if small else (8192, 4096, 14336, 8, 2)
    peer = make_peer_dispatcher(dist.group.WORLD, E, dev)
    if peer is None or E % W:
        return out
    cfg = preset_config("moe-tiny", hidden_size=H, intermediate_size=I, num_local_experts=E, num_experts_per_tok=k)
    torch.manual_seed(0)
    with torch.device(dev):
        base = LlamaMoEMLP(cfg).to(torch.bfloat16)
    for p in base.parameters():
        torch.nn.init.normal_(p, std=0.02)
    blocks = {"peer": ExpertParallelDecoderMoE(base, dist.group.WORLD, peer),
              "nccl": ExpertParallelDecoderMoE(base, dist.group.WORLD, None)}
    del base
    gen = torch.Generator(device="cpu").manual_seed(rank)
    x = torch.randn(T, H, generator=gen).to(dev, torch.bfloat16).requires_grad_(True)
    g = torch.randn(T, H, generator=gen).to(dev, torch.bfloat16)

    def step(blk):
        for p in blk.parameters():
            p.grad = None
        x.grad = None
        blk(x).backward(g)

    ms = {}
    for name, blk in blocks.items():
        v = torch.tensor([t(lambda: step(blk), iters=5)], device=dev)
        if W > 1:
            dist.all_reduce(v, op=dist.ReduceOp.MAX)
        ms[name] = float(v)
    flops = 3 * (T * k) * 3 * 2 * H * I
    out.append(dict(name=f"ep moe block fwd+bwd W={W} T={T} H={H} I={I} E={E} k={k}", ms=ms["peer"],
                    baseline_ms=ms["nccl"], tflops=flops / ms["peer"] / 1e9,
                    nvlink_gbs=4 * (T * k) * (W - 1) / W * H * 2 / ms["peer"] / 1e6 if W > 1 else None))
    torch.cuda.synchronize()
    peer.heap.check_status()
    peer.check()
    if own:
        dist.destroy_process_group()
    return out


def bench_moe(t, small):
    from .ops import moe
    out = []
    for T, H, I, E, k in ([(4096, 2048, 1024, 8, 2)] if small else [(8192, 4096, 1792, 8, 2), (8192, 2048, 1024, 64, 6)]):
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        wgu = (torch.randn(E, 2 * I, H, device="cuda") * 0.02).to(torch.bfloat16)
        wd = (torch.randn(E, H, I, device="cuda") * 0.02).to(torch.bfloat16)
        w, ids = torch.softmax(torch.randn(T, E, device="cuda"), -1).topk(k, -1)
        w = w.to(torch.bfloat16)
        ms = t(lambda: moe.moe_ffn(x, ids, w, wgu, wd))
        out.append(dict(name=f"moe_ffn fwd T={T} H={H} I={I} E={E} k={k}", ms=ms, baseline_ms=None,
                        tflops=2 * T * k * H * I * 3 / ms / 1e9))
    return out


def bench_layernorm(t, small):
    from .ops import norm
    out = []
    for rows, H in ([(8192, 4096)] if small else [(8192, 4096), (32768, 4096), (16384, 8192)]):
        x = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16)
        w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
        b = torch.zeros(H, device="cuda", dtype=torch.bfloat16)
        ms = t(lambda: norm.layernorm(x, w, b), graph=True)
        base = t(lambda: F.layer_norm(x, (H,), w, b), graph=True)
        out.append(dict(name=f"layernorm_fwd {rows}x{H}", ms=ms, baseline_ms=base, gbs=rows * H * 4 / ms / 1e6))
    return out


CASES = {"fp8": bench_fp8, "fp8_rowwise": bench_fp8_rowwise, "comm": bench_comm, "ep": bench_ep, "moe": bench_moe, "layernorm": bench_layernorm, "rmsnorm": bench_rmsnorm, "swiglu": bench_swiglu, "rope": bench_rope, "cross_entropy": bench_cross_entropy,
         "gemm": bench_gemm, "attention": bench_attention, "adamw": bench_adamw}


class BenchmarkSuite:
    """Object form of the kernel benchmarks (data_pipeline/trainer/kernels/benchmark_suite.py:97-338 has the same
    `run_*` / `report` surface): each `run_*` times one kernel family with CUDA events (L2 flushed between
    iterations) against the PyTorch op of the same maths and appends rows to `self.results`."""

    def __init__(self, small: bool = False, device: str = "cuda"):
        self.small, self.device = small, device
        self.results: list[dict] = []
        self._timer: Timer | None = None

    def _run(self, fn, **sizes) -> list[dict]:
        if not torch.cuda.is_available():
            return []
        if self._timer is None:
            self._timer = Timer(64 if self.small else 256)
        rows = fn(self._timer, self.small, **{k: v for k, v in sizes.items() if v is not None})
        self.results += rows
        return rows

    # the size arguments are the reference's (data_pipeline/trainer/kernels/benchmark_suite.py:111-300); None keeps this
    # suite's own shapes
    def run_rms_norm(self, batch_sizes=None, seq_lens=None, hidden_dims=None):
        shapes = None
        if batch_sizes or seq_lens or hidden_dims:
            shapes = [(b, s, d) for b in (batch_sizes or [4]) for s in (seq_lens or [2048]) for d in (hidden_dims or [4096])]
        return self._run(bench_rmsnorm, shapes=shapes)

    def run_layer_norm(self):
        return self._run(bench_layernorm)

    def run_fused_gelu(self, sizes=None):
        """`sizes`: (rows, cols) pairs."""
        return self._run(bench_gelu, counts=[r * c for r, c in sizes] if sizes else None)

    def run_swiglu(self, sizes=None):
        """`sizes`: (rows, intermediate size) pairs."""
        return self._run(bench_swiglu, sizes=list(sizes) if sizes else None)

    def run_fp8_quantization(self, sizes=None):
        """`sizes`: (rows, cols) of the activation that is quantised (and multiplied by a cols x cols weight)."""
        return self._run(bench_fp8, shapes=[(r, c, c) for r, c in sizes] if sizes else None)

    def run_rope(self, seq_lens=None, dim: int | None = None):
        return self._run(bench_rope, seq_lens=list(seq_lens) if seq_lens else None, dim=dim)

    def run_flash_attention(self, seq_lens=None, head_dim: int | None = None):
        if head_dim not in (None, 64, 128):
            raise ValueError("the flash kernels cover head dimensions 64 and 128")
        return self._run(bench_attention, seq_lens=list(seq_lens) if seq_lens else None, head_dim=head_dim)

    def run_cross_entropy(self, vocab_size: int | None = None, batch_tokens: int | None = None):
        return self._run(bench_cross_entropy, vocab_size=vocab_size,
                         token_counts=[int(batch_tokens)] if batch_tokens else None)

    def run_gemm(self):
        return self._run(bench_gemm)

    def run_optimizer(self):
        return self._run(bench_adamw)

    def run_moe(self):
        return self._run(bench_moe)

    def run_optimizer_kernels(self):
        return self._run(bench_optimizers)

    def run_all(self):
        for name in ("run_rms_norm", "run_layer_norm", "run_fused_gelu", "run_swiglu", "run_fp8_quantization",
                     "run_rope", "run_flash_attention", "run_cross_entropy", "run_gemm", "run_optimizer", "run_moe"):
            getattr(self, name)()
        return self.results

    def report(self) -> str:
        pk = peaks()
        tag = "of fallback" if pk.get("fallback") else "of measured"
        lines = []
        for r in self.results:
            frac = r["gbs"] / pk["hbm_gbs"] if "gbs" in r else r["tflops"] / pk["bf16_tflops"]
            rate = f"{r['gbs']:.0f} GB/s" if "gbs" in r else f"{r['tflops']:.0f} TFLOPS"
        if r.get("nvlink_gbs"):
            rate += f" ({r['nvlink_gbs']:.0f} GB/s in over NVLink)"
            sp = f"{r['baseline_ms'] / r['ms']:.2f}x" if r.get("baseline_ms") else "-"
            lines.append(f"{r['name']:<40s} {r['ms']:8.3f} ms  {sp:>7s}  {rate:>12s}  {frac:5.2f} {tag}")
        return "\n".join(lines)


def bench_gelu(t, small, counts=None):
    from .ops import activation
    out = []
    for n in (counts or ([1 << 24] if small else [1 << 24, 1 << 27])):
        x = torch.randn(n, device="cuda", dtype=torch.bfloat16)
        ms = t(lambda: activation.gelu(x, "tanh"), graph=True)
        base = t(lambda: F.gelu(x, approximate="tanh"), graph=True)
        out.append(dict(name=f"gelu n={n}", ms=ms, baseline_ms=base, gbs=2 * n * 2 / ms / 1e6))
    return out


CASES["gelu"] = bench_gelu


def bench_optimizers(t, small):
    """Per-tensor optimizer kernels (csrc/optim.cu) against the same optimizer class on its PyTorch-op path.
    GB/s counts the bytes the update must move once (parameter read + write, gradient, state read + write)."""
    import trainscale_b200.optim as O
    from .ops import optim as K
    n_side = 4096 if small else 8192
    out = []
    # fp32 parameters and gradients (torch ties a .grad's dtype to its parameter's)
    cases = [("adam8bit", O.Adam8bit, dict(lr=1e-4, block_size=2048), 8 + 4 + 4, False),
             ("lamb", O.LAMB, dict(lr=1e-3), 28 + 12, False),
             ("sophia", O.SophiaG, dict(lr=1e-4), 24, True),
             ("schedule_free", O.ScheduleFreeAdamW, dict(lr=1e-3), 28, False),
             ("adopt", O.ADOPT, dict(lr=1e-3), 28, False),
             ("adafactor", O.AdaFactor, dict(lr=1e-3, relative_step=False), 4 + 12 + 12, False)]
    for name, cls, kw, bytes_per_el, needs_h in cases:
        res = {}
        for path in ("kernel", "torch"):
            p = torch.randn(n_side, n_side, device="cuda").requires_grad_(True)
            p.grad = torch.randn(n_side, n_side, device="cuda")
            opt = cls([p], **kw)
            saved = K.native_ok
            if path == "torch":
                K.native_ok = lambda *a, **k: False
            try:
                if needs_h:
                    opt.update_hessian(1)
                opt.step()                      # state creation outside the timed region
                res[path] = t(opt.step, iters=5, warmup=2)
            finally:
                K.native_ok = saved
            del opt, p
            torch.cuda.empty_cache()
        n = n_side * n_side
        out.append(dict(name=f"{name} step {n_side}x{n_side}", ms=res["kernel"], baseline_ms=res["torch"],
                        gbs=n * bytes_per_el / res["kernel"] / 1e6))
    return out


CASES["optimizers"] = bench_optimizers


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None, choices=sorted(CASES))
    ap.add_argument("--small", action="store_true", help="one small shape per case (for profiler captures)")
    ap.add_argument("--json", default=None)
    ap.add_argument("--device", default="cuda")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("no CUDA device")
        return 0
    import os
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    if "LOCAL_RANK" in os.environ:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    if world > 1:      # `torchrun ... -m trainscale_b200.benchmark_suite --only comm|ep`: one rank per GPU
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    pk = peaks()
    t = Timer(64 if a.small else 256)
    rows = []
    for name, fn in CASES.items():
        if (a.only and name != a.only) or (not a.only and name in ("comm", "ep")):
            continue                   # the collective cases need symmetric memory and run only when asked for
        rows += fn(t, a.small)
    if rank != 0:
        return 0
    tag = "of fallback" if pk.get("fallback") else "of measured"
    for r in rows:
        frac = r["gbs"] / pk["hbm_gbs"] if "gbs" in r else r["tflops"] / pk["bf16_tflops"]
        r["fraction_of_peak"] = frac
        sp = f"{r['baseline_ms'] / r['ms']:.2f}x" if r.get("baseline_ms") else "  -  "
        rate = f"{r['gbs']:.0f} GB/s" if "gbs" in r else f"{r['tflops']:.0f} TFLOPS"
        if r.get("nvlink_gbs"):
            rate += f" ({r['nvlink_gbs']:.0f} GB/s in over NVLink)"
        print(f"{r['name']:<40s} {r['ms']:8.3f} ms  baseline {r.get('baseline_ms') or float('nan'):8.3f} ms  {sp:>7s}  "
              f"{rate:>12s}  {frac:5.2f} {tag}")
    if a.json:
        Path(a.json).write_text(json.dumps(rows, indent=1))
    from .ops import _lib
    _lib.raise_on_any_device_error()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())


class BenchmarkResult(NamedTuple):
    """One benchmark row in the reference's record form (data_pipeline/trainer/kernels/benchmark_suite.py:88)."""
    name: str
    kernel_ms: float
    baseline_ms: float
    speedup: float
    metric_name: str
    kernel_metric: float
    baseline_metric: float

    @classmethod
    def from_row(cls, row: dict) -> "BenchmarkResult":
        """From a row dictionary of this suite ({name, ms, baseline_ms, gbs | tflops})."""
        metric = "GB/s" if "gbs" in row else "TFLOPS"
        val = row.get("gbs", row.get("tflops", 0.0))
        base = row.get("baseline_ms") or float("nan")
        return cls(row["name"], row["ms"], base, base / row["ms"], metric, val, val * row["ms"] / base)


def do_bench_fallback(fn, warmup: int = 25, rep: int = 100, quantiles=None, return_mode: str = "mean"):
    """CUDA-event timing of `fn` in ms without Triton's helper: `rep` timed calls after `warmup`; returns the mean (or
    min / max / median by `return_mode`), or the requested quantiles as a list."""
    fn()
    torch.cuda.synchronize()
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(rep)]
    for a, b in pairs:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    times = torch.tensor([a.elapsed_time(b) for a, b in pairs])
    if quantiles is not None:
        return torch.quantile(times, torch.tensor(quantiles, dtype=torch.float32)).tolist()
    return float(getattr(times, return_mode)())
