"""torchrun case (gloo): ParallelEmbedding / ParallelMLP / ParallelSelfAttention / SequenceParallelLayerNorm built from
slices of full weights must reproduce the unsharded computation (outputs, input gradients, weight-slice gradients),
with and without sequence parallelism."""
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.nn.functional as F

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from trainscale_b200.ops.attention import attention_reference  # noqa: E402
from trainscale_b200.parallel import tp as TP  # noqa: E402

H, I, NH, NKV, D, S, V = 64, 96, 4, 2, 16, 8, 50


def rope(x):
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = torch.arange(x.shape[1], dtype=torch.float32)[:, None] * inv[None]
    cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    a, b = x[..., : D // 2], x[..., D // 2:]
    return torch.cat((a * cos - b * sin, b * cos + a * sin), -1)


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    mgr = TP.ProcessGroupManager.get().initialize(tensor_parallel_size=world)
    g = torch.Generator().manual_seed(0)
    W = {k: torch.randn(*s, generator=g) * 0.1 for k, s in dict(
        gate=(I, H), up=(I, H), down=(H, I), q=(NH * D, H), k=(NKV * D, H), v=(NKV * D, H), o=(H, NH * D),
        emb=(V, H), ln=(H,)).items()}
    x0 = torch.randn(1, S, H, generator=g)
    ids = torch.randint(0, V, (1, S), generator=g)
    ok = True
    for sp in (False, True):
        ctx = mgr.tp_context(sequence_parallel=sp)
        sl = lambda t, dim: t.chunk(world, dim)[rank].contiguous()   # noqa: E731
        mlp = TP.ParallelMLP(H, I, ctx, dtype=torch.float32)
        att = TP.ParallelSelfAttention(H, NH, ctx, NKV, D, dtype=torch.float32)
        ln = TP.SequenceParallelLayerNorm(H, dtype=torch.float32)
        with torch.no_grad():
            mlp.gate.weight.copy_(sl(W["gate"], 0)); mlp.up.weight.copy_(sl(W["up"], 0)); mlp.down.weight.copy_(sl(W["down"], 1))
            att.q_proj.weight.copy_(sl(W["q"], 0)); att.k_proj.weight.copy_(sl(W["k"], 0)); att.v_proj.weight.copy_(sl(W["v"], 0))
            att.o_proj.weight.copy_(sl(W["o"], 1)); ln.weight.copy_(1 + W["ln"])
        # reference
        xr = x0.clone().requires_grad_(True)
        lnw = (1 + W["ln"]).clone().requires_grad_(True)
        h = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * lnw
        q = rope((h @ W["q"].t()).view(1, S, NH, D)); k = rope((h @ W["k"].t()).view(1, S, NKV, D))
        v = (h @ W["v"].t()).view(1, S, NKV, D)
        a = attention_reference(q, k, v, causal=True).reshape(1, S, NH * D) @ W["o"].t()
        y_ref = a + (F.silu(a @ W["gate"].t()) * (a @ W["up"].t())) @ W["down"].t()
        y_ref.pow(2).sum().backward()
        # parallel
        xp = x0.clone().requires_grad_(True)
        xin = TP.scatter_to_sequence_parallel_region(xp.view(S, H), ctx).view(1, -1, H) if sp else xp
        a_p = att(ln(xin))
        y = a_p + mlp(a_p.view(-1, H) if sp else a_p).view(a_p.shape)
        y_full = TP.all_gather_from_sequence_parallel_region(y.view(-1, H), ctx).view(1, S, H) if sp else y
        # under SP every rank holds the full output after the gather; its backward reduce-scatters, summing `world` copies
        (y_full.pow(2).sum() / (world if sp else 1)).backward()
        if sp:
            TP.allreduce_sequence_parallel_grads(ln, ctx)
        e_y = float((y_full - y_ref).abs().max())
        e_x = float((xp.grad - xr.grad).abs().max())
        e_ln = float((ln.weight.grad - lnw.grad).abs().max())
        good = e_y < 1e-4 and e_x < 1e-3 and e_ln < 1e-3
        ok &= good
        if rank == 0:
            print(f"sp={sp}: |y|={e_y:.1e} |dx|={e_x:.1e} |dln|={e_ln:.1e} ok={good}", flush=True)
    ctx = mgr.tp_context()
    emb = TP.ParallelEmbedding(V, H, ctx, dtype=torch.float32)
    with torch.no_grad():
        emb.weight.copy_(W["emb"].chunk(world, 1)[rank])
    e = float((emb(ids) - F.embedding(ids, W["emb"])).abs().max())
    ok &= e == 0.0
    ok &= mgr.tp_size == world and mgr.dp_size == 1 and mgr.sp_group is mgr.tp_group
    flag = torch.tensor([0.0 if ok else 1.0])
    dist.all_reduce(flag)
    if rank == 0:
        print(f"RESULT ok={flag.item() == 0}")
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
