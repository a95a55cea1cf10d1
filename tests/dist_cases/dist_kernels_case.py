"""torchrun case (gloo, 4 ranks): the collective facade, the two-level all-reduce, the bucketed gradient hook and
the [data, pipeline, tensor] group factory."""
import copy
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.nn as nn

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from trainscale_b200.parallel import dist_kernels as DK  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    k = DK.get_distributed_kernels(DK.DistributedConfig(bucket_size_mb=0.001))
    ok = True
    t = torch.full((5,), float(rank + 1))
    ok &= float(k.all_reduce(t.clone())[0]) == sum(range(1, world + 1))
    a, b = torch.full((300,), float(rank)), torch.full((7,), float(rank), dtype=torch.float64)
    k.all_reduce_fused([a, b], average=True)
    ok &= abs(float(a[0]) - (world - 1) / 2) < 1e-6 and abs(float(b[0]) - (world - 1) / 2) < 1e-9
    g = k.all_gather(torch.full((2, 3), float(rank)), dim=1)
    ok &= g.shape == (2, 3 * world) and float(g[0, 3 * (world - 1)]) == world - 1
    full = torch.arange(world * 4, dtype=torch.float32).view(world * 2, 2)
    rs = k.reduce_scatter_tensor(None, full.clone())
    ok &= torch.equal(rs, full[2 * rank:2 * rank + 2] * world)
    sp = k.sequence_parallel_all_gather(torch.full((1, 2, 4), float(rank)), seq_dim=1)
    ok &= sp.shape == (1, 2 * world, 4)
    back = k.sequence_parallel_reduce_scatter(sp.clone(), seq_dim=1)
    ok &= torch.equal(back, torch.full((1, 2, 4), float(rank) * world))
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    got = k.pipeline_send_recv(torch.full((3,), float(rank)), torch.empty(3), nxt, prv)
    ok &= float(got[0]) == prv
    # the reference's call forms: asynchronous fused all-reduce (copy back in wait_pending), list reduce-scatter,
    # (x, dim, group) order of the sequence-parallel helpers, tagged point-to-point
    a2, b2 = torch.full((300,), float(rank)), torch.full((7,), float(rank), dtype=torch.float64)
    k.all_reduce_fused([a2, b2], average=True, async_op=True)
    k.wait_pending()
    ok &= abs(float(a2[0]) - (world - 1) / 2) < 1e-6 and abs(float(b2[0]) - (world - 1) / 2) < 1e-9
    mine_out = torch.empty(3)
    k.reduce_scatter(output=mine_out, input_tensors=[torch.full((3,), float(rank * 10 + r)) for r in range(world)])
    ok &= float(mine_out[0]) == sum(r * 10 + rank for r in range(world))
    sp0 = k.sequence_parallel_all_gather(x=torch.full((2, 4), float(rank)), dim=0, group=None, async_op=True)
    k.wait_pending()
    ok &= sp0.shape == (2 * world, 4) and float(sp0[2 * (world - 1), 0]) == world - 1
    got2 = k.pipeline_send_recv(torch.full((3,), float(rank)), torch.empty(3), nxt, prv, send_tag=5, recv_tag=5)
    ok &= float(got2[0]) == prv
    bc = k.broadcast(torch.full((2,), float(rank)), 1, None, async_op=True)
    k.wait_pending()
    ok &= float(bc[0]) == 1.0
    # groups: tp=2, pp=1 -> dp = world/2
    groups = DK.create_process_groups(tensor_parallel_size=2)
    ok &= dist.get_world_size(groups["tensor"]) == 2 and groups["pipeline"] is None
    ok &= (world == 2 and groups["data"] is None) or dist.get_world_size(groups["data"]) == world // 2
    # two-level all-reduce: local = tensor group, global = data group
    h = DK.HierarchicalCommunicator(groups["tensor"], groups["data"])
    x = torch.arange(11, dtype=torch.float32) + rank
    want = sum(torch.arange(11, dtype=torch.float32) + r for r in range(world))
    ok &= torch.allclose(h.hierarchical_all_reduce(x.clone()), want)
    # gradient hook vs plain averaging
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(8, 16), nn.Tanh(), nn.Linear(16, 4))
    ref = copy.deepcopy(m)
    hook = DK.GradientSyncHook(m.parameters(), DK.DistributedConfig(bucket_size_mb=0.0005))
    gen = torch.Generator().manual_seed(7)
    X = torch.randn(world * 2, 8, generator=gen)
    m(X[2 * rank:2 * rank + 2]).pow(2).mean().backward()
    hook.synchronize()
    ref(X).pow(2).mean().backward()
    ok &= all(torch.allclose(p.grad, q.grad, atol=1e-6) for p, q in zip(m.parameters(), ref.parameters()))
    ok &= len(hook._buckets) > 1
    hook.remove_hooks()
    # DDP compression hooks on a bucket: all ranks end with the same tensor, close to the exact mean
    from trainscale_b200.parallel import ddp as DDP
    gen = torch.Generator().manual_seed(100 + rank)
    mine = torch.randn(1003, generator=gen)
    exact = sum(torch.randn(1003, generator=torch.Generator().manual_seed(100 + r)) for r in range(world)) / world
    for name, hook, tol in (("bf16", DDP.BF16CompressionHook(), 2e-2), ("fp16", DDP.FP16CompressionHook(), 2e-3),
                            ("fp8", DDP.FP8CompressionHook(), 0.15), ("onebit", DDP.OneBitCompressionHook(), None),
                            ("topk", DDP.TopKSparsificationHook(0.25), None)):
        out = hook(dist.group.WORLD, mine.clone())
        same = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(same, out)
        good = all(torch.equal(same[0], t) for t in same)
        if tol is not None:
            good &= float((out - exact).abs().max()) < tol
        else:       # lossy with memory: what was delivered plus the mean of what every rank kept back is the exact mean
            err = hook.err[0]
            dist.all_reduce(err)
            good &= float((out + err / world - exact).abs().max()) < 1e-5
        ok &= good
        if rank == 0:
            print(f"hook {name}: ok={good}", flush=True)
    # AdaFactor on a row-sharded matrix == AdaFactor on the whole matrix
    from trainscale_b200.optim import AdaFactor, DistributedAdaFactor
    gen = torch.Generator().manual_seed(5)
    full = torch.randn(8 * world, 6, generator=gen)
    whole = full.clone().requires_grad_(True)
    shard = full[8 * rank:8 * rank + 8].clone().requires_grad_(True)
    oa, ob = AdaFactor([whole], lr=None, beta1=0.9, weight_decay=0.01), \
        DistributedAdaFactor([shard], lr=None, beta1=0.9, weight_decay=0.01)
    for _ in range(3):
        gr = torch.randn(8 * world, 6, generator=gen)
        whole.grad, shard.grad = gr.clone(), gr[8 * rank:8 * rank + 8].clone()
        oa.step()
        ob.step()
    e = float((shard - whole[8 * rank:8 * rank + 8]).abs().max())
    ok &= e < 1e-6
    if rank == 0:
        print(f"distributed adafactor: max diff {e:.1e}", flush=True)
    flag = torch.tensor([0.0 if ok else 1.0])
    dist.all_reduce(flag)
    if rank == 0:
        print(f"RESULT ok={flag.item() == 0}")
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
