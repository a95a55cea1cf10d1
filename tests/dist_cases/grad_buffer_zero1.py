"""torchrun case (gloo): contiguous buffers + bucketed reduce-scatter + ZeRO-1 optimizer on 2 ranks against AdamW on
one process with the whole batch; also the plain all-reduce (DDP) flavour of the buffer."""
import copy
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.nn as nn

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from trainscale_b200.optim import AdamW  # noqa: E402
from trainscale_b200.parallel.grad_buffer import (DistributedOptimizer, ParamAndGradBuffer, partition_buckets,  # noqa: E402
                                                  shard_buffer)


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    base = nn.Sequential(nn.Linear(32, 48), nn.GELU(), nn.Linear(48, 48), nn.GELU(), nn.Linear(48, 8))
    ref = copy.deepcopy(base)
    g = torch.Generator().manual_seed(1)
    data = [(torch.randn(4 * world, 32, generator=g), torch.randn(4 * world, 8, generator=g)) for _ in range(3)]
    ok = True

    # ZeRO-1
    model = copy.deepcopy(base)
    buf = ParamAndGradBuffer(model.parameters(), param_dtype=torch.float32, grad_dtype=torch.float32,
                             bucket_size=2000, use_distributed_optimizer=True)
    groups = partition_buckets([buf])
    opt = DistributedOptimizer([buf], lr=1e-2, weight_decay=0.01, max_grad_norm=0.5, bucket_groups=groups)
    ro = AdamW(ref.parameters(), lr=1e-2, weight_decay=0.01)
    for x, y in data:
        opt.zero_grad()
        nn.functional.mse_loss(model(x[4 * rank:4 * rank + 4]), y[4 * rank:4 * rank + 4]).backward()
        n = opt.step()
        nn.functional.mse_loss(ref(x), y).backward()
        nr = torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.5)
        ro.step()
        ro.zero_grad()
        ok &= abs(float(n) - float(nr)) < 1e-4 * max(1.0, float(nr))
    worst = max(float((a - b).abs().max()) for a, b in zip(model.parameters(), ref.parameters()))
    ok &= worst < 2e-4
    ok &= len(buf.buckets) >= 2 and all(b.grad_data.numel() % (world * 64) == 0 for b in buf.buckets)
    ok &= all(p.data_ptr() >= buf.param_data.data_ptr() for p in model.parameters())
    if rank == 0:
        print(f"zero1: buckets={len(buf.buckets)} max|w-ref|={worst:.2e} ok={ok}", flush=True)

    # all-reduce flavour with overlap hooks + host offload round trip
    model2 = copy.deepcopy(base)
    buf2 = ParamAndGradBuffer(model2.parameters(), param_dtype=torch.float32, grad_dtype=torch.float32, bucket_size=2000)
    groups2 = partition_buckets([buf2])
    x, y = data[0]
    nn.functional.mse_loss(model2(x[4 * rank:4 * rank + 4]), y[4 * rank:4 * rank + 4]).backward()
    for gr in groups2:
        gr.finish_grad_sync()
    ref2 = copy.deepcopy(base)
    nn.functional.mse_loss(ref2(x), y).backward()
    w2 = max(float((p.main_grad - q.grad).abs().max()) for p, q in zip(model2.parameters(), ref2.parameters()))
    snap = buf2.param_data.clone()
    freed = buf2.offload_to_cpu()
    buf2.reload_from_cpu()
    ok2 = w2 < 1e-6 and freed > 0 and torch.equal(buf2.param_data, snap) and len(shard_buffer(buf2.grad_data, world)) == world
    ok &= ok2
    if rank == 0:
        print(f"allreduce: max|g-ref|={w2:.2e} offload_bytes={freed} ok={ok2}", flush=True)
    flag = torch.tensor([0.0 if ok else 1.0])
    dist.all_reduce(flag)
    if rank == 0:
        print(f"RESULT ok={flag.item() == 0}")
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
