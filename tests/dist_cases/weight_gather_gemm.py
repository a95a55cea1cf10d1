"""torchrun case (CUDA): y = x @ gather_rows(W shards)^T with the weight all-gather inside the GEMM kernel, against
the product with the unsharded weight."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from trainscale_b200.ops import _lib  # noqa: E402
from trainscale_b200.parallel import tp as TP, tp_fused  # noqa: E402
from trainscale_b200.parallel.symm import SymmetricHeap  # noqa: E402


def main():
    rank, world, lr = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(lr)
    dist.init_process_group("nccl", device_id=torch.device("cuda", lr))
    dev = torch.device("cuda", lr)
    heap = SymmetricHeap.try_create(None, dev)
    assert heap is not None, "symmetric memory unavailable"
    heap.wait_cycles = int(5 * 1.9e9)
    ctx = TP.TPContext.from_group(dist.group.WORLD, False, "fused", heap)
    ok = True
    for M, N, K in ((4096, 6144, 1024), (8192, 4096, 4096), (512, 1024, 256)):     # the last one takes the fallback
        torch.manual_seed(1)
        w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
        dist.broadcast(w, 0)
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        shard = w[rank * N // world:(rank + 1) * N // world].contiguous()
        for _ in range(2):                                                          # second call reuses the buffers
            y = tp_fused.gather_weight_linear(x, shard, ctx)
        torch.cuda.synchronize()
        ref = x.float() @ w.float().t()
        err = ((y.float() - ref).abs().max() / ref.abs().max()).item()
        good = err < 2e-2 and heap.status.item() == 0
        ok &= good
        if rank == 0:
            print(f"M{M} N{N} K{K}: relerr {err:.2e} ok={good}", flush=True)
    _lib.raise_on_any_device_error()
    flag = torch.tensor([0.0 if ok else 1.0], device=dev)
    dist.all_reduce(flag)
    if rank == 0:
        print(f"RESULT weight_gather ok={flag.item() == 0}")
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
