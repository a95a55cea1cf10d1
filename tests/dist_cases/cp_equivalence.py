"""torchrun case: ring attention over a head-tail sharded sequence == full causal attention (forward + backward)."""
import math
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from trainscale_b200.ops.attention import attention_reference  # noqa: E402
from trainscale_b200.parallel import cp as CP  # noqa: E402


def main():
    cuda = "--cuda" in sys.argv
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if cuda:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
        dev, dtype = torch.device("cuda", int(os.environ["LOCAL_RANK"])), torch.bfloat16
    else:
        dist.init_process_group("gloo")
        dev, dtype = torch.device("cpu"), torch.float32
    Hq, Hkv, D = 4, 2, (128 if cuda else 16)
    S = (2048 if cuda else 64) * world
    g = torch.Generator().manual_seed(3)
    q = torch.randn(1, S, Hq, D, generator=g).to(dev, dtype)
    k = torch.randn(1, S, Hkv, D, generator=g).to(dev, dtype)
    v = torch.randn(1, S, Hkv, D, generator=g).to(dev, dtype)
    do = torch.randn(1, S, Hq, D, generator=g).to(dev, dtype)
    bal = CP.HeadTailBalancer(world, rank)
    ql, kl, vl, dol = [bal.shard(t).clone().requires_grad_(t is not do) for t in (q, k, v, do)]
    comm = sys.argv[sys.argv.index("--comm") + 1] if "--comm" in sys.argv else None
    out = CP.ring_attention(ql, kl, vl, dist.group.WORLD, comm=comm)
    out.backward(dol)
    if cuda:
        used = "peer" if CP._PeerKV._bufs else "ring"
        # device time of forward+backward, max over ranks (second and third call: buffers and heap exist by then)
        ms = 0.0
        for _ in range(3):
            q2, k2, v2 = (t.detach().clone().requires_grad_(True) for t in (ql, kl, vl))
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            CP.ring_attention(q2, k2, v2, dist.group.WORLD, comm=comm).backward(dol)
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b)
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            print(f"TIMING comm={comm} path={used} fwd+bwd {t.item():.3f} ms (S={S}, cp={world})", flush=True)
        from trainscale_b200.ops import _lib
        _lib.raise_on_any_device_error()
    qr, kr, vr = [t.float().clone().requires_grad_(True) for t in (q, k, v)]
    ref = attention_reference(qr, kr, vr, True)
    ref.backward(do.float())
    tol = 3e-2 if cuda else 1e-4

    def err(a, b):
        return (a.float() - b.float()).abs().max().item() / max(b.float().abs().max().item(), 1e-9)

    e = [err(out, bal.shard(ref)), err(ql.grad, bal.shard(qr.grad)), err(kl.grad, bal.shard(kr.grad)),
         err(vl.grad, bal.shard(vr.grad))]
    full = CP.gather_output(out.detach(), dist.group.WORLD)
    e.append(err(full, ref))
    ok = all(x < tol for x in e)
    print(f"RESULT rank={rank} cp={world} errs={[f'{x:.1e}' for x in e]} ok={ok}", flush=True)
    flag = torch.tensor([0.0 if ok else 1.0], device=dev)
    dist.all_reduce(flag)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
