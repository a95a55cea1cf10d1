"""torchrun case (gloo): the general pipeline API with one worker per rank.  Every schedule must leave, on each rank, the
gradients that a plain backward of the whole model gives for that rank's layers."""
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.nn as nn

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from trainscale_b200.parallel.pipeline import (DistributedContext, PipelineConfig, PipelineParallel,  # noqa: E402
                                               split_into_microbatches, split_model_into_stages)


def mk(n=8):
    torch.manual_seed(0)
    return nn.Sequential(*[nn.Sequential(nn.Linear(16, 16), nn.Tanh()) for _ in range(n)])


def main():
    dist.init_process_group("gloo")
    rank, P = dist.get_rank(), dist.get_world_size()
    ctx = DistributedContext(ranks=list(range(P)))
    torch.manual_seed(1)
    x, y = torch.randn(16, 16), torch.randn(16, 16)
    ref = mk()
    loss_ref = nn.functional.mse_loss(ref(x), y)
    loss_ref.backward()
    ok = True
    for sched, V, M in (("gpipe", 1, 4), ("1f1b", 1, 8), ("zero_bubble", 1, 8), ("interleaved", 2, 4), ("chimera", 1, 4)):
        cfg = PipelineConfig(num_stages=P, num_virtual_stages=V, num_microbatches=M, schedule=sched)
        n_virtual = P * V if sched != "chimera" else P
        all_stages = split_model_into_stages(mk(), n_virtual)
        ref_stages = split_model_into_stages(ref, n_virtual)
        if sched == "chimera":
            idx = [rank, P - 1 - rank]
            mine = [all_stages[rank], split_model_into_stages(mk(), n_virtual)[P - 1 - rank]]   # two separate replicas
        else:
            idx = [c * P + rank for c in range(V)]
            mine = [all_stages[i] for i in idx]
        pipe = PipelineParallel(mine, cfg, nn.functional.mse_loss, ctx=ctx)
        loss = pipe(split_into_microbatches(x, M), split_into_microbatches(y, M))
        worst = 0.0
        for st, i in zip(mine, idx):
            for a, b in zip(st.parameters(), ref_stages[i].parameters()):
                worst = max(worst, float((a.grad - b.grad).abs().max()))
        has_last = (n_virtual - 1) in idx
        good = worst < 1e-6 and (not has_last or abs(float(loss) - float(loss_ref)) < 1e-6 or sched == "chimera")
        if sched == "chimera" and has_last:
            # each rank that ends a direction sees the loss of its half of the micro-batches
            good = good and float(loss) > 0
        ok &= good
        print(f"rank {rank} {sched}: max grad diff {worst:.2e} loss {float(loss):.5f} ok={good}", flush=True)
    # neighbour-addressed sends: activations go down the pipe, gradients come back up; ends are no-ops
    from trainscale_b200.parallel.pipeline import P2PCommunicator
    comm = P2PCommunicator(ctx)
    good = comm.stage_id == rank and comm.prev_rank == (rank - 1 if rank else None) \
        and comm.next_rank == (rank + 1 if rank < P - 1 else None)
    act = torch.full((4, 3), float(rank))
    sent = comm.send_activation_async(act, 0)
    w, got = comm.recv_activation_async((4, 3), torch.float32, 0)
    good &= (sent is None) == (rank == P - 1) and (w is None) == (rank == 0)
    comm.synchronize_pending()
    if w is not None:
        good &= bool((got == rank - 1).all())
    comm.send_grad_async(torch.full((2,), 10.0 + rank), 0)
    w, got = comm.recv_grad_async(microbatch_id=0)
    comm.synchronize_pending()
    if w is not None:
        good &= bool((got == 11.0 + rank).all())
    ok &= bool(good)
    print(f"rank {rank} neighbour p2p ok={bool(good)}", flush=True)
    flag = torch.tensor([0.0 if ok else 1.0])
    dist.all_reduce(flag)
    if rank == 0:
        print(f"RESULT ok={flag.item() == 0}")
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
