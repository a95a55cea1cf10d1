"""torchrun case (gloo): ContextParallelEngine - shard, ring attention forward/backward, gather - against full causal
attention on one process."""
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from trainscale_b200.ops.attention import attention_reference  # noqa: E402
from trainscale_b200.parallel import cp as CP  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    eng = CP.create_context_parallel_engine(cp_degree=world, group=dist.group.WORLD).unwrap()
    S, Hq, Hkv, D = 16 * world, 4, 2, 16
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(1, S, h, D, generator=g) for h in (Hq, Hkv, Hkv))
    ids = torch.arange(S).unsqueeze(0)
    lids, llab, _, lpos = eng.shard_inputs(ids, labels=ids)
    ok = lids.shape[1] == S // world and torch.equal(lids, lpos)          # token id == global position here
    ok &= torch.equal(llab[llab >= 0], lids[llab >= 0] + 1)                 # labels were shifted before sharding
    idx = lpos[0]
    ql, kl, vl = (t[:, idx].clone().requires_grad_(True) for t in (q, k, v))
    out = CP.ContextParallelAttention(eng)(ql, kl, vl)
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    ref = attention_reference(qf, kf, vf, causal=True)
    w = torch.randn(1, S, Hq, D, generator=g)
    (out * w[:, idx]).sum().backward()
    (ref * w).sum().backward()
    e_o = float((out - ref[:, idx]).abs().max())
    e_q = float((ql.grad - qf.grad[:, idx]).abs().max())
    e_k = float((kl.grad - kf.grad[:, idx]).abs().max())
    full = eng.gather_output(out.detach())
    e_g = float((full - ref.detach()).abs().max())
    ok &= max(e_o, e_q, e_k, e_g) < 1e-4 and eng.get_metrics().steps == 1
    # the same engine API without ring attention: contiguous shards + all-to-all (heads must divide by the group size)
    eng2 = CP.create_context_parallel_engine(cp_degree=world, use_ring_attention=False, group=dist.group.WORLD).unwrap()
    _, _, _, pos2 = eng2.shard_inputs(ids)
    idx2 = pos2[0]
    ok &= torch.equal(idx2, torch.arange(rank * S // world, (rank + 1) * S // world))
    if Hq % world == 0 and Hkv % world == 0:
        out2 = eng2.ring_attention_forward(q[:, idx2], k[:, idx2], v[:, idx2])
        ok &= float((out2 - ref.detach()[:, idx2]).abs().max()) < 1e-4
        ok &= float((eng2.gather_output(out2) - ref.detach()).abs().max()) < 1e-4
    cpw = CP.ContextParallel(dist.group.WORLD)
    sh = cpw.shard_inputs({"input_ids": ids})
    ok &= torch.equal(cpw.restore_sequence(sh["input_ids"]), ids)
    print(f"rank {rank}: |o|={e_o:.1e} |dq|={e_q:.1e} |dk|={e_k:.1e} |gather|={e_g:.1e} ok={ok}", flush=True)
    flag = torch.tensor([0.0 if ok else 1.0])
    dist.all_reduce(flag)
    if rank == 0:
        print(f"RESULT ok={flag.item() == 0}")
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
