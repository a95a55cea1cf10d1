"""torchrun case: expert-parallel MoE (experts sharded over ranks, all-to-all dispatch/combine) == local MoE."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from trainscale_b200.parallel.ep import AllToAllDispatcher, ExpertParallelConfig, ExpertParallelMoE, MoELayer  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = ExpertParallelConfig(num_experts=4, top_k=2, hidden_size=32, intermediate_size=48)
    torch.manual_seed(0)
    ref = MoELayer(cfg)
    ep = ExpertParallelMoE(cfg, dist.group.WORLD)
    El = cfg.num_experts // world
    with torch.no_grad():
        ep.router.weight.copy_(ref.router.weight)
        ep.experts.w_gate_up.copy_(ref.experts.w_gate_up[rank * El:(rank + 1) * El])
        ep.experts.w_down.copy_(ref.experts.w_down[rank * El:(rank + 1) * El])
    torch.manual_seed(100 + rank)
    x = torch.randn(3, 7, 32, requires_grad=True)
    xr = x.detach().clone().requires_grad_(True)
    y, yr = ep(x), ref(xr)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g)
    e1 = (y - yr).abs().max().item()
    e2 = (x.grad - xr.grad).abs().max().item()
    # expert weight grads: sum over ranks of the reference grads for my experts
    gr = ref.experts.w_down.grad.clone()
    dist.all_reduce(gr)
    e3 = (ep.experts.w_down.grad - gr[rank * El:(rank + 1) * El]).abs().max().item()
    # capacity-slotted form of the dispatcher: identity experts, so combine(dispatch(x)) == x * (sum of its weights);
    # rows that arrive for a local expert are those of rank 0 then rank 1, counted per expert
    d = AllToAllDispatcher(cfg.num_experts, El, 8, dist.group.WORLD)
    flat = x.detach().reshape(-1, 32)
    out = ep.router(hidden_states=x.detach())
    mask = out.dispatch_mask.any(-1)
    rows, counts = d.dispatch(tokens=flat, dispatch_mask=mask)
    weights = torch.zeros(flat.shape[0], cfg.num_experts).scatter_(1, out.expert_indices, out.expert_weights.detach())
    kept = (mask.long().cumsum(0) - 1 < 8) & mask
    back = d.combine(expert_outputs=rows, combine_weights=weights, original_positions=torch.arange(flat.shape[0]),
                     num_tokens=flat.shape[0])
    e4 = (back - flat * (weights * kept).sum(1, keepdim=True)).abs().max().item()
    sent = kept.sum(0)
    dist.all_reduce(sent)
    e5 = float((counts - sent[rank * El:(rank + 1) * El]).abs().max())
    ok = e1 < 1e-5 and e2 < 1e-5 and e3 < 1e-5 and e4 < 1e-5 and e5 == 0 and rows.shape == (El, world * 8, 32)
    print(f"RESULT rank={rank} out={e1:.1e} dx={e2:.1e} dw={e3:.1e} slotted={e4:.1e}/{e5:.0f} ok={ok}", flush=True)
    flag = torch.tensor([0.0 if ok else 1.0])
    dist.all_reduce(flag)
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
