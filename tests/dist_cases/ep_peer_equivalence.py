"""torchrun case (NCCL, 1..8 GPUs): one mixture-of-experts block with its experts sharded over the ranks.  Three arms on
the same router weights, tokens (different on every rank) and output gradients:
  ref    all experts local (`LlamaMoEMLP`: device-side plan + grouped GEMMs)
  nccl   `ExpertParallelDecoderMoE` moving tokens with the library all-to-all
  peer   the same block on the peer-memory dispatcher (`parallel/ep_peer.py`)
Outputs, input gradients and router gradients are per-rank quantities and must agree across the arms; an owner's expert
gradients hold every rank's contributions, so they are compared with the all-reduced reference gradients.
With one rank the peer arm degenerates to local buffers, which still runs every kernel and the autograd wiring."""
import copy
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from trainscale_b200.models.llama import LlamaMoEMLP, preset_config  # noqa: E402
from trainscale_b200.ops import _lib  # noqa: E402
from trainscale_b200.parallel.ep import ExpertParallelDecoderMoE, make_peer_dispatcher  # noqa: E402


def run(block, x, g):
    x = x.clone().requires_grad_(True)
    y = block(x)
    (y.float() * g.float()).sum().backward()
    return y.detach().float(), x.grad.float()


def rel(a, b):
    return float((a - b).abs().max() / b.abs().max().clamp(min=1e-6))


def main():
    import os
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", local)
    E = 8
    cfg = preset_config("moe-tiny", hidden_size=256, intermediate_size=384, num_local_experts=E, num_experts_per_tok=2)
    torch.manual_seed(3)
    ref = LlamaMoEMLP(cfg)
    for p in ref.parameters():
        torch.nn.init.normal_(p, std=0.05)
    ref = ref.to(dev, torch.bfloat16)
    peer = make_peer_dispatcher(dist.group.WORLD, E, dev)
    assert peer is not None, "symmetric memory is not available on this machine"
    arms = {"nccl": ExpertParallelDecoderMoE(copy.deepcopy(ref), dist.group.WORLD, None),
            "peer": ExpertParallelDecoderMoE(copy.deepcopy(ref), dist.group.WORLD, peer)}
    ok = True
    for it, T in enumerate((300, 173)):                 # second call: fewer tokens through the same buffers
        gen = torch.Generator(device="cpu").manual_seed(100 * it + rank)
        x = (torch.randn(T, cfg.hidden_size, generator=gen) * 0.5).to(dev, torch.bfloat16)
        g = (torch.randn(T, cfg.hidden_size, generator=gen) * 0.5).to(dev, torch.bfloat16)
        for m in (ref, *arms.values()):
            m.zero_grad(set_to_none=True)
        y0, dx0 = run(ref, x, g)
        El = E // world
        want = {}
        for name in ("w_gate_up", "w_down"):
            t = getattr(ref, name).grad.float().clone()
            dist.all_reduce(t)
            want[name] = t[rank * El:(rank + 1) * El]
        for arm, blk in arms.items():
            y, dx = run(blk, x, g)
            errs = {"y": rel(y, y0), "dx": rel(dx, dx0), "router": rel(blk.router.grad.float(), ref.router.grad.float()),
                    "gate_up": rel(blk.w_gate_up.grad.float(), want["w_gate_up"]),
                    "down": rel(blk.w_down.grad.float(), want["w_down"])}
            good = all(v < 3e-2 for v in errs.values())
            ok = ok and good
            print(f"RESULT rank={rank} T={T} arm={arm} " + " ".join(f"{k}={v:.1e}" for k, v in errs.items()) +
                  f" ok={good}", flush=True)
    torch.cuda.synchronize()
    peer.heap.check_status()
    peer.check()
    _lib.raise_on_any_device_error()
    print(f"RESULT rank={rank} peer_calls={peer.calls} ok={ok}", flush=True)
    flag = torch.tensor([0.0 if ok else 1.0], device=dev)
    dist.all_reduce(flag)
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
