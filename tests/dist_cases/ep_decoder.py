"""torchrun case (gloo): a mixture-of-experts decoder with its experts sharded over 2 ranks (all-to-all dispatch) gives
the loss and gradients of the same model with all experts local.  Both ranks see the same batch here, so expert
gradients on the owner are the sum over the group's token copies: world x the single-process gradient."""
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from trainscale_b200.models.llama import build_model, preset_config  # noqa: E402
from trainscale_b200.parallel.ep import shard_model_for_expert_parallel  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = preset_config("moe-tiny", vocab_size=128, hidden_size=64, intermediate_size=96, head_dim=16)
    ref = build_model(cfg, dtype=torch.float32, device="cpu", seed=5)
    m = build_model(cfg, dtype=torch.float32, device="cpu", seed=5)
    assert shard_model_for_expert_parallel(m, dist.group.WORLD) == cfg.num_hidden_layers
    g = torch.Generator().manual_seed(9 + rank)                    # different tokens on every rank
    ids = torch.randint(0, 128, (2, 24), generator=g)
    out = m(ids, labels=ids)
    out.loss.backward()
    want = ref(ids, labels=ids)
    want.loss.backward()
    e_loss = abs(float(out.loss) - float(want.loss))
    # attention / router gradients are local quantities: equal to the single-process ones for this rank's tokens
    e_attn = float((m.model.layers[0].self_attn.wqkv.grad - ref.model.layers[0].self_attn.wqkv.grad).abs().max())
    e_router = float((m.model.layers[1].mlp.router.grad - ref.model.layers[1].mlp.router.grad).abs().max())
    # expert gradients: the owner holds the sum over ALL ranks' tokens; compare with the sum of the references
    El = cfg.num_local_experts // world
    mine = ref.model.layers[0].mlp.w_down.grad[rank * El:(rank + 1) * El].clone()
    allg = [torch.zeros_like(ref.model.layers[0].mlp.w_down.grad) for _ in range(world)]
    dist.all_gather(allg, ref.model.layers[0].mlp.w_down.grad)
    total = sum(allg)[rank * El:(rank + 1) * El]
    e_exp = float((m.model.layers[0].mlp.w_down.grad - total).abs().max())
    full_gu, _ = m.model.layers[0].mlp.full_expert_weights()
    e_w = float((full_gu - ref.model.layers[0].mlp.w_gate_up.detach()).abs().max())
    sd, sd_ref = m.to_hf_state_dict(), ref.to_hf_state_dict()          # export gathers the experts of every rank
    e_sd = max(float((sd[k] - sd_ref[k]).abs().max()) for k in sd_ref) if set(sd) == set(sd_ref) else 1.0
    ok = max(e_loss, e_attn, e_router, e_exp) < 2e-5 and e_w == 0.0 and e_sd == 0.0 and float(mine.abs().sum()) > 0
    print(f"RESULT rank={rank} loss={e_loss:.1e} attn={e_attn:.1e} router={e_router:.1e} experts={e_exp:.1e} ok={ok}",
          flush=True)
    flag = torch.tensor([0.0 if ok else 1.0])
    dist.all_reduce(flag)
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
