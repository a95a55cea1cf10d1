"""torchrun case: a sharded engine writes a torch.distributed.checkpoint directory; rank 0 then reads it back into a
fresh single-process engine and compares weights, moments and step with the gathered state of the run."""
import argparse
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from trainscale_b200.ckpt.dcp import load_dcp_checkpoint, save_dcp_checkpoint  # noqa: E402
from trainscale_b200.models.llama import LlamaConfig, build_model  # noqa: E402
from trainscale_b200.parallel.flat_engine import EngineConfig, FlatShardedEngine  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--strategy", default="FULL_SHARD")
    ap.add_argument("--dir", required=True)
    a = ap.parse_args()
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=16)
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=1)
    eng = FlatShardedEngine(model, EngineConfig(sharding_strategy=a.strategy, param_dtype=torch.float32, lr=1e-2,
                                                comm="nccl"), device=torch.device("cpu"))
    g = torch.Generator().manual_seed(3)
    for _ in range(2):
        ids = torch.randint(0, 128, (world * 2, 16), generator=g)
        mine = ids[rank * 2:(rank + 1) * 2]
        eng.backward(model(mine, labels=mine).loss)
        eng.step()
    save_dcp_checkpoint(eng, model, a.dir, epoch=1, step=2, extra={"note": "x"})
    # what the run holds, gathered
    with eng.summon_full_params():
        want_w = {n: p.detach().clone() for n, p in model.named_parameters()}
    want_m = {}
    for u in eng.units:
        parts = [torch.empty_like(u.exp_avg) for _ in range(world)]
        dist.all_gather(parts, u.exp_avg)
        want_m[u.name] = torch.cat(parts)[:u.used]
    ok = True
    if rank == 0:
        saved = dist.is_initialized, dist.get_world_size
        try:
            dist.is_initialized = lambda: False
            fresh = build_model(cfg, dtype=torch.float32, device="cpu", seed=99)
            e2 = FlatShardedEngine(fresh, EngineConfig(sharding_strategy="SHARD_GRAD_OP", param_dtype=torch.float32,
                                                       lr=1e-2), device=torch.device("cpu"))
            meta = load_dcp_checkpoint(e2, fresh, a.dir)
        finally:
            dist.is_initialized, dist.get_world_size = saved
        ok &= meta.get("api_version") == "dcp_modern_v2" and meta.get("step") == 2 and e2.step_count == eng.step_count
        for n, p in fresh.named_parameters():
            ok &= torch.allclose(p, want_w[n], atol=0, rtol=0)
        for u in e2.units:
            ok &= torch.equal(u.exp_avg[:u.used], want_m[u.name])
        print(f"RESULT dcp strategy={a.strategy} ok={bool(ok)}", flush=True)
    flag = torch.tensor([0.0 if ok else 1.0])
    dist.all_reduce(flag)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
