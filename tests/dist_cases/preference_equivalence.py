"""torchrun case: DPO with the policy under the sharded engine and the frozen reference held as parameter-only shards
(re-gathered layer by layer) equals a single-process run on the concatenated batch."""
import argparse
import copy
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from trainscale_b200.data.synthetic import SyntheticPreferenceDataset  # noqa: E402
from trainscale_b200.models.llama import LlamaConfig, build_model  # noqa: E402
from trainscale_b200.parallel.flat_engine import EngineConfig, FlatShardedEngine  # noqa: E402
from trainscale_b200.rl import PreferenceTrainer  # noqa: E402


def collate(items):
    return {k: torch.stack([it[k] for it in items]) for k in items[0]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--strategy", default="FULL_SHARD")
    ap.add_argument("--comm", default="auto")
    a = ap.parse_args()
    cuda = a.device == "cuda"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if cuda:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    else:
        dist.init_process_group("gloo")
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"])) if cuda else torch.device("cpu")
    dtype = torch.bfloat16 if cuda else torch.float32
    cfg = LlamaConfig(vocab_size=512, hidden_size=256 if cuda else 64, intermediate_size=512 if cuda else 128,
                      num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64 if cuda else 16)
    P, R, B = (128, 128, 2) if cuda else (8, 8, 2)
    # bf16: a smaller step keeps the three compared steps out of the saturated regime (loss -> 0 within two steps at
    # lr 1e-2), where rounding differences between the two runs are amplified into the gradient norm
    ec = dict(param_dtype=dtype, lr=2e-3 if cuda else 1e-2, weight_decay=0.0, max_grad_norm=1.0, eps=1e-3)
    policy = build_model(cfg, dtype=dtype, device=dev, seed=3)
    ref_model = copy.deepcopy(policy).eval()
    # the reference differs from the policy so that its terms do not cancel
    with torch.no_grad():
        for p in ref_model.parameters():
            p.mul_(1.05)
    oracle_policy, oracle_ref = copy.deepcopy(policy), copy.deepcopy(ref_model)
    eng = FlatShardedEngine(policy, EngineConfig(sharding_strategy=a.strategy, comm=a.comm, **ec), device=dev)
    ref_eng = FlatShardedEngine(ref_model, EngineConfig(sharding_strategy=a.strategy, comm=a.comm, **ec), device=dev,
                                frozen=True)
    assert all(u.master.numel() == 0 and u.flat_grad is None for u in ref_eng.units), "frozen units hold parameters only"
    saved = dist.get_world_size
    o_eng = FlatShardedEngine.__new__(FlatShardedEngine)
    try:
        dist.get_world_size = lambda g=None: 1
        o_eng.__init__(oracle_policy, EngineConfig(sharding_strategy="SHARD_GRAD_OP", comm="nccl", **ec), device=dev)
    finally:
        dist.get_world_size = saved
    tr = PreferenceTrainer(policy, eng, ref_model, "dpo", 0.5)
    o_tr = PreferenceTrainer(oracle_policy, o_eng, oracle_ref, "dpo", 0.5)
    ds = SyntheticPreferenceDataset(cfg.vocab_size, P, R, 64, seed=1)
    ok = True
    for step in range(3):
        items = [ds[step * world * B + i] for i in range(world * B)]
        full = {k: v.to(dev) for k, v in collate(items).items()}
        mine = {k: v.to(dev) for k, v in collate(items[rank * B:(rank + 1) * B]).items()}
        loss, _, gn = tr.train_step(mine)
        o_loss, _, o_gn = o_tr.train_step(full)
        t = loss.detach().float().reshape(1).clone()
        dist.all_reduce(t)
        l1, l0 = float(t) / world, float(o_loss)
        good = abs(l1 - l0) < (3e-2 if cuda else 1e-4) * max(1.0, abs(l0)) and \
            abs(float(gn) - float(o_gn)) < (8e-2 if cuda else 1e-3) * max(1.0, float(o_gn))
        ok &= good
        if rank == 0:
            print(f"step {step} loss={l1:.6f} oracle={l0:.6f} gn={float(gn):.5f} oracle={float(o_gn):.5f} ok={good}", flush=True)
    err = 0.0
    with eng.summon_full_params():
        for (n, p), (_, q) in zip(policy.named_parameters(), oracle_policy.named_parameters()):
            err = max(err, (p.float() - q.float()).abs().max().item())
    ok &= err < (3e-2 if cuda else 2e-4)
    if a.strategy == "FULL_SHARD":
        assert all(u.flat_param.untyped_storage().nbytes() == 0 for u in ref_eng.units if u.resharded)
        assert any(u.resharded for u in ref_eng.units)
    flag = torch.tensor([0.0 if ok else 1.0], device=dev)
    dist.all_reduce(flag)
    if cuda:
        from trainscale_b200.ops import _lib
        torch.cuda.synchronize()
        _lib.raise_on_any_device_error()
        eng.check_comm_status()
        ref_eng.check_comm_status()
    if rank == 0:
        print(f"RESULT preference strategy={a.strategy} fused={eng._symm is not None} max_param_err={err:.3e} "
              f"ok={flag.item() == 0}")
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
