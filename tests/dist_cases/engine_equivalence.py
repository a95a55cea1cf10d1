"""Launched under torch.distributed.run: trains a small decoder for a few steps with the flat engine in a given
(strategy, comm) mode and compares weights with a single-process run on the concatenated global batch."""
import argparse
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from trainscale_b200.models.llama import LlamaConfig, build_model  # noqa: E402
from trainscale_b200.parallel.flat_engine import EngineConfig, FlatShardedEngine  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--strategy", default="SHARD_GRAD_OP")
    ap.add_argument("--comm", default="auto")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--tol", type=float, default=2e-4)
    ap.add_argument("--recompute", action="store_true", help="layer-wise activation recomputation in both runs")
    ap.add_argument("--accum", type=int, default=1, help="micro-batches per optimizer step")
    ap.add_argument("--replicate", type=int, default=1, help="hybrid sharding: number of replicas of every shard")
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
    cfg = LlamaConfig(vocab_size=1024, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64)
    S, B = (256, 2) if cuda else (32, 2)
    model = build_model(cfg, dtype=dtype, device=dev, seed=3)
    ref = build_model(cfg, dtype=dtype, device=dev, seed=3)
    if a.recompute:
        model.gradient_checkpointing_enable(1)
        ref.gradient_checkpointing_enable(1)
    ec = dict(gradient_accumulation_steps=a.accum, param_dtype=dtype, lr=1e-2, weight_decay=0.01, max_grad_norm=1.0, eps=1e-3)  # large eps: no sign(g) blow-up of rounding noise
    shard_pg = rep_pg = None
    if a.replicate > 1:
        # ranks [0..S) [S..2S) ... are the shard groups; ranks with equal position in their group replicate each other
        S_ = world // a.replicate
        for g0 in range(a.replicate):
            grp = dist.new_group(list(range(g0 * S_, (g0 + 1) * S_)))
            if rank // S_ == g0:
                shard_pg = grp
        for j in range(S_):
            grp = dist.new_group(list(range(j, world, S_)))
            if rank % S_ == j:
                rep_pg = grp
    eng = FlatShardedEngine(model, EngineConfig(sharding_strategy=a.strategy, comm=a.comm, **ec), device=dev,
                            process_group=shard_pg, replicate_group=rep_pg)
    # the oracle: one process, global batch, no sharding (a private 1-rank view of the engine)
    ref_eng = FlatShardedEngine.__new__(FlatShardedEngine)
    saved = dist.get_world_size
    try:
        dist.get_world_size = lambda g=None: 1   # build the oracle engine as if alone
        ref_eng.__init__(ref, EngineConfig(sharding_strategy="SHARD_GRAD_OP", comm="nccl", **ec), device=dev)
    finally:
        dist.get_world_size = saved
    g = torch.Generator().manual_seed(11)
    fused = eng._symm is not None
    for step in range(a.steps):
        for micro in range(a.accum):
            ids = torch.randint(0, cfg.vocab_size, (world * B, S), generator=g).to(dev)
            mine = ids[rank * B:(rank + 1) * B]
            loss = model(mine, labels=mine, loss_scale=1.0 / a.accum).loss
            eng.backward(loss)
            rl = ref(ids, labels=ids, loss_scale=1.0 / a.accum).loss
            ref_eng.backward(rl)
        gn = eng.step()
        rgn = ref_eng.step()
        if cuda:
            torch.cuda.synchronize()
        assert abs(float(gn) - float(rgn)) < (5e-2 if cuda else 1e-3) * max(1.0, float(rgn)), (float(gn), float(rgn))
    err = 0.0
    with eng.summon_full_params():
        for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
            err = max(err, (p.float() - q.float()).abs().max().item())
    if a.strategy == "FULL_SHARD" and world > 1:
        assert all(u.flat_param.untyped_storage().nbytes() == 0 for u in eng.units if u.resharded), \
            "parameters must be re-sharded after use"
        assert any(u.resharded for u in eng.units)
    tol = 3e-2 if cuda else a.tol
    ok = err < tol
    flag = torch.tensor([0.0 if ok else 1.0], device=dev)
    dist.all_reduce(flag)
    if cuda:
        from trainscale_b200.ops import _lib
        _lib.raise_on_any_device_error()
        if eng._symm is not None:
            eng._symm.check_status()
    if rank == 0:
        print(f"RESULT strategy={a.strategy} comm={a.comm} fused={fused} max_param_err={err:.3e} ok={flag.item() == 0}")
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
