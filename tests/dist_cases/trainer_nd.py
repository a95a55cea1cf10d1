"""torchrun case: SOTATrainer driven by a config dict with pipeline or tensor+sequence parallelism.  Every step's loss
must match a single-process trainer fed the same global batches."""
import argparse
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from trainscale_b200.config.sota_config import SOTAConfig  # noqa: E402
from trainscale_b200.models.llama import LlamaConfig, build_model  # noqa: E402
from trainscale_b200.trainer.sota_trainer import SOTATrainer  # noqa: E402


CUDA = "--cuda" in sys.argv


COMM = sys.argv[sys.argv.index("--comm") + 1] if "--comm" in sys.argv else ("auto" if CUDA else "nccl")


def make_cfg(strategy, parallel, world, enabled):
    return SOTAConfig.from_dict({
        "training_mode": "full",
        "model": {"architecture": "llama-tiny"},
        "optimizer": {"type": "adamw", "learning_rate": 1e-2, "weight_decay": 0.0, "max_grad_norm": 1.0, "eps": 1e-3},
        "scheduler": {"type": "constant", "warmup_steps": 0},
        "loss": {"type": "chunked_ce"},
        "distributed": {"enabled": enabled, "backend": "nccl" if CUDA else "gloo", "strategy": strategy,
                        "world_size": world, "gradient_checkpointing": False, "parallel": parallel,
                        "comm": COMM},
        "hardware": {"precision": "bf16" if CUDA else "fp32", "device": "cuda" if CUDA else "cpu",
                     "device_id": int(os.environ.get("LOCAL_RANK", "0"))},
        "data": {"max_seq_length": 512 if CUDA else 32},
        "training": {"per_device_train_batch_size": 4, "gradient_accumulation_steps": 1, "max_steps": 100,
                     "logging_steps": 10 ** 9, "save_strategy": "no", "eval_strategy": "no",
                     "output_dir": "/tmp/ts_nd_case"},
    })


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="pp", choices=["pp", "sp", "cp", "ulysses", "tp_dp", "tp_pp", "ep"])
    ap.add_argument("--cuda", action="store_true", help="bf16 on GPUs through the CUDA kernels (fused TP path)")
    ap.add_argument("--comm", default=None, help="distributed.comm (default: auto on GPUs, nccl on CPU)")
    a = ap.parse_args()
    if CUDA:
        lr_ = int(os.environ["LOCAL_RANK"])
        torch.cuda.set_device(lr_)
        dist.init_process_group("nccl", device_id=torch.device("cuda", lr_))
    else:
        dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"])) if CUDA else torch.device("cpu")
    dt = torch.bfloat16 if CUDA else torch.float32
    S = 512 if CUDA else 32
    mcfg = LlamaConfig(vocab_size=256, hidden_size=256 if CUDA else 64, intermediate_size=512 if CUDA else 128,
                       num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=64 if CUDA else 16,
                       **(dict(num_local_experts=4, num_experts_per_tok=2) if a.mode == "ep" else {}))
    if a.mode == "pp":
        par = {"pp": world, "dp_shard": 1, "pp_schedule": "1f1b", "pp_microbatches": 2}
        strategy, B = "pipeline", 4
    elif a.mode in ("cp", "ulysses"):
        par = {"cp": world, "dp_shard": 1, "cp_balancer": "head_tail" if a.mode == "cp" else "ulysses"}
        strategy, B = "context_parallel", 1
    elif a.mode == "tp_pp":
        # 2 pipeline stages x tensor-parallel pairs with sequence parallelism: token-sharded activations inside and
        # between the stages, one sequence per pipeline micro-batch
        par = {"tp": 2, "pp": world // 2, "dp_shard": 1, "sp": True, "pp_schedule": "1f1b", "pp_microbatches": 2}
        strategy, B = "pipeline", 2
    elif a.mode == "ep":
        # data parallel ranks in expert-parallel pairs: each rank keeps 2 of the 4 experts of every layer
        par = {"ep": 2}
        strategy, B = "fsdp2", world
    elif a.mode == "tp_dp":
        # tensor parallel pairs x data parallel replicas: the clip must see the norm of the whole model, with the
        # parameters replicated inside a pair (norms, embedding, head) counted once
        par = {"tp": 2, "dp_shard": world // 2, "sp": True}
        strategy, B = "tensor_parallel", world // 2
    else:
        par = {"tp": world, "dp_shard": 1, "sp": True}
        strategy, B = "tensor_parallel", 1
    tr = SOTATrainer(make_cfg(strategy, par, world, True))
    tr.setup_model(model=build_model(mcfg, dtype=dt, device=dev, seed=7))
    tr.setup_optimizer()
    tr.setup_scheduler(100)
    # oracle: same model alone
    saved_init, saved_ws = dist.is_initialized, dist.get_world_size
    ref = SOTATrainer.__new__(SOTATrainer)
    env_ws = os.environ["WORLD_SIZE"]
    try:
        dist.is_initialized = lambda: False
        os.environ["WORLD_SIZE"] = "1"
        ref.__init__(make_cfg("single", {}, 1, False))
        ref.setup_model(model=build_model(mcfg, dtype=dt, device=dev, seed=7))
        ref.setup_optimizer()
        ref.setup_scheduler(100)
    finally:
        dist.is_initialized = saved_init
        os.environ["WORLD_SIZE"] = env_ws
    if CUDA:
        torch.cuda.set_device(dev)      # the single-process oracle selected its own default device
    g = torch.Generator().manual_seed(5)
    ok = True
    for step in range(3):
        ids = torch.randint(0, 256, (B, S), generator=g)
        mine = ids[rank // 2:rank // 2 + 1] if a.mode == "tp_dp" else (ids[rank:rank + 1] if a.mode == "ep" else ids)
        l1 = tr.train_step({"input_ids": mine, "labels": mine})
        try:
            dist.is_initialized = lambda: False
            l0 = ref.train_step({"input_ids": ids, "labels": ids})
        finally:
            dist.is_initialized = saved_init
        if a.mode in ("cp", "ulysses", "tp_dp", "ep"):
            # every rank reports the mean over ITS tokens; the shards are equal up to the one ignored last label
            t = torch.tensor([l1], device=dev)
            dist.all_reduce(t)
            l1 = float(t) / world
        good = abs(l1 - l0) < (3e-2 if CUDA else 2e-3) * max(1.0, abs(l0))
        if a.mode in ("tp_dp", "ep"):
            n1 = float(tr.engine.flat.last_grad_norm if a.mode == "tp_dp" else tr.engine.last_grad_norm)
            n0 = float(ref.engine.last_grad_norm)
            good &= abs(n1 - n0) < (3e-2 if CUDA else 1e-3) * max(1.0, n0)
            if rank == 0:
                print(f"step {step} grad_norm={n1:.5f} oracle={n0:.5f}", flush=True)
        ok &= good
        if rank == 0:
            print(f"step {step} mode={a.mode} loss={l1:.5f} oracle={l0:.5f} ok={good}", flush=True)
    if a.mode == "ep":
        peer = getattr(tr.engine, "peer", None)
        print(f"RESULT rank={rank} ep_peer_calls={0 if peer is None else peer.calls}", flush=True)
        tr.engine.check_comm_status()
    # one HuggingFace-layout checkpoint out of the model-parallel ranks: equal to the oracle's weights, and a resume
    # from it leaves every rank's shard / stage as it was
    import tempfile
    box = [tempfile.mkdtemp(prefix="ts_nd_ckpt_") if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    ck = Path(box[0]) / "checkpoint-3"
    tr.save_checkpoint(ck)
    exp = tr.export(output_dir=str(Path(box[0]) / "export"), fmt="safetensors")
    if rank == 0:
        from trainscale_b200.hub import ModelDeserializer
        want = ref.model.to_hf_state_dict()
        for d in (ck, exp):
            got = ModelDeserializer().load(d)
            same_keys = set(got) == set(want)
            worst = max(float((got[k].float().cpu() - want[k].float().cpu()).abs().max()) for k in want if k in got)
            shapes = all(got[k].shape == want[k].shape for k in want if k in got)
            good = same_keys and shapes and worst < (6e-2 if CUDA else 2e-3)
            ok &= good
            print(f"checkpoint {d.name}: keys={same_keys} shapes={shapes} max|diff|={worst:.2e} ok={good}", flush=True)
    own = tr.engine.stage_module if getattr(tr.engine, "pipelined", False) else tr.model     # a stage trains only its own layers
    before = {n: q.detach().clone() for n, q in own.named_parameters()}
    with torch.no_grad():
        for q in own.parameters():
            q.zero_()
    tr.load_checkpoint(ck)
    back = all(torch.equal(q.detach(), before[n]) for n, q in own.named_parameters())
    ok &= back
    if not back:
        bad = [n for n, q in own.named_parameters() if not torch.equal(q.detach(), before[n])]
        print(f"rank {rank}: not restored: {bad[:6]}", flush=True)
    if rank == 0:
        print(f"resume restores this rank's weights: {back}", flush=True)
    flag = torch.tensor([0.0 if ok else 1.0], device=dev)
    dist.all_reduce(flag)
    if CUDA:
        from trainscale_b200.ops import _lib
        _lib.raise_on_any_device_error()
        if rank == 0 and a.mode == "sp":
            from trainscale_b200.parallel import tp_fused
            print("tp comm:", tr.engine.tp.comm, "fused kernel calls:", tp_fused.CALLS)
            assert tp_fused.CALLS["gather_gemm"] > 0 and tp_fused.CALLS["gemm_reduce"] > 0, \
                "the decoder did not reach the fused tensor-parallel GEMMs"
    if rank == 0:
        print(f"RESULT mode={a.mode} ok={flag.item() == 0}")
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
