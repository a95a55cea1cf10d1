"""torchrun case: P pipeline stages (gloo / nccl p2p) reproduce the single-process loss and gradients."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from trainscale_b200.models.llama import LlamaConfig, build_model  # noqa: E402
from trainscale_b200.parallel import pp as PP  # noqa: E402


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
    cfg = LlamaConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=4,
                      num_attention_heads=2, num_key_value_heads=2, head_dim=64)
    B, S, M = 4, (256 if cuda else 32), 4
    ok = True
    for sched in ("gpipe", "1f1b", "zero_bubble"):
        ref = build_model(cfg, dtype=dtype, device=dev, seed=9)
        full = build_model(cfg, dtype=dtype, device=dev, seed=9)
        stage = PP.split_model_into_stages(full, world, rank)
        rt = PP.PipelineRuntime(stage, rank, world, schedule=sched)
        ids = torch.randint(0, cfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(2)).to(dev)
        mbs = PP.split_into_microbatches({"input_ids": ids, "labels": ids}, M)
        loss = rt.train_step(mbs, (B // M, S, 2 * cfg.hidden_size), dtype, dev)
        # oracle: mean over micro-batches of the per-micro-batch mean loss
        rl = 0.0
        for mb in mbs:
            l = ref(mb["input_ids"], labels=mb["labels"]).loss / M
            l.backward()
            rl += l.item()
        tol = 3e-2 if cuda else 1e-4
        good = True
        if rank == world - 1:
            good &= abs(loss.item() - rl) < tol
        # compare the gradient of the first layer owned by this stage
        li = PP.split_layers(cfg.num_hidden_layers, world)[rank][0]
        g_ref = ref.model.layers[li].mlp.w_down.grad.float()
        g = stage.layers[0].mlp.w_down.grad.float()
        e = (g - g_ref).abs().max().item() / max(g_ref.abs().max().item(), 1e-9)
        good &= e < (5e-2 if cuda else 1e-4)
        ok &= good
        print(f"RESULT rank={rank} sched={sched} grad_err={e:.2e} loss={(loss.item() if loss is not None else None)} ref={rl:.5f} ok={good}", flush=True)
    flag = torch.tensor([0.0 if ok else 1.0], device=dev)
    dist.all_reduce(flag)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
