"""torchrun case: TP-sharded decoder (with and without sequence parallelism) == unsharded decoder (loss + grads)."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from trainscale_b200.models.llama import LlamaConfig, build_model  # noqa: E402
from trainscale_b200.parallel import tp as TP  # noqa: E402


def main():
    cuda = "--cuda" in sys.argv
    fused = "--fused" in sys.argv
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if cuda:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
        dev, dtype = torch.device("cuda", int(os.environ["LOCAL_RANK"])), torch.bfloat16
    else:
        dist.init_process_group("gloo")
        dev, dtype = torch.device("cpu"), torch.float32
    # heads, FFN width and sequence grow with the group so that every rank keeps whole heads and 128-row blocks
    cfg = LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=256 * max(2, world), num_hidden_layers=2,
                      num_attention_heads=max(4, world), num_key_value_heads=max(2, world), head_dim=64)
    S = 128 * max(2, world) if cuda else 32
    ok = True
    heap = None
    if fused:
        from trainscale_b200.parallel.symm import SymmetricHeap
        heap = SymmetricHeap.try_create(None, dev)
        assert heap is not None, "symmetric memory unavailable"
    for sp in (False, True):
        ref = build_model(cfg, dtype=dtype, device=dev, seed=5)
        mod = build_model(cfg, dtype=dtype, device=dev, seed=5)
        ctx = TP.TPContext.from_group(dist.group.WORLD, sequence_parallel=sp, comm="fused" if fused else "nccl", heap=heap)
        TP.shard_model_for_tensor_parallel(mod, ctx)
        ids = torch.randint(0, cfg.vocab_size, (1, S), generator=torch.Generator().manual_seed(1)).to(dev)
        rl = ref(ids, labels=ids).loss
        rl.backward()
        if sp:
            # token-sharded residual stream between blocks: embed, split tokens, run layers, gather before the head
            x = mod.model.embed_tokens(ids)
            x = TP.scatter_to_sequence_parallel_region(x.view(S, -1), ctx).view(1, S // world, -1)
            cos, sin = mod.model.rope_tables(dev, S)
            res = None
            for layer in mod.model.layers:
                x, res = layer(x, res, cos, sin)
            x, _ = mod.model.norm(x, res)
            x = TP._GatherFromSeqForLoss.apply(x.view(S // world, -1), ctx).view(1, S, -1) if hasattr(TP, "_GatherFromSeqForLoss") \
                else TP.all_gather_from_sequence_parallel_region(x.view(S // world, -1), ctx).view(1, S, -1)
            from trainscale_b200.ops import cross_entropy
            tgt = torch.full_like(ids, -100)
            tgt[:, :-1] = ids[:, 1:]
            loss, _ = cross_entropy.fused_linear_cross_entropy(x, mod.head_weight, tgt)
            # every rank computed the full loss on gathered tokens: the reduce-scatter in backward sums W copies
            (loss / world).backward()
            TP.allreduce_sequence_parallel_grads(mod, ctx)
        else:
            loss = mod(ids, labels=ids).loss
            loss.backward()
        tol = 3e-2 if cuda else 2e-4
        e_loss = abs(loss.item() - rl.item())
        # compare one sharded weight gradient and one replicated gradient
        I = cfg.intermediate_size // world
        g_ref = ref.model.layers[0].mlp.w_down.grad[:, rank * I:(rank + 1) * I].float()
        g_tp = mod.model.layers[0].mlp.inner.w_down.grad.float()
        e_w = (g_ref - g_tp).abs().max().item() / max(g_ref.abs().max().item(), 1e-9)
        gn_ref = ref.model.layers[1].input_layernorm.weight.grad.float()
        gn_tp = mod.model.layers[1].input_layernorm.weight.grad.float()
        e_n = (gn_ref - gn_tp).abs().max().item() / max(gn_ref.abs().max().item(), 1e-9)
        ge_ref = ref.model.embed_tokens.weight.grad.float()
        ge_tp = mod.model.embed_tokens.weight.grad.float()
        e_e = (ge_ref - ge_tp).abs().max().item() / max(ge_ref.abs().max().item(), 1e-9)
        good = e_loss < tol and e_w < max(tol, 5e-4) * 3 and e_n < max(tol, 5e-4) * 3 and e_e < max(tol, 5e-4) * 3
        ok &= good
        if rank == 0:
            print(f"RESULT sp={sp} fused={fused} loss_err={e_loss:.2e} w_err={e_w:.2e} norm_err={e_n:.2e} emb_err={e_e:.2e} ok={good}")
    if cuda:
        from trainscale_b200.ops import _lib
        torch.cuda.synchronize()
        _lib.raise_on_any_device_error()
    flag = torch.tensor([0.0 if ok else 1.0], device=dev)
    dist.all_reduce(flag)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
