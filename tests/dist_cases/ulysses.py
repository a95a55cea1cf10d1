"""torchrun case (gloo): all-to-all (Ulysses) sequence-parallel attention == full attention, forward and backward."""
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from trainscale_b200.ops.attention import attention_reference  # noqa: E402
from trainscale_b200.parallel.cp import ulysses_attention  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, P = dist.get_rank(), dist.get_world_size()
    B, S, Hq, Hkv, D = 2, 8 * P, 4 * P, 2 * P, 16
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(B, S, h, D, generator=g) for h in (Hq, Hkv, Hkv))
    w = torch.randn(B, S, Hq, D, generator=g)
    sl = slice(rank * S // P, (rank + 1) * S // P)
    ok = True
    for causal, window in ((True, None), (False, None), (True, 5)):
        ql, kl, vl = (t[:, sl].clone().requires_grad_(True) for t in (q, k, v))
        out = ulysses_attention(ql, kl, vl, dist.group.WORLD, causal=causal, window=window)
        (out * w[:, sl]).sum().backward()
        qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
        ref = attention_reference(qf, kf, vf, causal, None, window)
        (ref * w).sum().backward()
        errs = [float((out - ref[:, sl]).abs().max()), float((ql.grad - qf.grad[:, sl]).abs().max()),
                float((kl.grad - kf.grad[:, sl]).abs().max()), float((vl.grad - vf.grad[:, sl]).abs().max())]
        good = max(errs) < 1e-4
        ok &= good
        if rank == 0:
            print(f"causal={causal} window={window}: errs={[f'{e:.1e}' for e in errs]} ok={good}", flush=True)
    flag = torch.tensor([0.0 if ok else 1.0])
    dist.all_reduce(flag)
    if rank == 0:
        print(f"RESULT ok={flag.item() == 0}")
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
