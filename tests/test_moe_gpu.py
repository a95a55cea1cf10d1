"""Grouped expert GEMM path (device-side plan, permute, grouped tcgen05 GEMMs, weighted combine) against the
per-expert loop in fp32."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(x, ids, w, wgu, wd):
    T, k = ids.shape
    out = torch.zeros(T, x.shape[1], dtype=torch.float32, device=x.device)
    for t_slot in range(k):
        for e in range(wgu.shape[0]):
            sel = ids[:, t_slot] == e
            if sel.any():
                h = x[sel].float() @ wgu[e].float().t()
                g, u = h.chunk(2, -1)
                y = (torch.nn.functional.silu(g) * u) @ wd[e].float().t()
                out[sel] += w[sel, t_slot].float().unsqueeze(1) * y
    return out


@pytest.mark.parametrize("T,H,I,E,k", [(300, 256, 384, 4, 2), (1024, 512, 256, 8, 2), (77, 128, 128, 16, 1),
                                       (2048, 256, 512, 3, 2)])
def test_moe_ffn_matches_expert_loop(T, H, I, E, k):
    from trainscale_b200.ops import moe, _lib
    torch.manual_seed(0)
    dev = "cuda"
    x = torch.randn(T, H, device=dev, dtype=torch.bfloat16).requires_grad_(True)
    wgu = (torch.randn(E, 2 * I, H, device=dev) / H ** 0.5).to(torch.bfloat16).requires_grad_(True)
    wd = (torch.randn(E, H, I, device=dev) / I ** 0.5).to(torch.bfloat16).requires_grad_(True)
    logits = torch.randn(T, E, device=dev)
    if E >= 8:
        logits[:, 5] = -1e9          # an expert that receives no token
    w, ids = torch.softmax(logits, -1).topk(k, dim=-1)
    w = w.to(torch.bfloat16).requires_grad_(True)
    out = moe.moe_ffn(x, ids, w, wgu, wd)
    do = torch.randn_like(out)
    out.backward(do)
    torch.cuda.synchronize()
    assert _lib.device_error("gemm")[0] == 0
    xr, wr, gur, dr = (t.detach().float().requires_grad_(True) for t in (x, w, wgu, wd))
    ref = _reference(xr, ids, wr, gur, dr)
    ref.backward(do.float())

    def close(a, b, tol=3e-2):
        return (a.float() - b).abs().max().item() <= tol * max(b.abs().max().item(), 1.0)

    assert close(out, ref)
    assert close(x.grad, xr.grad)
    assert close(w.grad, wr.grad, 5e-2)
    assert close(wgu.grad, gur.grad)
    assert close(wd.grad, dr.grad)
    if E >= 8:
        assert wgu.grad[5].abs().max().item() == 0.0 and wd.grad[5].abs().max().item() == 0.0


def test_moe_layer_uses_grouped_path_and_matches_loop():
    from trainscale_b200.parallel.ep import ExpertParallelConfig, MoELayer
    torch.manual_seed(1)
    cfg = ExpertParallelConfig(num_experts=4, top_k=2, hidden_size=256, intermediate_size=256, drop_tokens=False)
    layer = MoELayer(cfg, dtype=torch.bfloat16, device="cuda")
    x = torch.randn(2, 96, 256, device="cuda", dtype=torch.bfloat16)
    y = layer(x)
    x2 = x.reshape(-1, 256)
    w, idx, _ = layer.router(x2)
    from trainscale_b200.parallel.ep import permute_tokens, unpermute_tokens
    xs, order, counts = permute_tokens(x2, idx, 4)
    ys = layer.experts(xs, counts.tolist())
    ref = unpermute_tokens(ys, order, w, x2.shape[0])
    for s in layer.shared:
        ref = ref + s(x2)
    assert (y.reshape(-1, 256).float() - ref.float()).abs().max().item() < 3e-2 * max(ref.float().abs().max().item(), 1.0)


@pytest.mark.parametrize("T,E,k,norm", [(300, 8, 2, True), (1000, 64, 6, True), (77, 160, 8, False), (512, 5, 1, True)])
def test_router_topk_softmax_kernel(T, E, k, norm):
    from trainscale_b200.ops import moe
    torch.manual_seed(0)
    logits = torch.randn(T, E, device="cuda", requires_grad=True)
    w, idx, probs = moe.topk_softmax(logits, k, norm)
    ref_l = logits.detach().clone().requires_grad_(True)
    rp = torch.softmax(ref_l, -1)
    rw, ridx = rp.topk(k, -1)
    if norm:
        rw = rw / rw.sum(-1, keepdim=True)
    assert torch.equal(idx, ridx)
    assert torch.allclose(w, rw, atol=1e-6) and torch.allclose(probs, rp, atol=1e-6)
    gw, gp = torch.randn_like(w), torch.randn_like(probs)
    ((w * gw).sum() + (probs * gp).sum()).backward()
    ((rw * gw).sum() + (rp * gp).sum()).backward()
    assert torch.allclose(logits.grad, ref_l.grad, atol=1e-5)


def test_batched_multi_adapter_lora_on_grouped_gemm():
    """Per-token adapter ids -> low-rank updates through the MoE plan + grouped GEMMs, against the per-adapter loop."""
    import copy
    from trainscale_b200.inference.multi_lora import BatchedLoRA
    from trainscale_b200.lora import get_peft_model, lora_state_dict
    from trainscale_b200.models.llama import LlamaConfig, build_model
    from trainscale_b200.ops import _lib
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=1, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=128)
    m = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=0)
    get_peft_model(m, r=16)
    adapters = {}
    for name in ("a", "b", "c"):
        for n, p in m.named_parameters():
            if "lora_" in n:
                p.data = (torch.randn(p.shape, device="cuda") * 0.1).to(p.dtype)
        adapters[name] = copy.deepcopy(lora_state_dict(m))
    bl = BatchedLoRA(m, adapters)
    T = 777
    x = torch.randn(T, 512, device="cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, 4, (T,), device="cuda")             # 3 = no adapter
    n0 = _lib.LAUNCHES
    got = bl.delta(0, "wqkv", x, ids)
    assert _lib.LAUNCHES > n0
    A, B = bl.weights[(0, "wqkv")]
    want = torch.zeros(T, B.shape[1], device="cuda")
    for a in range(3):
        sel = ids == a
        want[sel] = (x[sel].float() @ A[a].float().t()) @ B[a].float().t()
    assert float(got[ids == 3].abs().max()) == 0.0
    err = float((got.float() - want).abs().max()) / float(want.abs().max())
    assert err < 3e-2, err
    _lib.raise_on_any_device_error()


def test_moe_decoder_on_gpu_matches_expert_loop():
    """The mixture-of-experts decoder in bf16 on the GPU: grouped-GEMM path (routing plan, permute, grouped tcgen05
    GEMMs, combine) against the loop over experts on the SAME routing decisions (both use the router kernel's top-k, so
    near-ties in the router cannot send tokens to different experts in the two runs)."""
    from trainscale_b200.models.llama import build_model, preset_config
    from trainscale_b200.ops import _lib
    from trainscale_b200.ops import moe as moe_ops
    cfg = preset_config("moe-tiny", vocab_size=512, attention_bias=True, head_dim=64)
    ids = torch.randint(0, 512, (2, 256), generator=torch.Generator().manual_seed(0)).cuda()

    def run(use_kernels: bool):
        m = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=3)
        saved = moe_ops.available
        if not use_kernels:
            moe_ops.available = lambda x: False
        try:
            out = m(ids, labels=ids)
            out.loss.backward()
        finally:
            moe_ops.available = saved
        mlp = m.model.layers[0].mlp
        return float(out.loss), mlp.w_down.grad.float(), mlp.w_gate_up.grad.float(), m.model.layers[1].mlp.router.grad.float()

    n0 = _lib.LAUNCHES
    got = run(True)
    fast_launches = _lib.LAUNCHES - n0
    want = run(False)
    assert fast_launches > 20
    assert abs(got[0] - want[0]) < 2e-3 * want[0]
    # bf16 GEMMs with bf16 intermediates against fp32 maths on the same bf16 weights: small in norm, and no single
    # element far off
    errs = {}
    for name, g, w in zip(("w_down", "w_gate_up", "router"), got[1:], want[1:]):
        assert torch.isfinite(g).all()
        errs[name] = (float((g - w).norm()) / (float(w.norm()) + 1e-12),
                      float((g - w).abs().max()) / (float(w.abs().max()) + 1e-12))
    # the router's gradient is a difference of nearly equal dot products (normalised top-k weights), so the bf16
    # rounding of the expert outputs is amplified there; the expert weights see it directly
    assert errs["w_down"][0] < 4e-2 and errs["w_gate_up"][0] < 4e-2 and errs["router"][0] < 0.15, errs
    assert all(worst < 0.25 for _, worst in errs.values()), errs
    _lib.raise_on_any_device_error()


@pytest.mark.parametrize("W,T,H,I,E,k", [(2, 200, 256, 128, 4, 2), (4, 333, 128, 256, 8, 2), (4, 64, 256, 128, 16, 1)])
def test_expert_parallel_peer_kernels_with_virtual_ranks_on_one_gpu(W, T, H, I, E, k):
    """The dispatch / combine kernels of the peer-memory expert-parallel path, driven for W "ranks" whose buffers all
    live on this GPU (no kernel of that path waits on another, so running the ranks' launches one after the other in
    stream order stands in for the barriers).  Every rank's output must equal the expert loop over ALL experts on its
    own tokens; the scaled push followed by an unweighted pull must give back the pushed rows times the weight sum."""
    from trainscale_b200.ops import moe, _lib
    from trainscale_b200.parallel import ep_peer
    torch.manual_seed(1)
    dev = torch.device("cuda")
    El = E // W
    wgu = (torch.randn(E, 2 * I, H, device=dev) / H ** 0.5).to(torch.bfloat16)
    wd = (torch.randn(E, H, I, device=dev) / I ** 0.5).to(torch.bfloat16)
    xs, idss, ws = [], [], []
    for r in range(W):
        n_tok = T - 7 * r if r % 2 else T                   # the kernels do not need equal token counts
        xs.append(torch.randn(n_tok, H, device=dev, dtype=torch.bfloat16))
        logits = torch.randn(n_tok, E, device=dev)
        if E >= 8:
            logits[:, 3] = -1e9                             # an expert nobody routes to
        w, ids = torch.softmax(logits, -1).topk(k, dim=-1)
        ws.append((w / w.sum(-1, keepdim=True)).float().contiguous())
        idss.append(ids)
    cap = ep_peer.padded_rows(W * T * k, El)
    tables = [torch.zeros(W * E, dtype=torch.int32, device=dev) for _ in range(W)]
    xbufs = [torch.full((cap, H), float("nan"), dtype=torch.bfloat16, device=dev) for _ in range(W)]
    ybufs = [torch.full((cap, H), float("nan"), dtype=torch.bfloat16, device=dev) for _ in range(W)]
    arr = lambda ts: ep_peer._arr([t.data_ptr() for t in ts])   # noqa: E731
    t_ptrs, x_ptrs, y_ptrs = arr(tables), arr(xbufs), arr(ybufs)
    overflow = torch.zeros(1, dtype=torch.int32, device=dev)
    local = [ep_peer.local_ranks(idss[r], E) for r in range(W)]
    for r in range(W):
        ep_peer.counts_push(t_ptrs, local[r][2], r, W, E)
    routes = [ep_peer.make_route(tables[r], local[r][0], local[r][1], r, W, E, cap, idss[r].shape[0], k, overflow)
              for r in range(W)]
    for r in range(W):
        ep_peer.push_rows(x_ptrs, xs[r], routes[r], W, record_rows=True)
    outs = []
    for r in range(W):
        rt = routes[r]
        xr = ep_peer.finalize(xbufs[r], rt, H)
        h = moe.grouped_linear(xr, wgu[r * El:(r + 1) * El].contiguous(), rt.plan)
        from trainscale_b200.ops import activation
        y = moe.grouped_linear(activation.glu(h, "silu"), wd[r * El:(r + 1) * El].contiguous(), rt.plan)
        ep_peer.copy_used(y, ybufs[r], rt, H)
        # received rows per local expert = what all ranks routed there
        want_real = torch.stack([sum((idss[s] == r * El + l).sum() for s in range(W)) for l in range(El)])
        assert torch.equal(rt.seg_real.long(), want_real.long())
    for r in range(W):
        out, ys = ep_peer.pull_combine(y_ptrs, routes[r], H, W, ws[r].reshape(-1), True, dev)
        outs.append(out)
        assert ys.shape == (idss[r].numel(), H)
    torch.cuda.synchronize()
    assert int(overflow.item()) == 0
    for r in range(W):
        ref = _reference(xs[r], idss[r], ws[r], wgu, wd)
        err = (outs[r].float() - ref).abs().max().item()
        assert err <= 3e-2 * max(ref.abs().max().item(), 1.0), (r, err)
    # backward-direction moves: scaled push of g, then an unweighted pull of the same rows
    gs = [torch.randn_like(x) for x in xs]
    for r in range(W):
        ep_peer.push_rows(x_ptrs, gs[r], routes[r], W, scale=ws[r].reshape(-1))
    for r in range(W):
        dy = ep_peer.finalize(xbufs[r], routes[r], H)
        used = int(routes[r].plan.seg_start[-1].item())
        assert torch.isfinite(dy[:used].float()).all()          # pad rows were zeroed, real rows overwritten
        ep_peer.copy_used(dy, ybufs[r], routes[r], H)
    for r in range(W):
        back, _ = ep_peer.pull_combine(y_ptrs, routes[r], H, W, None, False, dev)
        want = gs[r].float() * ws[r].to(torch.bfloat16).float().sum(-1, keepdim=True)
        assert (back.float() - want).abs().max().item() <= 3e-2 * max(want.abs().max().item(), 1.0)
    torch.cuda.synchronize()
    _lib.raise_on_any_device_error()


def test_expert_parallel_block_on_the_peer_dispatcher_single_rank():
    """The whole autograd path of the peer-memory expert-parallel block (route, dispatch, grouped GEMMs, combine and
    their backward moves) in a one-rank process group, against the local block and the all-to-all block."""
    import subprocess
    import sys
    from pathlib import Path
    case = Path(__file__).parent / "dist_cases" / "ep_peer_equivalence.py"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=1", "--master-addr",
           "127.0.0.1", "--master-port", "29781", str(case)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "arm=peer" in r.stdout and "ok=False" not in r.stdout
