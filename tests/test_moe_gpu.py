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
