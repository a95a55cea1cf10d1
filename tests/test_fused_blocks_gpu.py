"""norm->linear / GLU->linear recompute blocks against the separate ops and an fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref_norm_linear(x, res, nw, w, eps):
    h = x.float() + (0 if res is None else res.float())
    h = h.to(torch.bfloat16).float()
    y = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * nw.float()
    return y.to(torch.bfloat16).float() @ w.float().t(), h


@pytest.mark.parametrize("with_res", [False, True])
def test_norm_linear_matches_reference(with_res):
    from trainscale_b200.ops import fused_blocks
    torch.manual_seed(0)
    T, H, N = 512, 1024, 768
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    res = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True) if with_res else None
    nw = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(N, H, device="cuda") / H ** 0.5).to(torch.bfloat16).requires_grad_(True)
    out, h = fused_blocks.norm_linear(x, res, nw, w, 1e-5)
    gout, gh = torch.randn_like(out), torch.randn_like(h)
    (out.float() * gout.float()).sum().backward(retain_graph=True) if not with_res else \
        ((out.float() * gout.float()).sum() + (h.float() * gh.float()).sum()).backward()
    xr, nwr, wr = (t.detach().float().requires_grad_(True) for t in (x, nw, w))
    rr = res.detach().float().requires_grad_(True) if with_res else None
    hr = xr + (0 if rr is None else rr)
    yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-5) * nwr
    outr = yr @ wr.t()
    loss = (outr * gout.float()).sum() + ((hr * gh.float()).sum() if with_res else 0)
    loss.backward()

    def close(a, b, tol=3e-2):
        return (a.float() - b).abs().max().item() <= tol * max(b.abs().max().item(), 1.0)

    assert close(out, outr)
    assert close(x.grad, xr.grad)
    assert close(nw.grad, nwr.grad, 5e-2)
    assert close(w.grad, wr.grad)
    if with_res:
        assert close(res.grad, rr.grad)


def test_glu_linear_matches_reference():
    from trainscale_b200.ops import fused_blocks
    torch.manual_seed(1)
    T, I, N = 384, 1024, 512
    gu = torch.randn(T, 2 * I, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(N, I, device="cuda") / I ** 0.5).to(torch.bfloat16).requires_grad_(True)
    out = fused_blocks.glu_linear(gu, w, "silu")
    go = torch.randn_like(out)
    out.backward(go)
    gur, wr = gu.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    g, u = gur.chunk(2, -1)
    outr = (torch.nn.functional.silu(g) * u) @ wr.t()
    outr.backward(go.float())
    for a, b in ((out, outr), (gu.grad, gur.grad), (w.grad, wr.grad)):
        assert (a.float() - b).abs().max().item() <= 3e-2 * max(b.abs().max().item(), 1.0)


def test_decoder_layer_op_selective_equals_plain_path():
    from trainscale_b200.models.llama import LlamaConfig, LlamaForCausalLM
    torch.manual_seed(2)
    cfg = LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256)
    m = LlamaForCausalLM(cfg).cuda().to(torch.bfloat16).train()
    ids = torch.randint(0, 512, (2, 128), device="cuda")
    loss0 = m(input_ids=ids, labels=ids).loss
    loss0.backward()
    g0 = {n: p.grad.clone() for n, p in m.named_parameters()}
    m.zero_grad(set_to_none=True)
    m.op_selective_recompute(True)
    loss1 = m(input_ids=ids, labels=ids).loss
    loss1.backward()
    assert abs(loss0.item() - loss1.item()) < 1e-3
    for n, p in m.named_parameters():
        d = (p.grad.float() - g0[n].float()).abs().max().item()
        assert d <= 2e-2 * max(g0[n].float().abs().max().item(), 1e-3), n
