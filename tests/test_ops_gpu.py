"""Numerics of every sm_100a kernel against plain PyTorch fp32 math (small, odd and benchmark-like shapes)."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_err(got, ref):
    ref = ref.float()
    return (got.float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)


@pytest.fixture(autouse=True)
def _no_device_errors():
    yield
    from trainscale_b200.ops import _lib
    torch.cuda.synchronize()
    _lib.raise_on_any_device_error()


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (512, 384, 320), (1000, 520, 264), (2048, 4096, 1024)])
@pytest.mark.parametrize("bn", [0, 64, 128, 256])
def test_gemm_nt(M, N, K, bn):
    from trainscale_b200.ops import gemm
    torch.manual_seed(0)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    c = gemm.matmul_nt(a, b, bn=bn)
    assert rel_err(c, a.float() @ b.float().t()) < 1e-2


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (1000, 520, 264), (4096, 1024, 2048)])
def test_gemm_layouts_and_accumulate(M, N, K):
    from trainscale_b200.ops import gemm
    torch.manual_seed(1)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    bt = torch.randn(K, N, device=DEV, dtype=torch.bfloat16)
    assert rel_err(gemm.matmul_nn(a, bt), a.float() @ bt.float()) < 1e-2
    at = a.t().contiguous()
    assert rel_err(gemm.matmul_tn(at, bt), at.float().t() @ bt.float()) < 1e-2
    acc = torch.ones(M, N, device=DEV, dtype=torch.float32)
    gemm.matmul_tn(at, bt, out=acc, accumulate=True, alpha=0.5)
    assert rel_err(acc, 0.5 * (at.float().t() @ bt.float()) + 1) < 1e-4
    accb = torch.ones(M, N, device=DEV, dtype=torch.bfloat16)
    gemm.matmul_nn(a, bt, out=accb, accumulate=True)
    assert rel_err(accb, a.float() @ bt.float() + 1) < 1e-2


@pytest.mark.parametrize("M,N,K", [(8000, 4104, 1024), (2560, 2056, 520), (8192, 4096, 3584), (304, 264, 200)])
def test_gemm_paired_cta_kernel_every_layout_against_fp32(M, N, K):
    """bn=512 selects the cluster-of-two 256 x 256 kernel explicitly: forward (NT), dgrad (NN) and wgrad (TN) operand
    layouts, M and N that are not multiples of 256 (partial tiles on both edges), K with a tail, fp32 accumulation."""
    from trainscale_b200.ops import gemm
    torch.manual_seed(5)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    assert rel_err(gemm.matmul_nt(a, b, bn=512), ref) < 1e-2
    bt = b.t().contiguous()                                         # [K, N]: MN-major B
    assert rel_err(gemm.matmul_nn(a, bt, bn=512), ref) < 1e-2
    at = a.t().contiguous()                                         # [K, M]: MN-major A
    assert rel_err(gemm.matmul_tn(at, bt, bn=512), ref) < 1e-2
    acc = torch.full((M, N), 2.0, device=DEV, dtype=torch.float32)
    gemm.matmul_tn(at, bt, out=acc, accumulate=True, alpha=0.25, bn=512)
    assert rel_err(acc, 0.25 * ref + 2) < 1e-4
    # the default policy must pick the same kernel for the large shapes and agree bit for bit with the explicit choice
    if (M + 255) // 256 * ((N + 255) // 256) >= 74:
        assert torch.equal(gemm.matmul_nt(a, b), gemm.matmul_nt(a, b, bn=512))


def test_linear_autograd_matches_torch():
    from trainscale_b200.ops import gemm
    torch.manual_seed(2)
    x = torch.randn(3, 100, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(384, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = gemm.linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = F.linear(xr, wr)
    yr.backward(g.float())
    assert rel_err(y, yr) < 1e-2 and rel_err(x.grad, xr.grad) < 1e-2 and rel_err(w.grad, wr.grad) < 1e-2


@pytest.mark.parametrize("rows,H", [(7, 256), (300, 4096), (65, 1000 // 8 * 8), (33, 8192)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm_fwd_bwd(rows, H, with_res):
    from trainscale_b200.ops import norm
    torch.manual_seed(3)
    x = torch.randn(rows, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16).requires_grad_()
    res = torch.randn(rows, H, device=DEV, dtype=torch.bfloat16, requires_grad=True) if with_res else None
    y, r = norm.rmsnorm(x, w, 1e-5, res)
    gy, gr = torch.randn_like(y), torch.randn_like(y)
    (y.float() * gy.float()).sum().add((r.float() * gr.float()).sum()).backward()
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    rr = res.detach().float().requires_grad_() if with_res else None
    h = xr if rr is None else (xr + rr).detach().to(torch.bfloat16).float() + ((xr + rr) - (xr + rr).detach())
    yr = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    ((yr * gy.float()).sum() + (h * gr.float()).sum()).backward()
    assert rel_err(y, yr) < 1e-2
    assert rel_err(x.grad, xr.grad) < 2e-2
    assert rel_err(w.grad, wr.grad) < 2e-2
    if with_res:
        assert rel_err(res.grad, rr.grad) < 2e-2


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("with_pos", [False, True])
def test_rope_forward_backward(interleaved, with_pos):
    from trainscale_b200.ops import rope
    torch.manual_seed(4)
    B, S, Hq, Hkv, D = 2, 96, 4, 2, 64
    cos, sin = rope.rope_tables(256, D, 10000.0, DEV)
    qkv = torch.randn(B, S, (Hq + 2 * Hkv) * D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    pos = torch.randint(0, 256, (B, S), device=DEV) if with_pos else None
    out = rope.apply_rope_qkv(qkv, Hq + Hkv, D, cos, sin, pos, S, 3 if not with_pos else 0, interleaved)
    g = torch.randn_like(out)
    out.backward(g)
    positions = pos.reshape(-1) if with_pos else (torch.arange(B * S, device=DEV) % S) + 3
    x = qkv.detach().float().requires_grad_()
    rot = rope._rope_reference(x.view(B * S, -1)[:, :(Hq + Hkv) * D].reshape(B * S, Hq + Hkv, D), cos, sin, positions,
                               interleaved, 1.0)
    ref = torch.cat((rot.reshape(B * S, -1), x.view(B * S, -1)[:, (Hq + Hkv) * D:]), dim=-1).view_as(x)
    ref.backward(g.float())
    assert rel_err(out, ref) < 1e-2 and rel_err(qkv.grad, x.grad) < 1e-2


@pytest.mark.parametrize("act", ["silu", "gelu", "gelu_tanh"])
def test_glu(act):
    from trainscale_b200.ops import activation
    torch.manual_seed(5)
    gu = torch.randn(130, 2 * 344, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = activation.glu(gu, act)
    g = torch.randn_like(y)
    y.backward(g)
    x = gu.detach().float().requires_grad_()
    a, u = x.chunk(2, -1)
    ref = (F.silu(a) if act == "silu" else F.gelu(a, approximate="tanh" if act == "gelu_tanh" else "none")) * u
    ref.backward(g.float())
    assert rel_err(y, ref) < 1e-2 and rel_err(gu.grad, x.grad) < 2e-2


@pytest.mark.parametrize("T,V,chunk", [(100, 1000, 64), (513, 32000, 256), (64, 128256, 64)])
@pytest.mark.parametrize("smoothing,softcap", [(0.0, 0.0), (0.1, 30.0)])
def test_fused_linear_cross_entropy(T, V, chunk, smoothing, softcap):
    from trainscale_b200.ops import cross_entropy as ce
    torch.manual_seed(6)
    H = 256
    h = (0.5 * torch.randn(T, H, device=DEV)).to(torch.bfloat16).requires_grad_()
    w = (0.05 * torch.randn(V, H, device=DEV)).to(torch.bfloat16).requires_grad_()
    labels = torch.randint(0, V, (T,), device=DEV)
    labels[::7] = -100
    loss, count = ce.fused_linear_cross_entropy(h, w, labels, -100, smoothing, 1.0, softcap, chunk)
    loss.backward()
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lr_, cr = ce.linear_cross_entropy_reference(hr, wr, labels, -100, smoothing, 1.0, softcap)
    lr_.backward()
    assert count.item() == cr.item()
    assert abs(loss.item() - lr_.item()) < 2e-2 * max(1.0, abs(lr_.item()))
    assert rel_err(h.grad, hr.grad) < 3e-2 and rel_err(w.grad, wr.grad) < 3e-2


def test_token_logprobs():
    from trainscale_b200.ops import cross_entropy as ce
    torch.manual_seed(7)
    T, H, V = 200, 128, 5000
    h = (0.5 * torch.randn(T, H, device=DEV)).to(torch.bfloat16).requires_grad_()
    w = (0.05 * torch.randn(V, H, device=DEV)).to(torch.bfloat16).requires_grad_()
    labels = torch.randint(0, V, (T,), device=DEV)
    labels[:10] = -100
    lp = ce.fused_linear_token_logprobs(h, w, labels, -100, 64)
    g = torch.randn_like(lp)
    lp.backward(g)
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    ref = torch.log_softmax(hr @ wr.t(), -1).gather(1, labels.clamp(min=0)[:, None]).squeeze(1)
    ref = torch.where(labels == -100, torch.zeros_like(ref), ref)
    ref.backward(g)
    assert (lp - ref).abs().max().item() < 3e-2
    assert rel_err(h.grad, hr.grad) < 3e-2 and rel_err(w.grad, wr.grad) < 3e-2


@pytest.mark.parametrize("B,S,Hq,Hkv,D,causal", [(1, 256, 1, 1, 128, False), (2, 512, 4, 2, 128, True),
                                                 (1, 200, 2, 2, 128, True), (2, 1024, 4, 1, 64, True),
                                                 (1, 1000, 2, 2, 64, False)])
def test_flash_attention_fwd_bwd(B, S, Hq, Hkv, D, causal):
    from trainscale_b200.ops import flash
    from trainscale_b200.ops.attention import _split_qkv, attention_reference
    torch.manual_seed(8)
    qkv = torch.randn(B, S, (Hq + 2 * Hkv) * D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    o = flash.flash_attention_qkv(qkv, Hq, Hkv, D, causal)
    g = torch.randn_like(o)
    o.backward(g)
    x = qkv.detach().float().requires_grad_()
    q, k, v = _split_qkv(x, Hq, Hkv, D)
    ref = attention_reference(q, k, v, causal).reshape(B, S, Hq * D)
    ref.backward(g.float())
    assert rel_err(o, ref) < 2e-2
    for a, b in zip(qkv.grad.split((Hq * D, Hkv * D, Hkv * D), -1), x.grad.split((Hq * D, Hkv * D, Hkv * D), -1)):
        assert rel_err(a, b) < 2e-2


def test_flash_attention_packed_documents():
    from trainscale_b200.ops import flash
    from trainscale_b200.ops.attention import _split_qkv, attention_reference
    torch.manual_seed(9)
    B, S, Hq, Hkv, D = 1, 1024, 2, 1, 128
    cu = torch.tensor([0, 100, 356, 1000, 1024], device=DEV, dtype=torch.int32)
    qkv = torch.randn(B, S, (Hq + 2 * Hkv) * D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    o = flash.flash_attention_qkv(qkv, Hq, Hkv, D, True, None, cu, S)
    g = torch.randn_like(o)
    o.backward(g)
    x = qkv.detach().float().requires_grad_()
    q, k, v = _split_qkv(x, Hq, Hkv, D)
    doc = torch.bucketize(torch.arange(S, device=DEV), cu[1:].long(), right=True).view(B, S)
    ref = attention_reference(q, k, v, True, doc_ids=doc).reshape(B, S, Hq * D)
    ref.backward(g.float())
    assert rel_err(o, ref) < 2e-2 and rel_err(qkv.grad, x.grad) < 2e-2


def test_adamw_flat_matches_torch():
    from trainscale_b200.ops import optim
    torch.manual_seed(10)
    n = 100003
    p = torch.randn(n, device=DEV)
    ref = p.clone().requires_grad_()
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    lowp = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    for step in range(1, 4):
        g = torch.randn(n, device=DEV).to(torch.bfloat16)
        optim.adamw_flat_(p, m, v, g, lowp, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
        ref.grad = g.float()
        opt.step()
    assert (p - ref.detach()).abs().max().item() < 1e-5
    assert (lowp.float() - p).abs().max().item() < 2e-2


def test_clip_coefficient_and_skip_flag():
    from trainscale_b200.ops import optim
    n = 4096
    p = torch.ones(n, device=DEV)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    g = torch.full((n,), 2.0, device=DEV)
    ss = torch.zeros(1, device=DEV)
    flag = torch.zeros(1, device=DEV)
    optim.sumsq_(ss, g, flag)
    assert abs(ss.item() - 4.0 * n) < 1e-2 * 4 * n and flag.item() == 0
    p2 = p.clone()
    optim.adamw_flat_(p2, m.clone(), v.clone(), g, None, lr=0.1, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0,
                      step=1, sumsq=ss, max_norm=1.0)
    assert torch.allclose(p2, torch.full_like(p2, 0.9), atol=1e-4)   # first Adam step moves by lr regardless of scale
    flag.fill_(1.0)
    p3 = p.clone()
    optim.adamw_flat_(p3, m, v, g, None, lr=0.1, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1,
                      skip_flag=flag)
    assert torch.equal(p3, p)


def test_model_matches_reference_math_and_trains():
    """bf16 CUDA model vs the same weights run through the fp32 PyTorch paths."""
    from trainscale_b200.models.llama import LlamaConfig, build_model
    cfg = LlamaConfig(vocab_size=2048, hidden_size=256, intermediate_size=688, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64)
    m = build_model(cfg, dtype=torch.bfloat16, device=DEV, seed=0)
    ref = build_model(cfg, dtype=torch.float32, device="cpu", seed=0)
    ref.load_hf_state_dict({k: v.float().cpu() for k, v in m.to_hf_state_dict().items()})
    ids = torch.randint(0, 2048, (2, 256), device=DEV)
    out = m(ids, labels=ids)
    out.loss.backward()
    r = ref(ids.cpu(), labels=ids.cpu())
    r.loss.backward()
    assert abs(out.loss.item() - r.loss.item()) < 3e-2
    g1 = m.model.layers[0].mlp.w_down.grad.float().cpu()
    g2 = ref.model.layers[0].mlp.w_down.grad
    assert rel_err(g1, g2) < 6e-2


@pytest.mark.gpu
@pytest.mark.parametrize("rows,H,bias", [(64, 1024, True), (777, 4096, True), (33, 2048, False)])
def test_layernorm_fwd_bwd(rows, H, bias):
    from trainscale_b200.ops import norm
    torch.manual_seed(0)
    x = (torch.randn(rows, H, device="cuda") * 2 + 0.5).to(torch.bfloat16).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    b = (0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16).requires_grad_(True) if bias else None
    y = norm.layernorm(x, w, b, 1e-5)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    br = b.detach().float().requires_grad_(True) if bias else None
    yr = torch.nn.functional.layer_norm(xr, (H,), wr, br, 1e-5)
    yr.backward(dy.float())
    assert (y.float() - yr).abs().max().item() < 3e-2
    assert (x.grad.float() - xr.grad).abs().max().item() < 3e-2 * max(1.0, xr.grad.abs().max().item())
    assert (w.grad.float() - wr.grad).abs().max().item() < 2e-2 * max(1.0, wr.grad.abs().max().item())
    if bias:
        assert (b.grad.float() - br.grad).abs().max().item() < 2e-2 * max(1.0, br.grad.abs().max().item())


@pytest.mark.gpu
@pytest.mark.parametrize("S,Hq,Hkv,D,window,softcap", [
    (1024, 4, 2, 128, 256, 0.0), (1000, 2, 2, 64, 100, 0.0), (768, 4, 1, 128, 0, 30.0), (896, 2, 1, 128, 300, 50.0),
    (512, 2, 2, 128, 1, 0.0)])
def test_flash_window_softcap_fwd_bwd(S, Hq, Hkv, D, window, softcap):
    from trainscale_b200.ops import flash, _lib
    from trainscale_b200.ops.attention import attention_reference, _split_qkv
    torch.manual_seed(0)
    B = 2
    qkv = torch.randn(B, S, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
    o = flash.flash_attention_qkv(qkv, Hq, Hkv, D, True, None, None, None, window, softcap)
    do = torch.randn_like(o)
    o.backward(do)
    torch.cuda.synchronize()
    assert _lib.device_error("attention")[0] == 0
    q2 = qkv.detach().float().requires_grad_(True)
    q, k, v = _split_qkv(q2, Hq, Hkv, D)
    ref = attention_reference(q, k, v, True, None, window or None, softcap).reshape(B, S, Hq * D)
    ref.backward(do.float())
    assert (o.float() - ref).abs().max().item() < 3e-2
    sizes = [Hq * D, Hkv * D, Hkv * D]
    for a, b_ in zip(qkv.grad.split(sizes, -1), q2.grad.split(sizes, -1)):
        assert (a.float() - b_).abs().max().item() < 3e-2 * max(b_.abs().max().item(), 1.0)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,V,gamma", [(64, 1024, 2.0), (333, 32000, 1.5), (128, 128256, 2.0)])
def test_focal_loss_on_ce_kernel(rows, V, gamma):
    from trainscale_b200.losses import FocalLoss
    torch.manual_seed(0)
    logits = (torch.randn(rows, V, device="cuda") * 2).to(torch.bfloat16).requires_grad_(True)
    labels = torch.randint(0, V, (rows,), device="cuda")
    labels[::7] = -100
    fl = FocalLoss(gamma=gamma, alpha=0.25)
    loss = fl(logits, labels)
    loss.backward()
    ref_l = logits.detach().float().requires_grad_(True)
    valid = labels != -100
    logp = torch.log_softmax(ref_l[valid], -1).gather(1, labels[valid].unsqueeze(1)).squeeze(1)
    ref = (0.25 * -((1 - logp.exp()) ** gamma) * logp).mean()
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-3 * max(1.0, abs(ref.item()))
    err = (logits.grad.float() - ref_l.grad).abs().max().item()
    assert err < 3e-2 * max(ref_l.grad.abs().max().item(), 1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["silu", "gelu", "gelu_tanh"])
def test_plain_activation_kernel(name):
    from trainscale_b200.ops import activation
    torch.manual_seed(0)
    x = (torch.randn(513, 1024, device="cuda") * 2).to(torch.bfloat16).requires_grad_(True)
    y = activation.act(x, name)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_(True)
    yr = F.silu(xr) if name == "silu" else F.gelu(xr, approximate="tanh" if name == "gelu_tanh" else "none")
    yr.backward(dy.float())
    assert (y.float() - yr).abs().max().item() < 3e-2
    assert (x.grad.float() - xr.grad).abs().max().item() < 5e-2


@pytest.mark.gpu
@pytest.mark.parametrize("rows,V,smoothing", [(257, 1000, 0.0), (512, 32000, 0.1), (64, 4099, 0.0)])
def test_fused_cross_entropy_loss_module_forward_backward(rows, V, smoothing):
    """FusedCrossEntropyLoss on materialised bf16 logits: loss and d(logits) from the row kernel against fp32 PyTorch."""
    from trainscale_b200.losses import FusedCrossEntropyLoss
    torch.manual_seed(0)
    logits = (torch.randn(rows, V, device="cuda") * 2).to(torch.bfloat16).requires_grad_(True)
    labels = torch.randint(0, V, (rows,), device="cuda")
    labels[::7] = -100
    loss = FusedCrossEntropyLoss(label_smoothing=smoothing)(logits, labels)
    loss.backward()
    ref_in = logits.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(ref_in, labels, ignore_index=-100, label_smoothing=smoothing)
    ref.backward()
    assert abs(float(loss) - float(ref)) < 2e-3 * max(1.0, abs(float(ref)))
    torch.testing.assert_close(logits.grad.float(), ref_in.grad, rtol=2e-2, atol=2e-5)
    assert float(logits.grad[::7].abs().max()) == 0.0


@pytest.mark.gpu
def test_lora_linear_with_epilogue_accumulation():
    """Base projection + adapters accumulated by the GEMM epilogue into column blocks of the fused output, against the
    two-step path (separate delta tensor) and an fp32 reference; gradients of x, A and B."""
    from trainscale_b200.lora import FusedLoRA, LoRALinear
    from trainscale_b200.ops import gemm
    torch.manual_seed(0)
    T, K, N1, N2, r = 512, 1024, 1024, 256, 16
    dev, dt = "cuda", torch.bfloat16
    x = torch.randn(T, K, device=dev, dtype=dt).requires_grad_(True)
    w = (torch.randn(N1 + N2, K, device=dev) / K ** 0.5).to(dt)
    parts = [LoRALinear(K, N1, r, row0=0, total_rows=N1 + N2, dtype=dt, device=dev),
             LoRALinear(K, N2, r, row0=N1, total_rows=N1 + N2, dtype=dt, device=dev)]
    for p in parts:
        torch.nn.init.normal_(p.lora_B, std=0.05)
    mod = FusedLoRA(parts)
    dy = torch.randn(T, N1 + N2, device=dev, dtype=dt)
    y = mod.linear(x, w)
    y.backward(dy)
    got = [x.grad.clone()] + [p.grad.clone() for p in mod.parameters()]
    x.grad = None
    mod.zero_grad()
    # fp32 reference
    xf = x.detach().float().requires_grad_(True)
    ps = [(p.lora_A.detach().float().requires_grad_(True), p.lora_B.detach().float().requires_grad_(True), p) for p in parts]
    yf = xf @ w.float().t()
    yf = yf + torch.cat([(xf @ A.t()) @ B.t() * p.scaling for A, B, p in ps], dim=1)
    yf.backward(dy.float())
    torch.testing.assert_close(y.float(), yf, rtol=2e-2, atol=2e-2)
    want = [xf.grad] + [t.grad for A, B, _ in ps for t in (A, B)]
    for g, wv in zip(got, want):
        err = float((g.float() - wv).abs().max()) / max(1e-6, float(wv.abs().max()))
        assert err < 3e-2, err
    # two-step path gives the same output up to bf16 rounding of the intermediate delta
    y2 = gemm.linear(x, w) + mod(x)
    torch.testing.assert_close(y.float(), y2.float(), rtol=2e-2, atol=3e-2)


@pytest.mark.gpu
def test_kernel_layer_entry_points_on_gpu():
    """The public kernel-layer functions route bf16 CUDA tensors to the sm_100a kernels (launch counter moves) and
    agree with fp32 PyTorch."""
    import torch.nn.functional as F
    import trainscale_b200.kernels as K
    from trainscale_b200.ops import _lib
    torch.manual_seed(0)
    dev, dt = "cuda", torch.bfloat16
    caps = K.get_kernel_capabilities()
    assert caps["tcgen05"] and caps["flash_attention"] and caps["fp8"] and caps["optimizer_kernels"]
    n0 = _lib.LAUNCHES
    x, r = torch.randn(512, 1024, device=dev, dtype=dt), torch.randn(512, 1024, device=dev, dtype=dt)
    w = (torch.rand(1024, device=dev) + 0.5).to(dt)
    xf, rf, wf = x.float(), r.float(), w.float()
    y, res = K.fused_add_rms_layernorm(x, r, w, return_residual=True)
    h = xf + rf
    torch.testing.assert_close(y.float(), h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-6) * wf, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(K.fused_softmax(x).float(), torch.softmax(xf, -1), rtol=2e-2, atol=1e-4)
    torch.testing.assert_close(K.swiglu_forward(x, r).float(), F.silu(xf) * rf, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(K.fused_gelu(x).float(), F.gelu(xf, approximate="tanh"), rtol=2e-2, atol=2e-2)
    logits = torch.randn(256, 4096, device=dev, dtype=dt)
    labels = torch.randint(0, 4096, (256,), device=dev)
    assert abs(float(K.fast_cross_entropy_loss(logits, labels)) - float(F.cross_entropy(logits.float(), labels))) < 5e-3
    q = torch.randn(1, 512, 8, 128, device=dev, dtype=dt)
    k, v = torch.randn(1, 512, 2, 128, device=dev, dtype=dt), torch.randn(1, 512, 2, 128, device=dev, dtype=dt)
    torch.testing.assert_close(K.flash_attention(q, k, v).float(), K.naive_attention(q.float(), k.float(), v.float()),
                               rtol=3e-2, atol=3e-2)
    from trainscale_b200.ops.attention import attention_reference
    torch.testing.assert_close(K.flash_attention(q, k, v, softcap=20.0, window_size=128).float(),
                               attention_reference(q.float(), k.float(), v.float(), True, None, 128, 20.0),
                               rtol=3e-2, atol=3e-2)
    a, b = torch.randn(512, 1024, device=dev, dtype=dt), (torch.randn(768, 1024, device=dev) / 32).to(dt)
    ref = a.float() @ b.float().t()
    got = K.fp8_matmul_block_scaled(a, b).float()
    assert float((got - ref).abs().max()) / float(ref.abs().max()) < 8e-2
    rep = K.validate_lora_gradients(T=256, hidden=512, out=768, r=16)
    assert rep["passed"], rep
    sm = torch.randn(64, 1000, device=dev, dtype=dt).requires_grad_(True)
    K.fused_softmax(sm)[:, 3].sum().backward()
    sf = sm.detach().float().requires_grad_(True)
    torch.softmax(sf, -1)[:, 3].sum().backward()
    torch.testing.assert_close(sm.grad.float(), sf.grad, rtol=3e-2, atol=1e-4)
    assert _lib.LAUNCHES - n0 >= 10
    _lib.raise_on_any_device_error()


@pytest.mark.gpu
def test_registry_patchers_route_a_huggingface_model_onto_the_kernels():
    """An unconverted transformers Llama in bf16 on the GPU: after `auto_patch` + `auto_patch_attention` its norms, gated
    MLPs, rotary embedding and attention run on the framework kernels (launch counter moves) and the logits stay within
    bf16 noise of the original modules."""
    transformers = pytest.importorskip("transformers")
    from trainscale_b200.ops import _lib
    from trainscale_b200.registry import auto_patch, auto_patch_attention
    torch.manual_seed(0)
    cfg = transformers.LlamaConfig(vocab_size=1024, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                                   num_attention_heads=8, num_key_value_heads=2, head_dim=64)
    m = transformers.LlamaForCausalLM(cfg).to("cuda", torch.bfloat16).eval()
    ids = torch.randint(0, 1024, (1, 256), device="cuda")
    with torch.no_grad():
        ref = m(ids).logits.float()
        counts = auto_patch(m)
        n_attn = auto_patch_attention(m)
        n0 = _lib.LAUNCHES
        out = m(ids).logits.float()
    assert counts["layernorm"] == 5 and counts["mlp"] == 2 and n_attn == 2
    assert _lib.LAUNCHES - n0 >= 10
    err = float((out - ref).abs().max()) / float(ref.abs().max())
    assert err < 5e-2, err
    _lib.raise_on_any_device_error()
