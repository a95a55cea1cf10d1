"""fp8 quantisation kernels and the block-scaled tcgen05 GEMM against PyTorch fp32 math on the same fp8 values."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_quant_kernels_match_pytorch():
    from trainscale_b200.ops import fp8
    from trainscale_b200 import quantization as Q
    torch.manual_seed(0)
    w = torch.randn(300, 512, device="cuda", dtype=torch.bfloat16) * 3
    q, s = fp8.quant_block(w)
    qr, sr = Q.block_quantize_fp8(w)
    assert torch.allclose(s, sr, rtol=1e-6, atol=0)
    back, back_r = fp8.dequant(q, s, "block").float(), Q.block_dequantize_fp8(qr, sr).float()
    assert (back - back_r).abs().max().item() <= 0.07 * w.float().abs().max().item()   # at most one fp8 step apart
    assert (back - w.float()).abs().max().item() <= 0.07 * w.float().abs().max().item()
    x = torch.randn(257, 384, device="cuda", dtype=torch.bfloat16)
    xq, xs = fp8.quant_act(x)
    assert xs.shape == (3, 257)
    amax = x.float().view(257, 3, 128).abs().amax(-1).t() / 448.0
    assert torch.allclose(xs, amax.clamp(min=1e-12 / 448), rtol=1e-6)
    assert (fp8.dequant(xq, xs, "act").float() - x.float()).abs().max().item() <= 0.07 * x.float().abs().max().item()
    rq, rs = fp8.quant_row(x)
    assert (fp8.dequant(rq, rs, "row").float() - x.float()).abs().max().item() <= 0.07 * x.float().abs().max().item()


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (300, 384, 512), (1024, 1000, 1024), (4096, 4096, 4096)])
def test_fp8_gemm_forward(M, N, K):
    from trainscale_b200.ops import fp8, _lib
    torch.manual_seed(1)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
    xq, xs = fp8.quant_act(x)
    wq, ws = fp8.quant_block(w)
    y = fp8.gemm_fp8(xq, xs, wq, ws, N)
    torch.cuda.synchronize()
    assert _lib.device_error("fp8")[0] == 0
    ref = fp8.dequant(xq, xs, "act").float() @ fp8.dequant(wq, ws, "block").float().t()
    # the oracle's operands were rounded to bf16 after dequantisation: allow that much
    assert (y.float() - ref).abs().max().item() <= 2e-2 * max(ref.abs().max().item(), 1.0)
    full = x.float() @ w.float().t()
    assert (y.float() - full).abs().mean().item() <= 0.05 * full.abs().mean().item() + 1e-3


def test_fp8_linear_backward():
    from trainscale_b200.ops import fp8
    torch.manual_seed(2)
    M, N, K = 512, 768, 1024
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(N, K, device="cuda") / K ** 0.5).to(torch.bfloat16).requires_grad_(True)
    y = fp8.fp8_linear(x, w)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    (xr @ wr.t()).backward(dy.float())
    for a, b, tol in ((x.grad, xr.grad, 0.08), (w.grad, wr.grad, 0.03)):
        assert (a.float() - b).abs().mean().item() <= tol * b.abs().mean().item() + 1e-3
        assert (a.float() - b).abs().max().item() <= 0.15 * b.abs().max().item()


def test_fp8linear_module_uses_native_path():
    from trainscale_b200.quantization import FP8Linear
    torch.manual_seed(3)
    w = (torch.randn(256, 512, device="cuda") / 512 ** 0.5).to(torch.bfloat16)
    lin = FP8Linear(w).cuda()
    x = torch.randn(4, 64, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = lin(x)
    y.float().sum().backward()
    ref = x.detach().float() @ w.float().t()
    assert (y.float() - ref).abs().mean().item() <= 0.05 * ref.abs().mean().item() + 1e-3
    assert x.grad is not None and torch.isfinite(x.grad.float()).all()


def test_decoder_trains_with_fp8_projections():
    """enable_fp8(): layer projections on the fp8 kernel; loss tracks the bf16 model and goes down under training."""
    from trainscale_b200.models.llama import LlamaConfig, build_model
    from trainscale_b200.parallel.flat_engine import EngineConfig, FlatShardedEngine
    cfg = LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64)
    ref = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=0)
    m = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=0)
    m.enable_fp8(True)
    ids = torch.randint(0, 512, (4, 256), device="cuda", generator=torch.Generator(device="cuda").manual_seed(0))
    l_ref, l_fp8 = ref(ids, labels=ids).loss.item(), m(ids, labels=ids).loss.item()
    assert abs(l_ref - l_fp8) < 0.05 * l_ref
    eng = FlatShardedEngine(m, EngineConfig(lr=3e-3), device=torch.device("cuda"))
    losses = []
    for _ in range(8):
        loss = m(ids, labels=ids).loss
        eng.backward(loss)
        eng.step()
        losses.append(loss.item())
    assert all(l == l for l in losses) and losses[-1] < losses[0] - 0.3, losses
