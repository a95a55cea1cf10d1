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


# ------------------------------------------------------------------------------------------------ rowwise recipe
@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
def test_rowwise_and_colwise_quant_match_pytorch(fmt):
    from trainscale_b200.ops import fp8
    torch.manual_seed(0)
    fmax = {"e4m3": 448.0, "e5m2": 57344.0}[fmt]
    for R, C in [(257, 384), (64, 9216), (1000, 2056)]:
        x = torch.randn(R, C, device="cuda", dtype=torch.bfloat16) * torch.rand(R, 1, device="cuda").add(0.1).bfloat16()
        q, s = fp8.quant_rowwise(x, fmt)
        assert torch.allclose(s, x.float().abs().amax(1).clamp(min=1e-12) / fmax, rtol=1e-6)
        back = fp8.dequant_rowwise(q, s, 0)
        step = 2.0 ** (-3 if fmt == "e4m3" else -2)          # relative spacing of the format
        assert ((back - x.float()).abs() <= step * x.float().abs().amax(1, keepdim=True)).all()
        # the kernel multiplies by 1/s, the oracle divides: a value on a rounding boundary may land one step apart
        same = q.view(torch.uint8) == (x.float() / s.view(-1, 1)).to(q.dtype).view(torch.uint8)
        assert same.float().mean().item() > 0.995
        qc, sc = fp8.quant_colwise(x, fmt)
        assert torch.allclose(sc, x.float().abs().amax(0).clamp(min=1e-12) / fmax, rtol=1e-6)
        same = qc.view(torch.uint8) == (x.float() / sc.view(1, -1)).to(qc.dtype).view(torch.uint8)
        assert same.float().mean().item() > 0.995
        backc = fp8.dequant_rowwise(qc, sc, 1)
        assert ((backc - x.float()).abs() <= step * x.float().abs().amax(0, keepdim=True)).all()


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (304, 400, 528), (1008, 1072, 1040), (4096, 2048, 4096)])
def test_rowwise_gemm_all_layouts_match_fp32_on_the_same_fp8_values(M, N, K):
    """Forward (K-major x K-major), dgrad (K-major x MN-major) and wgrad (MN-major x MN-major) layouts, ragged shapes,
    against fp32 matmuls of the dequantised operands; bf16 and fp32 outputs, accumulation."""
    from trainscale_b200.ops import fp8, _lib
    torch.manual_seed(1)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
    aq, sa = fp8.quant_rowwise(a)
    bq, sb = fp8.quant_rowwise(b)
    ref = fp8.dequant_rowwise(aq, sa, 0) @ fp8.dequant_rowwise(bq, sb, 0).t()
    y = fp8.gemm_rowwise(aq, sa, bq, sb, M, N, K)
    tol = 1e-2 * max(ref.abs().max().item(), 1.0)
    assert (y.float() - ref).abs().max().item() <= tol
    y32 = torch.ones(M, N, device="cuda", dtype=torch.float32)
    fp8.gemm_rowwise(aq, sa, bq, sb, M, N, K, out=y32, accumulate=True)
    assert (y32 - 1.0 - ref).abs().max().item() <= 1e-3 * max(ref.abs().max().item(), 1.0)
    # B stored [K][N] (MN-major), column scales: c[m][n] = sum_k a[m][k] bt[k][n]
    bt = (torch.randn(K, N, device="cuda") / K ** 0.5).to(torch.bfloat16)
    btq, sbt = fp8.quant_colwise(bt, "e4m3")
    ref2 = fp8.dequant_rowwise(aq, sa, 0) @ fp8.dequant_rowwise(btq, sbt, 1)
    y2 = fp8.gemm_rowwise(aq, sa, btq, sbt, M, N, K, b_mn=True)
    assert (y2.float() - ref2).abs().max().item() <= 1e-2 * max(ref2.abs().max().item(), 1.0)
    # both operands MN-major (wgrad): c[m][n] = sum_k at[k][m] bt[k][n], A in E5M2
    at = torch.randn(K, M, device="cuda", dtype=torch.bfloat16)
    atq, sat = fp8.quant_colwise(at, "e5m2")
    ref3 = fp8.dequant_rowwise(atq, sat, 1).t() @ fp8.dequant_rowwise(btq, sbt, 1)
    y3 = fp8.gemm_rowwise(atq, sat, btq, sbt, M, N, K, a_mn=True, b_mn=True)
    assert (y3.float() - ref3).abs().max().item() <= 1e-2 * max(ref3.abs().max().item(), 1.0)
    torch.cuda.synchronize()
    assert _lib.device_error("fp8_rowwise")[0] == 0


@pytest.mark.parametrize("grad_fmt,tol", [("e4m3", 0.06), ("e5m2", 0.12)])
def test_fp8_rowwise_linear_forward_and_backward(grad_fmt, tol):
    from trainscale_b200.ops import fp8
    torch.manual_seed(2)
    M, N, K = 512, 768, 1024
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(N, K, device="cuda") / K ** 0.5).to(torch.bfloat16).requires_grad_(True)
    w.main_grad = torch.zeros(N, K, device="cuda", dtype=torch.float32)     # the engine's gradient buffer
    w.grad_added = False
    y = fp8.fp8_linear(x, w, recipe="rowwise", grad_format=grad_fmt)
    dy = torch.randn_like(y)
    y.backward(dy)
    assert w.grad is None and w.grad_added
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = xr @ wr.t()
    yr.backward(dy.float())
    assert (y.float() - yr).abs().mean().item() <= 0.05 * yr.abs().mean().item()
    for a, b in ((x.grad, xr.grad), (w.main_grad, wr.grad)):
        assert (a.float() - b).abs().mean().item() <= tol * b.abs().mean().item() + 1e-3
        assert (a.float() - b).abs().max().item() <= 3 * tol * b.abs().max().item()


def test_decoder_trains_with_fp8_rowwise_and_e5m2_gradients():
    from trainscale_b200.models.llama import LlamaConfig, build_model
    from trainscale_b200.parallel.flat_engine import EngineConfig, FlatShardedEngine
    cfg = LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64)
    model = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=0)
    model.enable_fp8(True, recipe="rowwise", grad_format="e5m2")
    eng = FlatShardedEngine(model, EngineConfig(lr=3e-3, weight_decay=0.0), device=torch.device("cuda"))
    ids = torch.randint(0, 512, (4, 256), device="cuda", generator=torch.Generator("cuda").manual_seed(0))
    losses = []
    for _ in range(8):
        out = model(ids, labels=ids)
        eng.backward(out.loss)
        eng.step()
        losses.append(float(out.loss.detach()))
    assert losses[-1] < losses[0] - 0.5, losses
