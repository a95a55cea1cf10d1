"""Optimizer step kernels (csrc/optim.cu) against the same optimizer class stepping fp32 / bf16 copies on the CPU
(the plain PyTorch formulas), over several steps so that the state carried between steps is covered too."""
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(300, 257), (5000,), (64, 1024), (33, 127)]      # the last one: element count not a multiple of 4


def _pair(dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    cpu = [torch.randn(s, generator=g).to(dtype).requires_grad_(True) for s in SHAPES]
    gpu = [p.detach().clone().cuda().requires_grad_(True) for p in cpu]
    return cpu, gpu


def _set_grads(cpu, gpu, step, grad_dtype):
    g = torch.Generator().manual_seed(100 + step)
    for pc, pg in zip(cpu, gpu):
        gr = (torch.randn(pc.shape, generator=g) * (0.5 + 0.1 * step)).to(grad_dtype)
        pc.grad = gr.clone()
        pg.grad = gr.cuda()


def _run(cls, kw, dtype, steps=4, before_step=None):
    from trainscale_b200.ops import _lib
    cpu, gpu = _pair(dtype)
    oc, og = cls(cpu, **kw), cls(gpu, **kw)
    n0 = _lib.LAUNCHES
    for s in range(steps):
        _set_grads(cpu, gpu, s, dtype)
        if before_step is not None:
            before_step(oc), before_step(og)
        oc.step(), og.step()
    torch.cuda.synchronize()
    assert _lib.LAUNCHES > n0, "the CUDA optimizer kernels did not run"
    _lib.raise_on_device_error("optim")
    return cpu, gpu, oc, og


def _close(cpu, gpu, dtype, rtol=2e-4, atol=2e-5):
    if dtype == torch.bfloat16:
        rtol, atol = 1.6e-2, 1e-3     # one bf16 ulp: an fp32 difference in the last bit can flip the rounding
    for pc, pg in zip(cpu, gpu):
        torch.testing.assert_close(pg.detach().cpu().float(), pc.detach().float(), rtol=rtol, atol=atol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name,kw", [
    ("LAMB", dict(lr=1e-2, weight_decay=0.01)),
    ("SophiaG", dict(lr=1e-2, rho=0.05, weight_decay=0.1)),
    ("ScheduleFreeAdamW", dict(lr=1e-2, weight_decay=0.01, warmup_steps=2)),
    ("ADOPT", dict(lr=1e-2, weight_decay=0.01)),
    ("AdaFactor", dict(lr=None)),
    ("AdaFactor", dict(lr=1e-2, beta1=0.9, weight_decay=0.01, scale_parameter=False, relative_step=False)),
])
def test_optimizer_kernels_match_reference_math(name, kw, dtype):
    import trainscale_b200.optim as O
    before = (lambda o: o.update_hessian(batch_size=4)) if name == "SophiaG" else None
    cpu, gpu, oc, og = _run(getattr(O, name), kw, dtype, before_step=before)
    _close(cpu, gpu, dtype)
    # fp32 moments carried between the steps agree as well
    for pc, pg in zip(cpu, gpu):
        for key in ("m", "v", "h", "z", "row", "col"):
            if key in oc.state[pc] and torch.is_tensor(oc.state[pc][key]) and dtype == torch.float32:
                torch.testing.assert_close(og.state[pg][key].cpu(), oc.state[pc][key], rtol=1e-3, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("block", [256, 2048])
def test_adam8bit_kernel(dtype, block):
    import trainscale_b200.optim as O
    kw = dict(lr=1e-2, weight_decay=0.01, block_size=block, min_8bit_size=1024)
    cpu, gpu, oc, og = _run(O.Adam8bit, kw, dtype, steps=3)
    for pc, pg in zip(cpu, gpu):
        # a value that lands within an ulp of a rounding tie may quantise one level apart: bounded, rare drift
        d = (pg.detach().cpu().float() - pc.detach().float()).abs()
        tol = 1.5e-3 if dtype == torch.float32 else 2e-2
        assert float(d.max()) < tol, float(d.max())
        sc, sg = oc.state[pc], og.state[pg]
        assert sg["m_q"].dtype == torch.int8 and sg["m_q"].shape == sc["m_q"].shape
        if dtype == torch.float32:
            assert float((d > 1e-5).float().mean()) < 1e-3
            lv = (sg["m_q"].cpu().int() - sc["m_q"].int()).abs()
            assert int(lv.max()) <= 1 and float((lv > 0).float().mean()) < 1e-3
            torch.testing.assert_close(sg["v_s"].cpu(), sc["v_s"], rtol=1e-4, atol=1e-9)


def test_quant8_roundtrip():
    from trainscale_b200.ops import optim as K
    from trainscale_b200.optim import _quantize_blockwise, _dequantize_blockwise
    x = torch.randn(3, 1000, device="cuda") * 3
    for block in K.QUANT_BLOCKS:
        q, s = K.quant8(x, block)
        qr, sr = _quantize_blockwise(x.cpu(), block)
        assert torch.equal(s.cpu(), sr)
        lv = (q.cpu().int() - qr.int()).abs()
        assert int(lv.max()) <= 1 and float((lv > 0).float().mean()) < 1e-4
        y = K.dequant8(q, s, x.shape, x.numel())
        torch.testing.assert_close(y.cpu(), _dequantize_blockwise(q.cpu(), sr, x.shape, x.numel()))
        assert float((y - x).abs().max()) <= float(s.max()) / 127 * 0.5 + 1e-6


@pytest.mark.parametrize("shape", [(256, 512), (768, 256), (1024, 1024)])
def test_newton_schulz_on_tcgen05_gemm(shape):
    """Muon's orthogonalisation in bf16 on the framework GEMM against the same iteration in fp32."""
    from trainscale_b200.optim import newton_schulz_orthogonalize
    torch.manual_seed(0)
    G = torch.randn(*shape, device="cuda")
    got = newton_schulz_orthogonalize(G, 5)
    assert got.dtype == torch.bfloat16 and got.shape == G.shape
    want = newton_schulz_orthogonalize(G.cpu(), 5)
    rel = float((got.float().cpu() - want).norm() / want.norm())
    assert rel < 4e-2, rel
    sv = torch.linalg.svdvals(got.float())
    # the quintic lands singular values in about [0.7, 1.2]; those that start near zero (square matrices) stay small
    assert float(sv.max()) < 1.4 and 0.6 < float(sv.median()) < 1.3
