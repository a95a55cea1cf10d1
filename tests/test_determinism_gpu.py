"""Run-twice bitwise determinism of the kernels: the same inputs must give the same bits on every launch.  A kernel
whose blocks race on shared state, read a buffer before its producer finished, or depend on scheduling order shows up
here as a difference between two runs.  (The only kernel that is order-dependent by design is the squared-norm
reduction, which sums with floating-point atomics; it is checked to a tolerance.)"""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV, DT = "cuda", torch.bfloat16


def _twice(fn, n: int = 3):
    outs = [fn() for _ in range(n)]
    torch.cuda.synchronize()
    first = outs[0] if isinstance(outs[0], (tuple, list)) else (outs[0],)
    for o in outs[1:]:
        o = o if isinstance(o, (tuple, list)) else (o,)
        for a, b in zip(first, o):
            assert torch.equal(a, b), f"run-to-run difference, max |d| = {float((a.float() - b.float()).abs().max())}"


@pytest.mark.parametrize("M,N,K", [(4096, 4096, 4096), (8192, 6144, 4096), (300, 520, 264), (128, 128, 64)])
def test_gemm_is_deterministic(M, N, K):
    from trainscale_b200.ops import gemm
    torch.manual_seed(0)
    a = torch.randn(M, K, device=DEV, dtype=DT)
    b = torch.randn(N, K, device=DEV, dtype=DT)
    _twice(lambda: gemm.matmul_nt(a, b))
    _twice(lambda: gemm.matmul_tn(a, torch.randn(M, 64, device=DEV, dtype=DT, generator=torch.Generator(DEV).manual_seed(1))))


def test_attention_forward_backward_is_deterministic():
    from trainscale_b200.ops import attention
    torch.manual_seed(0)
    qkv = torch.randn(2, 1024, (8 + 2 * 2) * 128, device=DEV, dtype=DT)
    do = torch.randn(2, 1024, 8 * 128, device=DEV, dtype=DT)

    def run():
        x = qkv.clone().requires_grad_(True)
        o = attention.attention_qkv(x, 8, 2, 128, True)
        o.backward(do)
        return o.detach(), x.grad

    _twice(run)


def test_row_kernels_are_deterministic():
    from trainscale_b200.ops import activation, cross_entropy, norm
    torch.manual_seed(0)
    x = torch.randn(2048, 4096, device=DEV, dtype=DT)
    r = torch.randn(2048, 4096, device=DEV, dtype=DT)
    w = (torch.rand(4096, device=DEV) + 0.5).to(DT)
    dy = torch.randn(2048, 4096, device=DEV, dtype=DT)

    def rms():
        xx, ww = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        y, res = norm.rmsnorm(xx, ww, 1e-5, r)
        (y.float() * dy.float()).sum().backward()
        return y.detach(), res.detach(), xx.grad, ww.grad

    def ln():
        xx, ww = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        y = norm.layernorm(xx, ww, None, 1e-5)
        y.backward(dy)
        return y.detach(), xx.grad, ww.grad

    def glu():
        xx = torch.cat((x, r), -1).requires_grad_(True)
        y = activation.glu(xx, "silu")
        y.backward(dy)
        return y.detach(), xx.grad

    _twice(rms)
    _twice(ln)
    _twice(glu)
    logits = torch.randn(1024, 32000, device=DEV, dtype=DT)
    labels = torch.randint(0, 32000, (1024,), device=DEV)

    def ce():
        z = logits.clone().requires_grad_(True)
        rows = cross_entropy.cross_entropy_rows(z, labels)
        rows.sum().backward()
        return rows.detach(), z.grad

    _twice(ce)


def test_fused_lm_head_loss_moe_and_optimizer_are_deterministic():
    from trainscale_b200.ops import cross_entropy, moe
    from trainscale_b200.ops import optim as K
    torch.manual_seed(0)
    h = torch.randn(4096, 1024, device=DEV, dtype=DT)
    W = (torch.randn(8192, 1024, device=DEV) / 32).to(DT)
    tgt = torch.randint(0, 8192, (4096,), device=DEV)

    def head():
        hh, ww = h.clone().requires_grad_(True), W.clone().requires_grad_(True)
        loss, _ = cross_entropy.fused_linear_cross_entropy(hh, ww, tgt, chunk_tokens=1024)
        loss.backward()
        return loss.detach(), hh.grad, ww.grad

    _twice(head)
    x = torch.randn(1500, 512, device=DEV, dtype=DT)
    ids = torch.randint(0, 8, (1500, 2), device=DEV, dtype=torch.int32)
    wts = torch.softmax(torch.randn(1500, 2, device=DEV), -1).to(DT)
    wgu = (torch.randn(8, 1024, 512, device=DEV) / 23).to(DT)
    wd = (torch.randn(8, 512, 512, device=DEV) / 23).to(DT)

    def ffn():
        xx, a, b = x.clone().requires_grad_(True), wgu.clone().requires_grad_(True), wd.clone().requires_grad_(True)
        y = moe.moe_ffn(xx, ids, wts, a, b)
        y.float().pow(2).sum().backward()
        return y.detach(), xx.grad, a.grad, b.grad

    _twice(ffn)
    n = 1 << 22
    g = torch.randn(n, device=DEV, dtype=DT)

    def adamw():
        master = torch.linspace(-1, 1, n, device=DEV)
        m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
        low = torch.empty(n, device=DEV, dtype=DT)
        for step in (1, 2):
            K.adamw_flat_(master, m, v, g, low, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
        return master, m, v, low

    _twice(adamw)
    # the one order-dependent reduction: floating-point atomics, equal to a tolerance only
    outs = []
    for _ in range(3):
        s = torch.zeros(1, device=DEV)
        K.sumsq_(s, g)
        outs.append(float(s))
    assert max(outs) - min(outs) <= 1e-5 * max(outs)
