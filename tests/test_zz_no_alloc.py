"""The allocation-free RMSNorm backward (`ts_rmsnorm_bwd_noalloc`, csrc/no_alloc.h) against the ordinary entry point.

Some users of the library cannot allocate device memory where they call it (a fixed memory budget, a host runtime
without PyTorch's allocator, a step audited to make no allocator calls), so this variant keeps its workspace inside
the library.  The test calls it through its exported C symbol, twice in a row with different inputs (the workspace
keeps the previous call's contents, which must not leak into the next result), and checks the size limit.
This file is named so that pytest collects it last.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _inputs(rows, H, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16, generator=g)
    dy = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16, generator=g)
    dres = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16, generator=g)
    w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).to(torch.bfloat16)
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
    return x, dy, dres, w, rstd


def _run_existing(lib, x, dy, dres, w, rstd):
    rows, H = x.shape
    parts = lib.ts_rmsnorm_bwd_parts(ctypes.c_longlong(rows))
    partial = torch.empty(parts, H, dtype=torch.float32, device="cuda")
    dx = torch.empty_like(x)
    dw = torch.empty(H, dtype=torch.float32, device="cuda")
    rc = lib.ts_rmsnorm_bwd(_ptr(dy), _ptr(x), _ptr(w), _ptr(rstd), _ptr(dres), _ptr(dx), _ptr(partial), _ptr(dw), None, 0,
                            ctypes.c_longlong(rows), H, ctypes.c_float(0.0),
                            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    return dx, dw


def _run_noalloc(lib, x, dy, dres, w, rstd, dx, dw):
    rows, H = x.shape
    return lib.ts_rmsnorm_bwd_noalloc(_ptr(dy), _ptr(x), _ptr(w), _ptr(rstd), _ptr(dres), _ptr(dx), _ptr(dw), None, 0,
                                      ctypes.c_longlong(rows), H, ctypes.c_float(0.0),
                                      ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_noalloc_entry_point_matches_existing_twice_in_a_row():
    from trainscale_b200.ops import _lib
    lib = _lib.load("elementwise")
    assert hasattr(lib, "ts_rmsnorm_bwd_noalloc")
    # outputs are allocated before the calls: the entry point itself must not need any allocation
    cases = [(_inputs(1000, 4096, 1)), (_inputs(333, 1024, 2))]
    outs = [(torch.empty_like(c[0]), torch.empty(c[0].shape[1], dtype=torch.float32, device="cuda")) for c in cases]
    # the set-up call (address look-up of the built-in workspace, lazy loading of the kernels) is made first, so the
    # driver-level free-memory figure below sees only what the two measured calls do
    (x, dy, dres, w, rstd), (dx, dw) = cases[0], outs[0]
    assert _run_noalloc(lib, x, dy, dres, w, rstd, dx, dw) == 0
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]
    for (x, dy, dres, w, rstd), (dx, dw) in zip(cases, outs):      # two calls in a row, second one smaller
        assert _run_noalloc(lib, x, dy, dres, w, rstd, dx, dw) == 0
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    # a raw cudaMalloc inside the library would not show in PyTorch's counter, but it does lower the device's free bytes
    assert torch.cuda.mem_get_info()[0] >= free_before
    for (x, dy, dres, w, rstd), (dx, dw) in zip(cases, outs):
        rdx, rdw = _run_existing(lib, x, dy, dres, w, rstd)
        torch.cuda.synchronize()
        assert (dx.float() - rdx.float()).abs().max().item() <= 2e-2 * max(rdx.float().abs().max().item(), 1.0)
        assert (dw - rdw).abs().max().item() <= 2e-2 * max(rdw.abs().max().item(), 1.0)
    _lib.raise_on_any_device_error()


def test_noalloc_entry_point_rejects_sizes_beyond_its_workspace():
    from trainscale_b200.ops import _lib
    lib = _lib.load("elementwise")
    x, dy, dres, w, rstd = _inputs(4, 8192 + 8, 3)
    dx, dw = torch.empty_like(x), torch.empty(x.shape[1], dtype=torch.float32, device="cuda")
    assert _run_noalloc(lib, x, dy, dres, w, rstd, dx, dw) == -20
    x2, dy2, dres2, w2, rstd2 = _inputs(4, 8192, 4)                  # exactly the limit is accepted
    dx2, dw2 = torch.empty_like(x2), torch.empty(8192, dtype=torch.float32, device="cuda")
    assert _run_noalloc(lib, x2, dy2, dres2, w2, rstd2, dx2, dw2) == 0
    torch.cuda.synchronize()
    rdx, rdw = _run_existing(lib, x2, dy2, dres2, w2, rstd2)
    assert (dw2 - rdw).abs().max().item() <= 2e-2 * max(rdw.abs().max().item(), 1.0)
