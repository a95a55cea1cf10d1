"""The bounds-checked debug build (TS_DEBUG=1): clean on correct launches, and an access outside its tensor is skipped
and reported instead of made.  Each case runs in a child process so that the debug libraries are the ones loaded."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _run(code: str, **env) -> str:
    e = dict(os.environ, TS_DEBUG="1", PYTHONPATH=str(ROOT), **env)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, env=e, cwd=str(ROOT))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    return r.stdout


def test_debug_libraries_are_clean_on_correct_launches():
    out = _run("""
import torch
from trainscale_b200.ops import _lib, build, fp8, gemm, norm
assert build.DEBUG and build.LIB_DIR.name == "lib_debug"
torch.manual_seed(0)
a = torch.randn(1000, 264, device="cuda", dtype=torch.bfloat16)
b = torch.randn(520, 264, device="cuda", dtype=torch.bfloat16)
ref = a.float() @ b.float().t()
for bn in (0, 128, 512):
    c = gemm.matmul_nt(a, b, bn=bn)
    assert (c.float() - ref).abs().max() / ref.abs().max() < 1e-2
aq, sa = fp8.quant_rowwise(torch.randn(304, 528, device="cuda", dtype=torch.bfloat16))
bq, sb = fp8.quant_rowwise(torch.randn(400, 528, device="cuda", dtype=torch.bfloat16))
y = fp8.gemm_rowwise(aq, sa, bq, sb, 304, 400, 528)
want = fp8.dequant_rowwise(aq, sa, 0) @ fp8.dequant_rowwise(bq, sb, 0).t()
assert (y.float() - want).abs().max() <= 1e-2 * want.abs().max()
x = torch.randn(65, 4096, device="cuda", dtype=torch.bfloat16)
norm.rmsnorm(x, torch.ones(4096, device="cuda", dtype=torch.bfloat16))
torch.cuda.synchronize()
_lib.raise_on_any_device_error()
print("CLEAN")
""")
    assert "CLEAN" in out


def test_store_outside_the_output_is_skipped_and_reported():
    """The debug launcher is told that C ends 100 rows early (its test hook): the epilogue's bounds check keeps the
    kernel from writing those rows and the error word names the check; no out-of-bounds access is made."""
    out = _run("""
import torch
from trainscale_b200.ops import _lib, gemm
a = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16)
b = torch.randn(384, 256, device="cuda", dtype=torch.bfloat16)
c = torch.full((512, 384), 7.0, device="cuda", dtype=torch.bfloat16)
gemm.matmul_nt(a, b, out=c)
torch.cuda.synchronize()
code, site, _, _ = _lib.device_error("gemm")
assert code == 5 and site == 7000, (code, site)
assert bool((c[412:] == 7.0).all()), "rows beyond the declared extent were written"
ref = a.float() @ b.float().t()
assert (c[:412].float() - ref[:412]).abs().max() / ref.abs().max() < 1e-2
_lib.clear_device_error("gemm")
print("REPORTED")
""", TS_DEBUG_SHRINK_C_ROWS="100")
    assert "REPORTED" in out


def test_canaries_around_symmetric_buffers():
    out = _run("""
import os, torch, torch.distributed as dist
os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", "29799")
torch.cuda.set_device(0)
dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
from trainscale_b200.core.errors import CommunicationError
from trainscale_b200.parallel.symm import SymmetricHeap
heap = SymmetricHeap.try_create(None, torch.device("cuda", 0))
if heap is None:
    print("NO_SYMM")
else:
    t = heap.alloc(1024, torch.float32)
    t.fill_(3.0)                      # the whole buffer, and nothing else
    heap.check_canaries()
    buf, _ = heap.lookup(t)
    buf.raw[-1] = 0                   # what an overrun by one byte would leave behind
    try:
        heap.check_canaries()
        print("MISSED")
    except CommunicationError:
        print("CAUGHT")
dist.destroy_process_group()
""")
    assert "CAUGHT" in out or "NO_SYMM" in out
