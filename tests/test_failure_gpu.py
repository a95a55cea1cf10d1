"""Device-side wait limits: a wait on a flag that nothing sets must give up after its limit, report through the status
word and the library's error word, and leave the context usable (no trap, no fault, no endless loop)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_flag_wait_times_out_and_reports():
    from trainscale_b200.parallel import fused_comm
    status, err = fused_comm.wait_selftest(limit_cycles=2_000_000)       # about a millisecond
    assert status == 1
    assert err[0] == 2 and err[1] == 990                                  # ERR_FLAG_TIMEOUT at the self-test's site
    # the context is still usable and the error word was cleared by the helper
    x = torch.ones(1024, device="cuda")
    assert float((x * 2).sum()) == 2048.0
    from trainscale_b200.ops import _lib
    assert _lib.device_error("comm")[0] == 0
