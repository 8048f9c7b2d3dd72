"""GPU: a bounded device-side wait that runs out returns an error status; nothing faults or hangs.

`mvpa_selftest_wait_timeout` launches one warp that waits, with a one-millisecond deadline on the
GPU's nanosecond timer, on an mbarrier nothing arrives at.  The kernel must come back, the status
word must carry its code, `mvpa_workspace_status` must report MVPA_ERR_DEVICE, and the context
must stay usable (a regular forward afterwards works)."""
import ctypes
import time

import pytest
import torch

import attentions
import mvpa_native as nat

pytestmark = pytest.mark.gpu


def test_wait_gives_up_and_reports(cuda):
    lib = nat.lib()
    ws = torch.zeros(256, dtype=torch.uint8, device=cuda)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    t0 = time.perf_counter()
    nat.check(lib.mvpa_selftest_wait_timeout(ws.data_ptr(), 256, 1000, stream), "selftest launch")
    st = lib.mvpa_workspace_status(ws.data_ptr(), 256, stream)
    elapsed = time.perf_counter() - t0
    assert st == -7 and "code 59" in nat.last_error()          # MVPA_ERR_DEVICE, the self-test's wait
    assert elapsed < 1.0, f"a 1 ms deadline took {elapsed:.3f} s"
    assert ws.view(torch.int32)[0].item() == 59
    # the context is intact: an ordinary forward runs and reports a clean status
    g = torch.Generator().manual_seed(5)
    r = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).to(cuda)
    o = attentions.flashmvpa(r(1, 2, 4 * 32, 64), r(1, 2, 1, 64), r(1, 2, 1, 64), r(1, 2, 1, 64), r(1, 2, 4 * 32, 64),
                             r(1, 2, 4, 64), r(1, 2, 32, 64), r(1, 2, 4 * 32, 64), causal=True, sm_scale=0.125,
                             window_size=10)
    assert torch.isfinite(o.float()).all()


def test_selftest_argument_checks(cuda):
    lib = nat.lib()
    ws = torch.zeros(256, dtype=torch.uint8, device=cuda)
    assert lib.mvpa_selftest_wait_timeout(ws.data_ptr(), 16, 1000, None) == -4
    assert lib.mvpa_selftest_wait_timeout(ws.data_ptr(), 256, 0, None) == -1
