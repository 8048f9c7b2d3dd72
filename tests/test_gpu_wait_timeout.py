"""GPU: a bounded device-side wait that runs out returns an error status; nothing faults or hangs.

`mvpa_selftest_wait_timeout` launches one warp that waits, with a one-millisecond deadline on the
GPU's nanosecond timer, on an mbarrier nothing arrives at.  The kernel must come back, the status
word must carry its code, `mvpa_workspace_status` must report MVPA_ERR_DEVICE, and the context
must stay usable (a regular forward afterwards works).  The same for the flags between GPUs of
the peer-load transport (`mvpa_peer_wait`): a slot nothing writes makes the wait run out."""
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


def test_peer_flags_signal_wait_and_timeout(cuda):
    """The flags of the peer-load transport on one GPU: a signal makes a later wait pass; a wait on a slot
    nothing writes gives up after its deadline, sets the status word and leaves the context usable; the
    gather kernel copies its pieces bit for bit."""
    lib = nat.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    flags = torch.zeros(64, dtype=torch.int32, device=cuda)
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    slot = lambda i: flags.data_ptr() + 4 * i
    two = (ctypes.c_void_p * 2)(slot(0), slot(1))
    nat.check(lib.mvpa_peer_signal(two, 2, 7, None, stream), "signal")
    nat.check(lib.mvpa_peer_wait(two, 2, 7, None, 2000, ctypes.c_void_p(status.data_ptr()), stream), "wait")
    nat.check(lib.mvpa_peer_wait(two, 2, 5, None, 2000, ctypes.c_void_p(status.data_ptr()), stream), "wait for an earlier step")
    base = torch.tensor([4], dtype=torch.int32, device=cuda)        # a step counter on the device: 4 + 3 = 7, 4 - 1 = 3
    nat.check(lib.mvpa_peer_wait(two, 2, 3, ctypes.c_void_p(base.data_ptr()), 2000, ctypes.c_void_p(status.data_ptr()), stream), "wait, device base")
    nat.check(lib.mvpa_peer_wait(two, 2, 0xFFFFFFFF, ctypes.c_void_p(base.data_ptr()), 2000, ctypes.c_void_p(status.data_ptr()), stream), "wait, base - 1")
    torch.cuda.synchronize()
    assert flags[:2].tolist() == [7, 7] and status.item() == 0
    one = (ctypes.c_void_p * 1)(slot(2))                             # nothing ever writes slot 2
    t0 = time.perf_counter()
    nat.check(lib.mvpa_peer_wait(one, 1, 1, None, 2000, ctypes.c_void_p(status.data_ptr()), stream), "wait that runs out")
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0 and status.item() == 1
    src = torch.arange(3 * 70000, dtype=torch.int32, device=cuda).view(3, 70000)     # 280 000 bytes per piece
    dst = torch.zeros_like(src)
    n = 3
    nat.check(lib.mvpa_peer_gather((ctypes.c_void_p * n)(*[dst[i].data_ptr() for i in range(n)]),
                                   (ctypes.c_void_p * n)(*[src[i].data_ptr() for i in range(n)]),
                                   (ctypes.c_int64 * n)(280000, 16, 0), n, stream), "gather")
    torch.cuda.synchronize()
    assert torch.equal(dst[0], src[0]) and torch.equal(dst[1, :4], src[1, :4]) and int(dst[1, 4:].abs().sum()) == 0
    assert int(dst[2].abs().sum()) == 0
    assert lib.mvpa_peer_gather((ctypes.c_void_p * 1)(dst.data_ptr()), (ctypes.c_void_p * 1)(src.data_ptr()),
                                (ctypes.c_int64 * 1)(24), 1, stream) == -3      # not a multiple of 16 bytes
