"""GPU: `mvpa_fwd_noalloc`, the forward for hosts that may not allocate device memory on the path
that runs attention (a server whose memory pool took the whole device, a plugin execute hook).
Its scratch lives in a fixed device array inside the library, shared by every call, so the check
is two calls in a row on different problems: each must match `mvpa_fwd` (which gets a fresh,
caller-owned workspace) on the same inputs, i.e. nothing of the first call may leak into the second.

Collected last on purpose (file name), so a failure here cannot hide the other GPU tests.
"""
import ctypes

import pytest
import torch

import mvpa_native as nat

pytestmark = pytest.mark.gpu

# The two entry points run the same kernels on the same inputs, so the results must be identical;
# both also leave a status word that has to read "no wait gave up".


def _inputs(dev, seed, B, H, Hkv, T, C, D):
    g = torch.Generator().manual_seed(seed)
    N = T * C
    r = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).to(dev)
    return dict(q=r(B, H, N, D), k=r(B, Hkv, N, D), v=r(B, Hkv, N, D), u=r(Hkv, D), vt=r(Hkv, D), z=r(Hkv, D),
                rt=r(Hkv, T, D), rc=r(Hkv, C, D)), nat.Problem(B, H, Hkv, T, C, D, 10, nat.MVPA_BF16, D ** -0.5, 0)


def _call(t, prob, noalloc):
    lib = nat.lib()
    o = torch.empty_like(t["q"])
    lse = torch.empty(t["q"].shape[0] * t["q"].shape[1], t["q"].shape[2], device=o.device, dtype=torch.float32)
    tens = [nat.Tensor(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2)) for x in (t["q"], t["k"], t["v"], o)]
    ref = [ctypes.byref(x) for x in tens]
    small = [t[n].data_ptr() for n in ("u", "vt", "z", "rt", "rc")]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    if noalloc:
        st = lib.mvpa_fwd_noalloc(ctypes.byref(prob), ref[0], ref[1], ref[2], *small, ref[3], lse.data_ptr(), stream)
    else:
        n = lib.mvpa_fwd_workspace_bytes(ctypes.byref(prob))
        ws = torch.empty(max(n, 16), dtype=torch.uint8, device=o.device)
        st = lib.mvpa_fwd(ctypes.byref(prob), ref[0], ref[1], ref[2], *small, ref[3], lse.data_ptr(),
                          ws.data_ptr(), n, stream)
    nat.check(st, "mvpa_fwd_noalloc" if noalloc else "mvpa_fwd")
    if noalloc:
        nat.check(lib.mvpa_noalloc_status(stream), "mvpa_fwd_noalloc kernels")
    else:
        nat.check(lib.mvpa_workspace_status(ws.data_ptr(), n, stream), "mvpa_fwd kernels")
    torch.cuda.synchronize()
    return o, lse


def test_noalloc_matches_workspace_entry_point_twice_in_a_row(cuda):
    first = _inputs(cuda, 41, 1, 4, 2, 14, 64, 64)     # GQA, two time steps per tile, light tiles
    second = _inputs(cuda, 42, 2, 2, 2, 13, 100, 128)  # other head count, ragged channels, D = 128
    for t, prob in (first, second, first):
        o_ref, lse_ref = _call(t, prob, noalloc=False)
        o_new, lse_new = _call(t, prob, noalloc=True)
        assert torch.isfinite(o_new.float()).all()
        assert torch.equal(o_new, o_ref)
        assert torch.equal(lse_new, lse_ref)


def test_noalloc_rejects_what_it_cannot_hold(cuda):
    lib = nat.lib()
    t, prob = _inputs(cuda, 43, 1, 2, 2, 4, 16, 32)    # D = 32: not a tensor-core forward shape
    tens = [nat.Tensor(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2)) for x in (t["q"], t["k"], t["v"], t["q"])]
    ref = [ctypes.byref(x) for x in tens]
    small = [t[n].data_ptr() for n in ("u", "vt", "z", "rt", "rc")]
    st = lib.mvpa_fwd_noalloc(ctypes.byref(prob), ref[0], ref[1], ref[2], *small, ref[3], None, None)
    assert st == -6 and "mvpa_fwd" in nat.last_error()
    big = nat.Problem(1, 128, 128, 2, 32, 64, 10, nat.MVPA_BF16, 0.125, 0)   # 128 kv heads > 64
    st = lib.mvpa_fwd_noalloc(ctypes.byref(big), ref[0], ref[1], ref[2], *small, ref[3], None, None)
    assert st == -4 and "64" in nat.last_error()
