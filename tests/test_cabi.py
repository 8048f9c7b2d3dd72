"""CPU: the C-ABI library builds, loads, exports every symbol `include/mvpa.h` declares, and
rejects bad arguments with the documented codes before touching a device."""
import ctypes
import os
import re

import mvpa_native as nat
from conftest import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "mvpa.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mvpa_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = nat.lib()
    names = _declared()
    assert {"mvpa_fwd", "mvpa_bwd", "mvpa_fwd_workspace_bytes", "mvpa_bwd_workspace_bytes",
            "mvpa_last_error_string", "mvpa_launch_count", "mvpa_abi_version"} <= set(names)
    for n in names:
        assert hasattr(lib, n), n
    assert set(nat.EXPORTS) <= set(names)
    assert lib.mvpa_abi_version() >= 1


def _prob(**kw):
    d = dict(B=1, H=4, Hkv=2, T=4, C=4, D=64, window=10, dtype=nat.MVPA_F32, sm_scale=0.125, flags=0,
             q_time_begin=0, q_time_count=0)
    d.update(kw)
    return nat.Problem(*[d[f[0]] for f in nat.Problem._fields_])


def _call_fwd(prob, ptr=256, stride_n=64):
    lib = nat.lib()
    t = nat.Tensor(ptr, 64 * 16, 64 * 16 * 4, stride_n)
    r = ctypes.byref(t)
    return lib.mvpa_fwd(ctypes.byref(prob), r, r, r, 256, 256, 256, 256, 256, r, None, None, 0, None)


def test_argument_errors_are_reported_without_a_device():
    assert _call_fwd(_prob(H=3)) == -1 and "divisible" in nat.last_error()
    assert _call_fwd(_prob(D=48)) == -1 and "head dim" in nat.last_error()
    assert _call_fwd(_prob(T=0)) == -1
    assert _call_fwd(_prob(dtype=7)) == -2
    assert _call_fwd(_prob(dtype=nat.MVPA_F16, H=3)) == -1   # fp16 is a known element type: the shape is what fails
    assert _call_fwd(_prob(), ptr=260) == -3 and "16" in nat.last_error()
    assert _call_fwd(_prob(), stride_n=63) == -3
    assert _call_fwd(_prob(flags=1)) == -1
    assert _call_fwd(_prob(q_time_begin=3, q_time_count=2)) == -1 and "time range" in nat.last_error()


def test_workspace_queries():
    lib = nat.lib()
    p = _prob(B=2, H=4, Hkv=2, T=8, C=4, D=64)
    n = 2 * 4 * 32
    need = lib.mvpa_bwd_workspace_bytes(ctypes.byref(p))
    assert need >= 4 * (2 * n * (8 + 4) + n)
    assert lib.mvpa_fwd_workspace_bytes(ctypes.byref(p)) == 0  # fp32 forward needs no scratch
    assert lib.mvpa_bwd_workspace_bytes(ctypes.byref(_prob(D=48))) == 0
    # fp16 runs on the same fp32-arithmetic kernels: same scratch as fp32
    p16 = _prob(B=2, H=4, Hkv=2, T=8, C=4, D=64, dtype=nat.MVPA_F16)
    assert lib.mvpa_fwd_workspace_bytes(ctypes.byref(p16)) == 0
    assert lib.mvpa_bwd_workspace_bytes(ctypes.byref(p16)) == need


def test_python_constants_match_the_header():
    """Element-type codes of the ctypes shim are the header's `#define`s."""
    text = open(os.path.join(ROOT, "include", "mvpa.h")).read()
    defs = {m.group(1): int(m.group(2)) for m in re.finditer(r"#define\s+(MVPA_[A-Z0-9_]+)\s+\(?(-?\d+)\)?", text)}
    for name in ("MVPA_F32", "MVPA_BF16", "MVPA_F16"):
        assert defs[name] == getattr(nat, name), name
    assert defs["MVPA_OK"] == 0 and defs["MVPA_ERR_DTYPE"] == -2 and defs["MVPA_ERR_SHAPE"] == -1
