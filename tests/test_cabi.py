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
    assert lib.mvpa_abi_version() == nat.ABI_VERSION


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


_CTYPES = {"int32_t": ctypes.c_int32, "float": ctypes.c_float, "void*": ctypes.c_void_p, "int64_t": ctypes.c_int64}


def _header_struct(name):
    """(field, ctypes type) pairs of `struct <name>` as `include/mvpa.h` declares them."""
    text = open(os.path.join(ROOT, "include", "mvpa.h")).read()
    body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (name, name), text, flags=re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for decl in body.split(";"):
        decl = decl.strip()
        if not decl:
            continue
        m = re.match(r"(int32_t|int64_t|float|void\s*\*)\s*(.*)", decl)
        ctype = _CTYPES[m.group(1).replace(" ", "")]
        fields += [(n.strip(), ctype) for n in m.group(2).split(",")]
    return fields


def _integration_structs():
    """The `Problem` / `Tensor` classes of the binding shown in INTEGRATION.md, executed as written."""
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    block = next(b for b in re.findall(r"```python\n(.*?)```", text, flags=re.S) if "class Problem" in b)
    defs = block[block.index("class Problem"):block.index("lib = ctypes.CDLL")]
    ns = {"ctypes": ctypes}
    exec(defs, ns)
    return ns["Problem"], ns["Tensor"]


def test_struct_layouts_match_the_header():
    """`mvpa_problem` / `mvpa_tensor`: field names, order and types agree between the header, the
    ctypes shim and the binding printed in INTEGRATION.md (a struct that is short hands the library
    garbage in its last fields)."""
    doc_problem, doc_tensor = _integration_structs()
    for cname, shim, doc in (("mvpa_problem", nat.Problem, doc_problem), ("mvpa_tensor", nat.Tensor, doc_tensor)):
        want = _header_struct(cname)
        for cls in (shim, doc):
            assert [(n, t) for n, t in cls._fields_] == want, (cname, cls)
            assert ctypes.sizeof(cls) == ctypes.sizeof(shim)
    assert ctypes.sizeof(nat.Problem) == 48 and ctypes.sizeof(nat.Tensor) == 32


def test_integration_binding_passes_every_problem_field():
    """The `Problem(...)` call in INTEGRATION.md's binding gives one value per struct field."""
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    call = re.search(r"p = Problem\((.*?)\)[^\n]*\n\s+o = ", text, flags=re.S).group(1)
    call = re.sub(r"#[^\n]*", "", call)
    depth, args, cur = 0, [], ""
    for ch in call:
        depth += ch in "([{"
        depth -= ch in ")]}"
        if ch == "," and depth == 0:
            args.append(cur)
            cur = ""
        else:
            cur += ch
    args.append(cur)
    assert len(args) == len(nat.Problem._fields_)
