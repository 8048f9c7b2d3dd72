"""Loader and builder of the Flash-MVPA shared library (C ABI in ``include/mvpa.h``).

The library is compiled in-tree with ``nvcc`` for sm_100a only and bound through
``ctypes``; PyTorch supplies device memory and the CUDA stream, nothing else.
There is no fallback: if the library is missing and cannot be built, importing
callers get an ``ImportError``.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_HERE, "csrc")
_INCLUDE = os.path.join(os.path.dirname(_HERE), "include")
LIB_PATH = os.path.join(_HERE, "libmvpa_b200.so")
HASH_PATH = LIB_PATH + ".srchash"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared", "--use_fast_math",
]

MVPA_F32, MVPA_BF16, MVPA_F16 = 0, 1, 2

_lock = threading.Lock()
_lib = None


def sources():
    return sorted(os.path.join(_CSRC, f) for f in os.listdir(_CSRC) if f.endswith(".cu"))


def _source_hash() -> str:
    """Digest of everything the binary depends on (file times do not survive a copy)."""
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    deps = sorted(os.path.join(_CSRC, f) for f in os.listdir(_CSRC)) + [os.path.join(_INCLUDE, "mvpa.h")]
    for d in deps:
        h.update(os.path.basename(d).encode())
        with open(d, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _stale() -> bool:
    if not (os.path.exists(LIB_PATH) and os.path.exists(HASH_PATH)):
        return True
    with open(HASH_PATH) as f:
        return f.read().strip() != _source_hash()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile ``csrc/*.cu`` into ``libmvpa_b200.so`` (cross-compiles without a GPU)."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise ImportError("nvcc not found: cannot build libmvpa_b200.so")
    tmp = LIB_PATH + ".tmp"
    cmd = [nvcc, *NVCC_FLAGS, "-I", _INCLUDE, "-I", _CSRC, *sources(), "-o", tmp]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise ImportError("building libmvpa_b200.so failed:\n" + res.stdout + res.stderr)
    os.replace(tmp, LIB_PATH)
    with open(HASH_PATH, "w") as f:
        f.write(_source_hash())
    if verbose:
        print(res.stderr)
    return LIB_PATH


class Problem(ctypes.Structure):
    _fields_ = [("B", ctypes.c_int32), ("H", ctypes.c_int32), ("Hkv", ctypes.c_int32),
                ("T", ctypes.c_int32), ("C", ctypes.c_int32), ("D", ctypes.c_int32),
                ("window", ctypes.c_int32), ("dtype", ctypes.c_int32),
                ("sm_scale", ctypes.c_float), ("flags", ctypes.c_int32),
                ("q_time_begin", ctypes.c_int32), ("q_time_count", ctypes.c_int32)]


class Tensor(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("stride_b", ctypes.c_int64),
                ("stride_h", ctypes.c_int64), ("stride_n", ctypes.c_int64)]


EXPORTS = ("mvpa_fwd", "mvpa_bwd", "mvpa_fwd_workspace_bytes", "mvpa_bwd_workspace_bytes",
           "mvpa_last_error_string", "mvpa_launch_count", "mvpa_abi_version",
           "mvpa_workspace_status", "mvpa_fwd_noalloc", "mvpa_bwd_status", "mvpa_noalloc_status",
           "mvpa_selftest_wait_timeout", "mvpa_rmsnorm", "mvpa_silu_mul", "mvpa_wave_encode_size",
           "mvpa_wave_encode", "mvpa_channel_mean", "mvpa_contrastive_logits", "mvpa_peer_gather", "mvpa_peer_signal",
           "mvpa_peer_wait")
ABI_VERSION = 3   # mvpa_abi_version() of the header this shim was written against


def lib() -> ctypes.CDLL:
    """The loaded library; builds it first when the sources are newer than the binary."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if _stale():
            try:
                build()
            except ImportError:
                if not os.path.exists(LIB_PATH):
                    raise
        try:
            L = ctypes.CDLL(LIB_PATH)
        except OSError as e:  # no silent fallback: the CUDA library is the product
            raise ImportError(f"cannot load {LIB_PATH}: {e}") from e
        P, Tn, vp = ctypes.POINTER(Problem), ctypes.POINTER(Tensor), ctypes.c_void_p
        L.mvpa_fwd_workspace_bytes.restype = ctypes.c_size_t
        L.mvpa_fwd_workspace_bytes.argtypes = [P]
        L.mvpa_bwd_workspace_bytes.restype = ctypes.c_size_t
        L.mvpa_bwd_workspace_bytes.argtypes = [P]
        L.mvpa_fwd.restype = ctypes.c_int
        L.mvpa_fwd.argtypes = [P, Tn, Tn, Tn, vp, vp, vp, vp, vp, Tn, vp, vp, ctypes.c_size_t, vp]
        L.mvpa_bwd.restype = ctypes.c_int
        L.mvpa_bwd.argtypes = [P, Tn, Tn, Tn, vp, vp, vp, vp, vp, Tn, vp, Tn, Tn, Tn, Tn,
                               vp, vp, vp, vp, vp, vp, ctypes.c_size_t, vp]
        L.mvpa_fwd_noalloc.restype = ctypes.c_int
        L.mvpa_fwd_noalloc.argtypes = [P, Tn, Tn, Tn, vp, vp, vp, vp, vp, Tn, vp, vp]
        L.mvpa_workspace_status.restype = ctypes.c_int
        L.mvpa_workspace_status.argtypes = [vp, ctypes.c_size_t, vp]
        L.mvpa_bwd_status.restype = ctypes.c_int
        L.mvpa_bwd_status.argtypes = [P, vp, ctypes.c_size_t, vp]
        L.mvpa_noalloc_status.restype = ctypes.c_int
        L.mvpa_noalloc_status.argtypes = [vp]
        L.mvpa_selftest_wait_timeout.restype = ctypes.c_int
        L.mvpa_selftest_wait_timeout.argtypes = [vp, ctypes.c_size_t, ctypes.c_uint32, vp]
        i32, i64, f32 = ctypes.c_int32, ctypes.c_int64, ctypes.c_float
        L.mvpa_rmsnorm.restype = ctypes.c_int
        L.mvpa_rmsnorm.argtypes = [vp, vp, vp, vp, vp, i64, i32, f32, i32, vp]
        L.mvpa_silu_mul.restype = ctypes.c_int
        L.mvpa_silu_mul.argtypes = [vp, vp, i64, vp, i64, i64, i32, i32, vp]
        L.mvpa_wave_encode_size.restype = i32
        L.mvpa_wave_encode_size.argtypes = [i32, ctypes.POINTER(i32), i32]
        L.mvpa_wave_encode.restype = ctypes.c_int
        L.mvpa_wave_encode.argtypes = [vp, i64, i32, ctypes.POINTER(f32), ctypes.POINTER(f32), vp, vp, i64, i32, i64,
                                       i32, f32, vp]
        L.mvpa_peer_signal.restype = ctypes.c_int
        L.mvpa_peer_signal.argtypes = [vp, i32, ctypes.c_uint32, vp, vp]
        L.mvpa_peer_wait.restype = ctypes.c_int
        L.mvpa_peer_wait.argtypes = [vp, i32, ctypes.c_uint32, vp, ctypes.c_uint32, vp, vp]
        L.mvpa_peer_gather.restype = ctypes.c_int
        L.mvpa_peer_gather.argtypes = [vp, vp, vp, i32, vp]
        L.mvpa_channel_mean.restype = ctypes.c_int
        L.mvpa_channel_mean.argtypes = [vp, vp, i32, i32, i32, i32, i32, vp]
        L.mvpa_contrastive_logits.restype = ctypes.c_int
        L.mvpa_contrastive_logits.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32, f32, i32, vp]
        L.mvpa_last_error_string.restype = ctypes.c_char_p
        L.mvpa_launch_count.restype = ctypes.c_uint64
        L.mvpa_abi_version.restype = ctypes.c_int
        if L.mvpa_abi_version() != ABI_VERSION:  # e.g. a stale binary kept because the rebuild failed
            raise ImportError(f"{LIB_PATH} has ABI version {L.mvpa_abi_version()}, this shim needs {ABI_VERSION}: "
                              "rebuild it (python __graft_entry__.py)")
        _lib = L
        return L


def last_error() -> str:
    return lib().mvpa_last_error_string().decode()


def check(status: int, what: str) -> None:
    """Raise like the reference does (`attentions/attn.py:1034-1045`): RuntimeError."""
    if status != 0:
        raise RuntimeError(f"{what} failed (status {status}): {last_error()}")
