"""`flash_mvpa` — drop-in for the reference operator of the same name
(`attentions/attn.py:1317-1366`), backed by the sm_100a CUDA library.

Same signature and argument meaning as the reference.  What differs inside:
the relative-score matrices of `_rel_bias` (`attentions/attn.py:1305-1314`) are
never materialised, the Triton kernels are replaced by the C-ABI calls
`mvpa_fwd` / `mvpa_bwd` (``include/mvpa.h``), and the backward returns the
gradients of all eight tensors directly instead of leaving part of the work to
autograd.  There is no CPU path: tensors must live on a CUDA device.
"""
from __future__ import annotations

import ctypes
import math
import os

import torch

import mvpa_native as _nat


# MVPA_CHECK_STATUS=1: read the kernels' status word back after every forward and backward (synchronises).
_CHECK_STATUS = os.environ.get("MVPA_CHECK_STATUS", "0") == "1"


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _nat.MVPA_BF16
    if t.dtype == torch.float32:
        return _nat.MVPA_F32
    if t.dtype == torch.float16:
        return _nat.MVPA_F16
    raise RuntimeError(f"flash_mvpa: dtype {t.dtype} not supported (bfloat16, float16 or float32)")


def _tensor(t: torch.Tensor) -> _nat.Tensor:
    return _nat.Tensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def _rows(t: torch.Tensor) -> torch.Tensor:
    """(B,H,N,D) with a contiguous last dim and 16-byte aligned strides, copying only if needed."""
    es = t.element_size()
    if t.stride(-1) != 1 or any((s * es) % 16 for s in t.stride()[:-1]) or t.data_ptr() % 16:
        t = t.contiguous()
    return t


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _problem(q, k, r_time, r_chan, sm_scale, window, q_time=(0, 0)) -> _nat.Problem:
    B, H, N, D = q.shape
    return _nat.Problem(B, H, k.shape[1], r_time.shape[-2], r_chan.shape[-2], D, int(window),
                        _dtype_code(q), float(sm_scale), 0, int(q_time[0]), int(q_time[1]))


class FlashMVPA(torch.autograd.Function):
    """Autograd wrapper; the counterpart of the reference's `FlashMVPA`
    (`attentions/attn.py:1013-1302`), taking the relative keys themselves instead of
    pre-multiplied score matrices."""

    @staticmethod
    def forward(ctx, q, u, vt, z, k, r_time, r_chan, v, sm_scale, window, q_time=(0, 0)):
        if not q.is_cuda:
            raise RuntimeError("flash_mvpa: tensors must be on a CUDA device (no CPU path)")
        lib = _nat.lib()
        q, k, v = _rows(q), _rows(k), _rows(v)
        u, vt, z, r_time, r_chan = (x.contiguous() for x in (u, vt, z, r_time, r_chan))
        prob = _problem(q, k, r_time, r_chan, sm_scale, window, q_time)
        o = torch.empty_like(q)
        lse = torch.empty((q.shape[0] * q.shape[1], q.shape[2]), device=q.device, dtype=torch.float32)
        nbytes = lib.mvpa_fwd_workspace_bytes(ctypes.byref(prob))
        ws = torch.empty(max(nbytes, 16), device=q.device, dtype=torch.uint8)
        tq, tk, tv, to = _tensor(q), _tensor(k), _tensor(v), _tensor(o)
        with torch.cuda.device(q.device):
            st = lib.mvpa_fwd(ctypes.byref(prob), ctypes.byref(tq), ctypes.byref(tk), ctypes.byref(tv),
                              u.data_ptr(), vt.data_ptr(), z.data_ptr(), r_time.data_ptr(),
                              r_chan.data_ptr(), ctypes.byref(to), lse.data_ptr(), ws.data_ptr(),
                              nbytes, _stream())
        _nat.check(st, "mvpa_fwd")
        if _CHECK_STATUS and nbytes:  # debugging aid: synchronises the stream
            _nat.check(lib.mvpa_workspace_status(ws.data_ptr(), nbytes, _stream()), "mvpa_fwd kernels")
        ctx.save_for_backward(q, u, vt, z, k, r_time, r_chan, v, o, lse)
        ctx.sm_scale, ctx.window, ctx.q_time = sm_scale, window, q_time
        return o

    @staticmethod
    def backward(ctx, do):
        q, u, vt, z, k, r_time, r_chan, v, o, lse = ctx.saved_tensors
        if ctx.q_time[1]:
            raise NotImplementedError("flash_mvpa: backward through a query time range is not implemented")
        lib = _nat.lib()
        do = _rows(do)
        prob = _problem(q, k, r_time, r_chan, ctx.sm_scale, ctx.window)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        # the five small gradients leave the library as fp32: one buffer, so that one cast serves all of them
        shapes = (u.shape, vt.shape, z.shape, r_time.shape, r_chan.shape)
        sizes = [(math.prod(sh) + 3) // 4 * 4 for sh in shapes]             # 16-byte aligned pieces
        small = torch.empty(sum(sizes), device=q.device, dtype=torch.float32)
        du, dvt, dz, drt, drc = (piece[:math.prod(sh)].view(sh) for piece, sh in zip(small.split(sizes), shapes))
        nbytes = lib.mvpa_bwd_workspace_bytes(ctypes.byref(prob))
        ws = torch.empty(max(nbytes, 16), device=q.device, dtype=torch.uint8)
        T = [_tensor(x) for x in (q, k, v, o, do, dq, dk, dv)]
        r = [ctypes.byref(x) for x in T]
        with torch.cuda.device(q.device):
            st = lib.mvpa_bwd(ctypes.byref(prob), r[0], r[1], r[2], u.data_ptr(), vt.data_ptr(),
                              z.data_ptr(), r_time.data_ptr(), r_chan.data_ptr(), r[3], lse.data_ptr(),
                              r[4], r[5], r[6], r[7], du.data_ptr(), dvt.data_ptr(), dz.data_ptr(),
                              drt.data_ptr(), drc.data_ptr(), ws.data_ptr(), nbytes, _stream())
        _nat.check(st, "mvpa_bwd")
        if _CHECK_STATUS:  # debugging aid: synchronises the stream
            _nat.check(lib.mvpa_bwd_status(ctypes.byref(prob), ws.data_ptr(), nbytes, _stream()), "mvpa_bwd kernels")
        small = small.to(q.dtype)
        du, dvt, dz, drt, drc = (piece[:math.prod(sh)].view(sh) for piece, sh in zip(small.split(sizes), shapes))
        return (dq, du, dvt, dz, dk, drt, drc, dv, None, None, None)


def flash_mvpa_into(out, q, u, vt, z, k, r_time, r_chan, v, sm_scale, window_size=10, q_time_range=None):
    """Inference form of `flash_mvpa`: no autograd record, no log-sum-exp output, and the result goes into
    `out`, a caller-owned (B,H,N,D) tensor that may be a strided view (e.g. a column block of the buffer the
    next projection reads).  u, vt, z (Hkv,D); r_time (Hkv,T,D); r_chan (Hkv,C,D).  `q_time_range=(t0, n)`:
    `q` and `out` hold only the tokens of time steps t0..t0+n-1 (see `flash_mvpa`).  No counterpart in the
    reference, whose operator always allocates its output (`attentions/attn.py:1047`)."""
    if not q.is_cuda:
        raise RuntimeError("flash_mvpa: tensors must be on a CUDA device (no CPU path)")
    lib = _nat.lib()
    q, k, v = _rows(q), _rows(k), _rows(v)
    u, vt, z, r_time, r_chan = (x.contiguous() for x in (u, vt, z, r_time, r_chan))
    es = out.element_size()
    if out.stride(-1) != 1 or any((st * es) % 16 for st in out.stride()[:-1]) or out.data_ptr() % 16 or out.shape != q.shape:
        raise RuntimeError("flash_mvpa_into: `out` must have q's shape, a contiguous last dimension and 16-byte aligned strides")
    q_time = (0, 0) if q_time_range is None else (int(q_time_range[0]), int(q_time_range[1]))
    prob = _problem(q, k, r_time, r_chan, sm_scale, window_size, q_time)
    nbytes = lib.mvpa_fwd_workspace_bytes(ctypes.byref(prob))
    ws = torch.empty(max(nbytes, 16), device=q.device, dtype=torch.uint8)
    tq, tk, tv, to = _tensor(q), _tensor(k), _tensor(v), _tensor(out)
    with torch.cuda.device(q.device):
        st = lib.mvpa_fwd(ctypes.byref(prob), ctypes.byref(tq), ctypes.byref(tk), ctypes.byref(tv),
                          u.data_ptr(), vt.data_ptr(), z.data_ptr(), r_time.data_ptr(), r_chan.data_ptr(),
                          ctypes.byref(to), None, ws.data_ptr(), nbytes, _stream())
    _nat.check(st, "mvpa_fwd")
    if _CHECK_STATUS and nbytes:
        _nat.check(lib.mvpa_workspace_status(ws.data_ptr(), nbytes, _stream()), "mvpa_fwd kernels")
    return out


def flash_mvpa(q, q_bias, q_btime, q_bchan, k_glob, k_time, k_chan, v, causal, sm_scale,
               window_size=0, p_drop=0.0, sequence_parallel=False, rel_bias_time=True,
               rel_bias_chan=True, generator=None, q_time_range=None):
    """Fused multi-variate parallel attention.

    q (B,H,N,D); q_bias/q_btime/q_bchan (1,Hkv,1,D) = u/v/z; k_glob, v (B,Hkv,N,D);
    k_time (1,Hkv,T,D); k_chan (1,Hkv,C,D); N == T*C, token n = t*C + c.  Returns o (B,H,N,D).

    As in the reference, causality is forced on whenever a relative term is used
    (`attentions/attn.py:1335-1336`) and the same shape checks raise
    (`:1339, 1344`).  `sequence_parallel` only chose a launch geometry in the
    reference (`:1165-1172`) and is accepted and ignored.  Structured attention dropout
    (`:1052-1062`) is applied to V on the way in (see below); runs with both relative terms off are
    not implemented and raise.

    `q_time_range=(t0, n)` (an extension, forward only): `q` holds only the tokens of time steps
    [t0, t0+n) while the keys, values and relative keys describe the whole sequence — what one
    rank computes when a long sample is sharded by query time blocks (`mvpa_shard`).
    """
    if not (rel_bias_time or rel_bias_chan):
        raise NotImplementedError("flash_mvpa: at least one relative term is required (without them the "
                                  "reference runs a plain windowed attention, which these kernels are not)")
    # One term switched off: the reference kernels skip it and change nothing else
    # (`attentions/attn.py:187-216, 241-308`), which is the same attention with that term's relative key
    # at zero; its key and its query bias then receive zero gradients, as in the reference.
    if not rel_bias_time:
        k_time = k_time * 0
    if not rel_bias_chan:
        k_chan = k_chan * 0
    if p_drop and not 0 < p_drop < 1:
        raise ValueError(f"flash_mvpa: p_drop must be in [0, 1), got {p_drop}")
    q_heads, kv_heads = q.shape[1], v.shape[1]
    assert q_heads % kv_heads == 0, "Q heads must be divisible by KV heads."
    n_ctx, time_ctx, chan_ctx = k_glob.shape[2], k_time.shape[2], k_chan.shape[2]
    assert n_ctx == time_ctx * chan_ctx
    q_time = (0, 0)
    if q_time_range is not None:
        q_time = (int(q_time_range[0]), int(q_time_range[1]))
        assert q_time[1] > 0 and q.shape[2] == q_time[1] * chan_ctx
    else:
        assert q.shape[2] == n_ctx
    assert q.shape[-1] == k_glob.shape[-1] == v.shape[-1]
    assert q.shape[-1] in {16, 32, 64, 128}
    D = q.shape[-1]
    if p_drop and p_drop > 0:
        # Structured dropout of the reference (`attentions/attn.py:1052-1062, 316-321`): whole key time
        # steps and key channels are dropped, each with probability 1 - sqrt(1 - p_drop), and the kept
        # probabilities are divided by 1 - p_drop after the softmax denominator is taken.  The mask depends
        # on the key alone, so P_dropped V = (P (mask V)) / (1 - p_drop): one exact 0/1 pass over V before the
        # kernels and one fp32 scaling of their output (the reference divides P in fp32, `:235`), and autograd
        # carries both into dV and dO.  Same draws in the same order as the reference (channels, then time
        # steps), so a generator seeded alike gives the same mask.
        p_per_dim = 1 - math.sqrt(1 - p_drop)
        chan_keep = torch.rand(chan_ctx, device=q.device, generator=generator) > p_per_dim
        time_keep = torch.rand(time_ctx, device=q.device, generator=generator) > p_per_dim
        keep = (time_keep[:, None] & chan_keep[None, :]).reshape(1, 1, n_ctx, 1)
        v = v * keep.to(v.dtype)
    u, vt, z = (x.reshape(kv_heads, D) for x in (q_bias, q_btime, q_bchan))
    o = FlashMVPA.apply(q, u, vt, z, k_glob, k_time.reshape(kv_heads, time_ctx, D),
                        k_chan.reshape(kv_heads, chan_ctx, D), v, sm_scale, window_size, q_time)
    if p_drop and p_drop > 0:
        o = (o.float() * (1.0 / (1 - p_drop))).to(o.dtype)
    return o
