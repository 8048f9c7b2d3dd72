"""Torch-tensor front ends of the C-ABI kernels that surround the attention in an MVPFormer block,
its encoder and its heads (``include/mvpa.h``: mvpa_rmsnorm, mvpa_silu_mul, mvpa_wave_encode,
mvpa_channel_mean, mvpa_contrastive_logits).  Forward only: these are the inference kernels; the
modules in ``models/`` fall back to differentiable torch expressions when gradients are required.
CUDA tensors only, bf16 or fp32.
"""
from __future__ import annotations

import ctypes
import functools

import numpy as np
import torch

import mvpa_native as _nat


def _code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _nat.MVPA_BF16
    if t.dtype == torch.float32:
        return _nat.MVPA_F32
    raise RuntimeError(f"mvpa_ops: dtype {t.dtype} not supported (bfloat16 or float32)")


def _stream(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("mvpa_ops: tensors must be on a CUDA device (no CPU path)")


def rmsnorm(x, weight, eps, add=None, sum_out=None, out=None):
    """y = rmsnorm(h) * weight over the last dimension, h = x (+ add).  With `add`, h is written to `sum_out`
    (which may be `x` itself: the update is elementwise).  Returns y."""
    _need_cuda(x, weight, add)
    E = x.shape[-1]
    x2 = x.reshape(-1, E)
    assert x2.is_contiguous() and weight.is_contiguous() and weight.dtype == x.dtype
    y = torch.empty_like(x2) if out is None else out
    if add is not None:
        assert add.dtype == x.dtype and add.reshape(-1, E).is_contiguous()
    with torch.cuda.device(x.device):
        st = _nat.lib().mvpa_rmsnorm(x2.data_ptr(), add.data_ptr() if add is not None else None, weight.data_ptr(),
                                     sum_out.data_ptr() if sum_out is not None else None, y.data_ptr(), x2.shape[0], E,
                                     float(eps), _code(x), _stream(x))
    _nat.check(st, "mvpa_rmsnorm")
    return y.view(x.shape)


def silu_mul(gate, up, out):
    """out = silu(gate) * up for 2-D views with unit inner stride (column blocks of wider buffers are fine)."""
    _need_cuda(gate, up, out)
    rows, width = gate.shape
    assert up.shape == gate.shape and out.shape == gate.shape
    assert gate.stride(1) == up.stride(1) == out.stride(1) == 1 and gate.stride(0) == up.stride(0)
    with torch.cuda.device(gate.device):
        st = _nat.lib().mvpa_silu_mul(gate.data_ptr(), up.data_ptr(), gate.stride(0), out.data_ptr(), out.stride(0), rows,
                                      width, _code(gate), _stream(gate))
    _nat.check(st, "mvpa_silu_mul")
    return out


@functools.lru_cache(maxsize=None)
def db4_filters():
    """Decomposition filters (dec_lo, dec_hi) of the Daubechies wavelet with four vanishing moments, eight
    taps, derived numerically: |H(w)|^2 = 2 cos^8(w/2) P(sin^2(w/2)), P(y) = 1 + 4y + 10y^2 + 20y^3;
    the roots of P map to z through y = (2 - z - 1/z) / 4, the three roots inside the unit circle give the
    minimum-phase ("extremal phase") scaling filter h, normalised to sum sqrt(2).  Conventions of `pywt`
    (which `models/fftencoder.py:62` takes its filters from): dec_lo = h reversed, dec_hi[k] = -(-1)^k h[k]."""
    y_roots = np.roots([20.0, 10.0, 4.0, 1.0])
    z_roots = []
    for y in y_roots:
        pair = np.roots([1.0, -(2.0 - 4.0 * y), 1.0])
        z_roots.append(pair[np.argmin(np.abs(pair))])
    h = np.poly(np.concatenate([-np.ones(4), np.array(z_roots)])).real
    h *= np.sqrt(2.0) / h.sum()
    dec_lo = h[::-1].copy()
    dec_hi = np.array([-((-1) ** k) * h[k] for k in range(8)])
    return dec_lo.astype(np.float32), dec_hi.astype(np.float32)


def wave_sizes(segment_len: int):
    """(per-level coefficient counts finest first, total row length) of the encoder's transform."""
    levels = (ctypes.c_int32 * 16)()
    total = _nat.lib().mvpa_wave_encode_size(int(segment_len), levels, 16)
    sizes, n = [], segment_len
    while len(sizes) < 16 and levels[len(sizes)] > 0:
        sizes.append(int(levels[len(sizes)]))
    return sizes, int(total)


def wave_encode(x, ln_weight, eps=1e-5, pad_to=None):
    """x (rows, len) fp32 / bf16 -> (rows, pad_to or total) in ln_weight's dtype: wavelet coefficients of every
    level, RMS-normalised and scaled by ln_weight; columns past the coefficient count are zero."""
    _need_cuda(x, ln_weight)
    rows, n = x.shape
    assert x.stride(1) == 1
    _, total = wave_sizes(n)
    ld_out = total if pad_to is None else int(pad_to)
    assert ln_weight.numel() == total and ln_weight.is_contiguous()
    out = torch.empty((rows, ld_out), dtype=ln_weight.dtype, device=x.device)
    lo, hi = db4_filters()
    fp = ctypes.POINTER(ctypes.c_float)
    with torch.cuda.device(x.device):
        st = _nat.lib().mvpa_wave_encode(x.data_ptr(), x.stride(0), _code(x), lo.ctypes.data_as(fp), hi.ctypes.data_as(fp),
                                         ln_weight.data_ptr(), out.data_ptr(), ld_out, _code(ln_weight), rows, n,
                                         float(eps), _stream(x))
    _nat.check(st, "mvpa_wave_encode")
    return out


def channel_mean(h):
    """h (B,T,C,E) -> (B,E): mean over the channels of the last time step."""
    _need_cuda(h)
    B, T, C, E = h.shape
    assert h.is_contiguous()
    out = torch.empty((B, E), dtype=h.dtype, device=h.device)
    with torch.cuda.device(h.device):
        st = _nat.lib().mvpa_channel_mean(h.data_ptr(), out.data_ptr(), B, T, C, E, _code(h), _stream(h))
    _nat.check(st, "mvpa_channel_mean")
    return out


def contrastive_logits(pred, enc, negatives, temperature):
    """pred, enc (B,T,C,E); negatives (B,T,C,K) int32 rows of enc.view(-1, E).  Returns (B*(T-1)*C, 1+K) fp32."""
    _need_cuda(pred, enc, negatives)
    B, T, C, E = pred.shape
    K = negatives.shape[-1]
    assert enc.shape == pred.shape and pred.is_contiguous() and enc.is_contiguous() and enc.dtype == pred.dtype
    assert negatives.dtype == torch.int32 and negatives.is_contiguous() and negatives.shape[:3] == (B, T, C)
    out = torch.empty((B * (T - 1) * C, K + 1), dtype=torch.float32, device=pred.device)
    with torch.cuda.device(pred.device):
        st = _nat.lib().mvpa_contrastive_logits(pred.data_ptr(), enc.data_ptr(), negatives.data_ptr(), out.data_ptr(), B, T,
                                                C, E, K, float(temperature), _code(pred), _stream(pred))
    _nat.check(st, "mvpa_contrastive_logits")
    return out
