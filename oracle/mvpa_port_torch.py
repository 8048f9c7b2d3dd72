"""Torch (CPU) port of the reference's materialised PyTorch attention.

TEST / BASELINE INFRASTRUCTURE ONLY: the timed CPU arm of `bench.py` and an
autograd cross-check in `tests/`.  The product path never imports this file.

It performs the same sequence of dense operations as
`MVPFormerGQAAttention._rel_attn` (`layers/mvpa.py:173-278`) — three batched
matmuls, two gathers, window zero-fill, scaling, time-block causal mask,
softmax over a materialised (N,N) matrix and the PV matmul — so its run time on
the host cores stands in for the reference's CPU path, which cannot be
imported where the reference checkout is absent.  Index maps are built in closed
form instead of by the reference's pad-and-reshape.
"""
from __future__ import annotations

import torch


def rel_attn(q, u, v, z, k, r_time, r_chan, val, sm_scale, window=10):
    """q (B,H,N,D); u,v,z (Hkv,D); k,val (B,Hkv,N,D); r_time (Hkv,T,D); r_chan (Hkv,C,D).

    Returns o (B,H,N,D).  Differentiable through torch autograd.
    """
    B, H, N, D = q.shape
    Hkv = k.shape[1]
    g = H // Hkv
    T, C = r_time.shape[-2], r_chan.shape[-2]
    assert N == T * C

    def heads(x):  # (.., Hkv, ..) -> H heads
        return x.repeat_interleave(g, dim=-3) if g > 1 else x

    u, v, z = (a.reshape(Hkv, 1, D) for a in (u, v, z))
    kk, vv = heads(k), heads(val)
    rt, rc = heads(r_time.reshape(Hkv, T, D)), heads(r_chan.reshape(Hkv, C, D))
    content = torch.matmul(q + heads(u), kk.transpose(-1, -2))  # layers/mvpa.py:222
    t_att = torch.matmul(q + heads(v), rt.transpose(-1, -2))    # layers/mvpa.py:223
    c_att = torch.matmul(q + heads(z), rc.transpose(-1, -2))    # layers/mvpa.py:224
    n = torch.arange(N, device=q.device)
    tt, cc = n // C, n % C
    dt = tt[:, None] - tt[None, :]
    tidx = (T - 1 - dt).clamp(0, T - 1)
    cidx = C - 1 - (cc[:, None] - cc[None, :]).abs()
    s = torch.gather(t_att, -1, tidx.expand(B, H, N, N)) \
        + torch.gather(c_att, -1, cidx.expand(B, H, N, N))      # layers/mvpa.py:225-229
    win = (dt.abs() <= window) | (tt[:, None] == T - 1)         # layers/mvpa.py:231-244
    s = s + content.masked_fill(~win, 0.0)                      # layers/mvpa.py:245
    s = s * sm_scale                                            # layers/mvpa.py:246-252
    s = s.masked_fill(dt < 0, torch.finfo(s.dtype).min)         # layers/mvpa.py:255-264
    p = torch.softmax(s, dim=-1)                                # layers/mvpa.py:272
    return torch.matmul(p, vv)                                  # layers/mvpa.py:277
