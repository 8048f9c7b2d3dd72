"""CPU: the numpy oracle and its torch port against the reference's own outputs
(`tests/golden/*.npz`, produced by `tests/golden/make_golden.py`)."""
import numpy as np
import pytest
import torch

import mvpa_oracle as mo
import mvpa_port_torch as mp
from conftest import golden_op_cases, load_golden

GRADS = ("dq", "du", "dv", "dz", "dk", "dr_time", "dr_chan", "dval")


def _args(g):
    return (g["q"], g["u"], g["v"], g["z"], g["k"], g["r_time"], g["r_chan"], g["val"])


@pytest.mark.parametrize("name", golden_op_cases())
def test_forward_matches_reference(name):
    g = load_golden(name)
    o, lse = mo.mvpa_forward(*_args(g), float(g["sm_scale"]))
    assert np.abs(o - g["o"]).max() < 5e-6
    assert np.isfinite(lse).all()


@pytest.mark.parametrize("name", [n for n in golden_op_cases() if n != "cfg1"])
def test_backward_matches_reference(name):
    g = load_golden(name)
    gr = mo.mvpa_backward(*_args(g), g["do"], float(g["sm_scale"]))
    for k in GRADS:
        scale = max(1.0, np.abs(g[k]).max())
        assert np.abs(gr[k] - g[k]).max() / scale < 5e-6, k


@pytest.mark.parametrize("name", ["gqa2_t24_c5", "t11_c4", "t6_c22_d64"])
def test_torch_port_matches_reference(name):
    g = load_golden(name)
    t = [torch.tensor(a, requires_grad=True) for a in _args(g)]
    o = mp.rel_attn(*t, float(g["sm_scale"]))
    assert (o.detach().numpy() - g["o"]).__abs__().max() < 5e-6
    o.backward(torch.tensor(g["do"]))
    for x, k in zip(t, ("dq", "du", "dv", "dz", "dk", "dr_time", "dr_chan", "dval")):
        assert np.abs(x.grad.numpy() - g[k]).max() / max(1.0, np.abs(g[k]).max()) < 5e-6, k


@pytest.mark.parametrize("T,C", [(1, 1), (1, 5), (11, 3), (12, 16), (25, 22), (5, 64)])
def test_index_maps_equal_rel_shift(T, C):
    """Closed-form index maps vs a literal pad-and-reshape shift (`layers/mvpa.py:127-159`)."""
    N = T * C
    x = np.arange(N * T, dtype=np.int64).reshape(N, T)
    # Transformer-XL shift: view as (T, N), prepend a zero row, view back, drop first row
    padded = np.concatenate([np.zeros((T, 1), np.int64), x.reshape(T, N)], axis=1).reshape(N + 1, T)
    shifted = padded[1:].reshape(N, T)                       # shifted[i, j]
    tidx = mo.rel_time_index(T, C)
    tt = np.arange(N) // C
    for i in range(0, N, max(1, N // 17)):
        for k in range(N):
            if tt[k] <= tt[i]:
                # `repeat_channel` expands time columns over channels (`layers/mvpa.py:227`)
                assert shifted[i, tt[k]] == x[i, tidx[i, k]]
    cidx = mo.rel_chan_index(T, C)
    cc = np.arange(N) % C
    assert (cidx == C - 1 - np.abs(cc[:, None] - cc[None, :])).all()
    assert cidx.min() >= 0 and cidx.max() == C - 1


def test_window_last_row_and_zero_fill():
    """Outside the window the content term is zeroed, not masked, and the last time row sees all
    content (`layers/mvpa.py:230-245`)."""
    rng = np.random.default_rng(0)
    B, H, T, C, D = 1, 1, 14, 2, 8
    N = T * C
    q, k, v = (rng.standard_normal((B, H, N, D)) for _ in range(3))
    z0 = np.zeros((1, D))
    rt, rc = np.zeros((1, T, D)), np.zeros((1, C, D))
    o, _, p = mo.mvpa_forward(q, z0, z0, z0, k, rt, rc, v, 1.0, window=10, return_probs=True)
    i = 12 * C          # time 12: keys at time 0,1 are outside the window -> score 0, weight > 0
    assert (p[0, 0, i, : 2 * C] > 0).all()
    s = q[0, 0, i] @ k[0, 0].T
    s[: 2 * C] = 0.0
    s = s[: 13 * C]
    ref = np.exp(s - s.max()); ref /= ref.sum()
    assert np.abs(p[0, 0, i, : 13 * C] - ref).max() < 1e-12
    j = 13 * C          # last time row: full content everywhere
    s = q[0, 0, j] @ k[0, 0].T
    ref = np.exp(s - s.max()); ref /= ref.sum()
    assert np.abs(p[0, 0, j] - ref).max() < 1e-12


def test_flop_count_matches_baseline_table():
    f = mo.algorithmic_flops(4, 16, 64, 64, 64)
    assert f["p_c"] == 8519680 and f["p_w"] == 2875392
    assert abs(f["f_alg"] / 1e12 - 0.0976) < 1e-3 and abs(f["f_dense"] / 1e12 - 0.1396) < 1e-3


def test_staged_reference_layer_agrees_with_the_port():
    """Where the build has staged the reference's own layer under baseline/_ref/ (the CPU arm of the
    benchmark then times it instead of the port), both give the same attention output on the same draws."""
    import importlib.util
    import os
    import sys

    import pytest
    import torch
    from conftest import ROOT
    spec = importlib.util.spec_from_file_location("bench_for_test", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    argv, sys.argv = sys.argv, ["bench.py"]
    try:
        spec.loader.exec_module(bench)
    finally:
        sys.argv = argv
    if bench.reference_layer_class() is None:
        pytest.skip("baseline/_ref/ is not staged here")
    sample = dict(B=1, H=4, Hkv=2, T=13, C=6, D=16, window=10)
    fn, kind = bench.cpu_attention(sample, seed=3)
    assert kind == "reference"
    with torch.no_grad():
        ref = fn()[0]                                        # (B,H,T,C,D)
    bench._REF_LAYER = False                                 # the same draws through the port
    fn2, kind2 = bench.cpu_attention(sample, seed=3)
    assert kind2 == "port"
    with torch.no_grad():
        out = fn2()                                          # (B,H,N,D)
    assert (ref.reshape(out.shape) - out).abs().max() <= 5e-6
