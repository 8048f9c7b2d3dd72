"""GPU parity tests of the operator, through `attentions.flashmvpa` -> ctypes -> C ABI.

Tolerances (against the fp32/fp64 oracle on the same inputs):
  fp32 I/O : max-abs error <= 1e-4 * max|reference|
  bf16 I/O : max-abs error <= 2e-2   (inputs rounded to bf16 first, oracle fed the rounded values)
  fp16 I/O : max-abs error <= 4e-3 * max(1, max|reference|)   (same, rounded to fp16; fp32 arithmetic inside)
"""
import numpy as np
import pytest
import torch

import mvpa_oracle as mo
from conftest import golden_op_cases, load_golden

pytestmark = pytest.mark.gpu

GRADS = ("dq", "du", "dv", "dz", "dk", "dr_time", "dr_chan", "dval")
F32_REL = 1e-4
BF16_ABS = 2e-2
F16_ABS = 4e-3


def _op(dev, g, dtype, grads=False, window=10):
    import attentions
    B, H, Hkv, T, C, D = (int(x) for x in g["dims"])
    t = {k: torch.tensor(np.asarray(g[k], np.float32), device=dev, dtype=dtype, requires_grad=grads)
         for k in ("q", "u", "v", "z", "k", "r_time", "r_chan", "val")}
    o = attentions.flashmvpa(
        t["q"], t["u"].view(1, Hkv, 1, D), t["v"].view(1, Hkv, 1, D), t["z"].view(1, Hkv, 1, D),
        t["k"], t["r_time"].view(1, Hkv, T, D), t["r_chan"].view(1, Hkv, C, D), t["val"],
        causal=True, sm_scale=float(g["sm_scale"]), window_size=window, p_drop=0,
        rel_bias_chan=True, rel_bias_time=True)
    return o, t


def _np(x):
    return x.detach().float().cpu().numpy()


def _rounded(g, dtype=torch.bfloat16):
    """Copy of a case with every input rounded to bf16 / fp16 (what those kernels actually see)."""
    r = dict(g)
    for k in ("q", "u", "v", "z", "k", "r_time", "r_chan", "val", "do"):
        if k in r:
            r[k] = torch.tensor(r[k]).to(dtype).float().numpy()
    return r


def random_case(seed, B, H, Hkv, T, C, D, scale=1.0):
    rng = np.random.default_rng(seed)
    N = T * C
    f = lambda *s: (scale * rng.standard_normal(s)).astype(np.float32)
    return dict(q=f(B, H, N, D), k=f(B, Hkv, N, D), val=f(B, Hkv, N, D), u=f(Hkv, D), v=f(Hkv, D),
                z=f(Hkv, D), r_time=f(Hkv, T, D), r_chan=f(Hkv, C, D), do=f(B, H, N, D),
                dims=np.array([B, H, Hkv, T, C, D]), sm_scale=np.float64(D ** -0.5))


def _oracle_args(g):
    return (g["q"], g["u"], g["v"], g["z"], g["k"], g["r_time"], g["r_chan"], g["val"])


@pytest.mark.parametrize("name", golden_op_cases())
def test_fp32_forward_vs_reference_golden(cuda, name):
    g = load_golden(name)
    o, _ = _op(cuda, g, torch.float32)
    assert np.abs(_np(o) - g["o"]).max() <= F32_REL * np.abs(g["o"]).max()


@pytest.mark.parametrize("name", [n for n in golden_op_cases() if n != "cfg1"])
def test_fp32_backward_vs_reference_golden(cuda, name):
    g = load_golden(name)
    o, t = _op(cuda, g, torch.float32, grads=True)
    o.backward(torch.tensor(g["do"], device=cuda))
    for key, gk in zip(("q", "u", "v", "z", "k", "r_time", "r_chan", "val"), GRADS):
        ref = g[gk]
        err = np.abs(_np(t[key].grad).reshape(ref.shape) - ref).max()
        assert err <= F32_REL * max(1.0, np.abs(ref).max()), (gk, err)


@pytest.mark.parametrize("name", golden_op_cases())
def test_bf16_forward_vs_oracle_on_golden_inputs(cuda, name):
    g = _rounded(load_golden(name))
    ref, _ = mo.mvpa_forward(*_oracle_args(g), float(g["sm_scale"]))
    o, _ = _op(cuda, g, torch.bfloat16)
    assert np.abs(_np(o) - ref).max() <= BF16_ABS


@pytest.mark.parametrize("name", ["gqa2_t24_c5", "t11_c4", "t16_c16_d64", "t6_c22_d64", "t2_c128_d128"])
def test_bf16_backward_vs_oracle_on_golden_inputs(cuda, name):
    g = _rounded(load_golden(name))
    ref = mo.mvpa_backward(*_oracle_args(g), g["do"], float(g["sm_scale"]))
    o, t = _op(cuda, g, torch.bfloat16, grads=True)
    o.backward(torch.tensor(g["do"], device=cuda, dtype=torch.bfloat16))
    for key, gk in zip(("q", "u", "v", "z", "k", "r_time", "r_chan", "val"), GRADS):
        r = ref[gk]
        err = np.abs(_np(t[key].grad).reshape(r.shape) - r).max()
        assert err <= BF16_ABS * max(1.0, np.abs(r).max()), (gk, err)


SHAPES = [  # B, H, Hkv, T, C, D
    (1, 2, 2, 24, 32, 64),    # mixed window tiles
    (2, 2, 1, 13, 64, 64),    # GQA g=2, two time steps per 128-key tile
    (1, 2, 2, 14, 128, 64),   # one time step per tile, light tiles appear (t >= 11)
    (1, 2, 1, 12, 128, 128),  # D=128
    (1, 3, 1, 16, 22, 64),    # g=3, ragged channels
    (1, 1, 1, 30, 16, 64),
    (1, 2, 2, 3, 100, 128),
    (1, 1, 1, 40, 7, 32),
    (1, 1, 1, 9, 130, 16),
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_forward_random_shapes_vs_oracle(cuda, shape, dtype):
    g = random_case(100 + sum(shape), *shape)
    dt = getattr(torch, dtype)
    if dt == torch.bfloat16:
        g = _rounded(g)
    ref, lse = mo.mvpa_forward(*_oracle_args(g), float(g["sm_scale"]))
    o, _ = _op(cuda, g, dt)
    err = np.abs(_np(o) - ref).max()
    assert err <= (BF16_ABS if dt == torch.bfloat16 else F32_REL * np.abs(ref).max()), err


@pytest.mark.parametrize("shape", [(1, 2, 1, 13, 16, 64), (1, 2, 2, 12, 32, 32), (1, 1, 1, 3, 128, 128)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_backward_random_shapes_vs_oracle(cuda, shape, dtype):
    g = random_case(200 + sum(shape), *shape)
    dt = getattr(torch, dtype)
    if dt == torch.bfloat16:
        g = _rounded(g)
    ref = mo.mvpa_backward(*_oracle_args(g), g["do"], float(g["sm_scale"]))
    o, t = _op(cuda, g, dt, grads=True)
    o.backward(torch.tensor(g["do"], device=cuda, dtype=dt))
    tol = BF16_ABS if dt == torch.bfloat16 else F32_REL
    for key, gk in zip(("q", "u", "v", "z", "k", "r_time", "r_chan", "val"), GRADS):
        r = ref[gk]
        err = np.abs(_np(t[key].grad).reshape(r.shape) - r).max()
        assert err <= tol * max(1.0, np.abs(r).max()), (gk, err)


@pytest.mark.parametrize("shape", [(1, 2, 1, 13, 16, 64), (2, 2, 2, 5, 33, 128), (1, 3, 1, 12, 32, 32),
                                   (1, 1, 1, 14, 128, 64)])
def test_fp16_forward_and_backward_vs_oracle(cuda, shape):
    """The reference operator takes fp16 as well as bf16 / fp32 (`attn.py:1013-1138` has no dtype check
    beyond "all equal"); here fp16 runs on the fp32-arithmetic kernels, so only I/O rounding shows."""
    g = _rounded(random_case(300 + sum(shape), *shape), torch.float16)
    ref_o, _ = mo.mvpa_forward(*_oracle_args(g), float(g["sm_scale"]))
    ref = mo.mvpa_backward(*_oracle_args(g), g["do"], float(g["sm_scale"]))
    o, t = _op(cuda, g, torch.float16, grads=True)
    assert o.dtype == torch.float16
    assert np.abs(_np(o) - ref_o).max() <= F16_ABS * max(1.0, np.abs(ref_o).max())
    o.backward(torch.tensor(g["do"], device=cuda, dtype=torch.float16))
    for key, gk in zip(("q", "u", "v", "z", "k", "r_time", "r_chan", "val"), GRADS):
        r = ref[gk]
        assert t[key].grad.dtype == torch.float16
        err = np.abs(_np(t[key].grad).reshape(r.shape) - r).max()
        assert err <= F16_ABS * max(1.0, np.abs(r).max()), (gk, err)


def test_no_window_flag(cuda):
    g = random_case(7, 1, 2, 2, 14, 8, 32)
    ref, _ = mo.mvpa_forward(*_oracle_args(g), float(g["sm_scale"]), window=10 ** 6)
    o, _ = _op(cuda, g, torch.float32, window=0)   # reference: window_size=0 means not windowed
    assert np.abs(_np(o) - ref).max() <= F32_REL * np.abs(ref).max()


# window variants of the tensor-core kernels: not windowed (0), narrower than a tile (1, 3), wider than the
# sequence (T + 5); one shape with four time steps per tile (C <= 32), one with a single time step per tile
# and T large enough for tiles wholly outside the window (C = 128), and the degenerate T = 1 / C = 1.
WINDOW_SHAPES = [(1, 2, 1, 24, 32, 64), (1, 2, 2, 16, 128, 64), (1, 2, 1, 14, 100, 128), (1, 2, 2, 20, 60, 128)]


@pytest.mark.parametrize("window", [0, 1, 3, "T+5"])
@pytest.mark.parametrize("shape", WINDOW_SHAPES)
def test_bf16_window_variants_forward_and_backward_vs_oracle(cuda, shape, window):
    T = shape[3]
    w = T + 5 if window == "T+5" else window
    g = _rounded(random_case(400 + sum(shape) + w, *shape))
    w_oracle = 10 ** 6 if w == 0 else w       # the reference's window_size = 0 means "not windowed"
    ref_o, _ = mo.mvpa_forward(*_oracle_args(g), float(g["sm_scale"]), window=w_oracle)
    ref = mo.mvpa_backward(*_oracle_args(g), g["do"], float(g["sm_scale"]), window=w_oracle)
    o, t = _op(cuda, g, torch.bfloat16, grads=True, window=w)
    assert np.abs(_np(o) - ref_o).max() <= BF16_ABS
    o.backward(torch.tensor(g["do"], device=cuda, dtype=torch.bfloat16))
    for key, gk in zip(("q", "u", "v", "z", "k", "r_time", "r_chan", "val"), GRADS):
        r = ref[gk]
        err = np.abs(_np(t[key].grad).reshape(r.shape) - r).max()
        assert err <= BF16_ABS * max(1.0, np.abs(r).max()), (gk, err)


@pytest.mark.parametrize("shape", [(1, 2, 2, 1, 64, 64), (1, 2, 1, 1, 128, 128), (1, 2, 2, 40, 1, 64),
                                   (1, 2, 1, 128, 1, 128)])
def test_bf16_single_time_step_or_channel_on_the_tensor_cores(cuda, shape):
    """T = 1 and C = 1 at head dims 64 / 128, i.e. on the tensor-core kernels (the goldens cover these
    two edge cases at D = 16, which the CUDA-core kernels take)."""
    g = _rounded(random_case(500 + sum(shape), *shape))
    ref_o, _ = mo.mvpa_forward(*_oracle_args(g), float(g["sm_scale"]))
    ref = mo.mvpa_backward(*_oracle_args(g), g["do"], float(g["sm_scale"]))
    o, t = _op(cuda, g, torch.bfloat16, grads=True)
    assert np.abs(_np(o) - ref_o).max() <= BF16_ABS
    o.backward(torch.tensor(g["do"], device=cuda, dtype=torch.bfloat16))
    for key, gk in zip(("q", "u", "v", "z", "k", "r_time", "r_chan", "val"), GRADS):
        r = ref[gk]
        err = np.abs(_np(t[key].grad).reshape(r.shape) - r).max()
        # With a single time step (or channel) that relative score is the same for every key of a row, so its
        # gradient is a row sum of dS, exactly zero: what the kernels return there is the bf16 rounding of dS
        # (delta is taken from the bf16-rounded O, so sum_k P (dP - delta) is off by ~0.4 % of delta per row)
        # summed over all rows, which does not scale with the (zero) reference; the fp32 goldens pin the zero.
        cancels = (gk in ("dr_time", "dv") and shape[3] == 1) or (gk in ("dr_chan", "dz") and shape[4] == 1)
        tol = 0.25 if cancels else BF16_ABS * max(1.0, np.abs(r).max())
        assert err <= tol, (gk, err)


def test_strided_inputs_match_contiguous(cuda):
    """Heads may be handed over as strided views of a (B, N, H, D) buffer."""
    import attentions
    g = random_case(9, 2, 4, 2, 6, 16, 64)
    B, H, Hkv, T, C, D = (int(x) for x in g["dims"])
    tt = {k: torch.tensor(g[k], device=cuda) for k in g if k not in ("dims", "sm_scale")}
    kw = dict(causal=True, sm_scale=float(g["sm_scale"]), window_size=10)
    bias = [tt[k].view(1, Hkv, 1, D) for k in ("u", "v", "z")]
    rel = [tt["r_time"].view(1, Hkv, T, D), tt["r_chan"].view(1, Hkv, C, D)]
    o1 = attentions.flashmvpa(tt["q"], *bias, tt["k"], *rel, tt["val"], **kw)
    qs = tt["q"].permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    ks = tt["k"].permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    vs = tt["val"].permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    assert not qs.is_contiguous()
    o2 = attentions.flashmvpa(qs, *bias, ks, *rel, vs, **kw)
    assert o2.stride() == qs.stride()
    assert torch.equal(o1, o2)


@pytest.mark.parametrize("shape", [(2, 4, 2, 12, 32, 64), (1, 2, 1, 13, 128, 128)])
def test_bf16_backward_strided_inputs_match_contiguous(cuda, shape):
    """The layer hands the tensor-core kernels strided head views of (B, N, heads, D) projection
    buffers and autograd hands back a strided dO: gradients must equal those of the contiguous call
    (dq, dk, dv bit for bit; the relative-key and bias gradients are summed with atomics, so to 1e-2)."""
    import attentions
    g = random_case(11, *shape)
    B, H, Hkv, T, C, D = shape
    kw = dict(causal=True, sm_scale=float(g["sm_scale"]), window_size=10)
    bf = lambda a: torch.tensor(a, device=cuda, dtype=torch.bfloat16)

    def run(strided):
        small = {k: bf(g[k]).requires_grad_(True) for k in ("u", "v", "z", "r_time", "r_chan")}
        big = {}
        for k in ("q", "k", "val"):
            x = bf(g[k])
            big[k] = (x.permute(0, 2, 1, 3).contiguous() if strided else x).requires_grad_(True)
        view = (lambda x: x.permute(0, 2, 1, 3)) if strided else (lambda x: x)
        do = bf(g["do"])
        if strided:
            do = do.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
            assert not view(big["q"]).is_contiguous() and not do.is_contiguous()
        o = attentions.flashmvpa(view(big["q"]), *[small[k].view(1, Hkv, 1, D) for k in ("u", "v", "z")],
                                 view(big["k"]), small["r_time"].view(1, Hkv, T, D),
                                 small["r_chan"].view(1, Hkv, C, D), view(big["val"]), **kw)
        o.backward(do)
        grads = {k: view(big[k].grad) for k in big}
        grads.update({k: small[k].grad for k in small})
        return o, grads

    o1, g1 = run(False)
    o2, g2 = run(True)
    assert torch.equal(o1, o2)
    for k in ("q", "k", "val"):
        assert torch.equal(g1[k], g2[k]), k
    for k in ("u", "v", "z", "r_time", "r_chan"):
        a, b = g1[k].float(), g2[k].float()
        assert (a - b).abs().max() <= 1e-2 * max(1.0, a.abs().max().item()), k


@pytest.mark.parametrize("off", ["time", "chan"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_relative_term_switched_off(cuda, off, dtype):
    """`rel_bias_time=False` / `rel_bias_chan=False`: the reference kernels skip that term only
    (`attn.py:187-216`); oracle = the same attention with that term's relative key at zero."""
    import attentions
    shape = (1, 2, 1, 13, 32, 64)
    B, H, Hkv, T, C, D = shape
    dt = getattr(torch, dtype)
    g = random_case(400, *shape)
    if dt == torch.bfloat16:
        g = _rounded(g)
    gz = dict(g)
    gz["r_time" if off == "time" else "r_chan"] = np.zeros_like(g["r_time" if off == "time" else "r_chan"])
    ref_o, _ = mo.mvpa_forward(*_oracle_args(gz), float(g["sm_scale"]))
    ref = mo.mvpa_backward(*_oracle_args(gz), g["do"], float(g["sm_scale"]))
    t = {k: torch.tensor(g[k], device=cuda, dtype=dt, requires_grad=True)
         for k in ("q", "u", "v", "z", "k", "r_time", "r_chan", "val")}
    o = attentions.flashmvpa(
        t["q"], t["u"].view(1, Hkv, 1, D), t["v"].view(1, Hkv, 1, D), t["z"].view(1, Hkv, 1, D),
        t["k"], t["r_time"].view(1, Hkv, T, D), t["r_chan"].view(1, Hkv, C, D), t["val"],
        causal=True, sm_scale=float(g["sm_scale"]), window_size=10, p_drop=0,
        rel_bias_time=off != "time", rel_bias_chan=off != "chan")
    tol = BF16_ABS if dt == torch.bfloat16 else F32_REL
    assert np.abs(_np(o) - ref_o).max() <= tol * max(1.0, np.abs(ref_o).max())
    o.backward(torch.tensor(g["do"], device=cuda, dtype=dt))
    dead = ("r_time", "v") if off == "time" else ("r_chan", "z")   # the skipped term's key and query bias
    for key, gk in zip(("q", "u", "v", "z", "k", "r_time", "r_chan", "val"), GRADS):
        if key in dead:
            assert float(t[key].grad.abs().max()) == 0.0, key
            continue
        r = ref[gk]
        err = np.abs(_np(t[key].grad).reshape(r.shape) - r).max()
        assert err <= tol * max(1.0, np.abs(r).max()), (gk, err)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_structured_dropout_is_a_key_mask_on_v(cuda, dtype):
    """`p_drop > 0` (`attn.py:1052-1062, 316-321`): key time steps and key channels are dropped with
    probability 1 - sqrt(1 - p) each, kept probabilities divided by 1 - p after the softmax sum.
    Oracle: the same draws from a generator seeded alike (channels first, then time steps), applied
    to V.  Forward and all gradients."""
    import math
    import attentions
    shape = (1, 2, 1, 13, 32, 64)
    B, H, Hkv, T, C, D = shape
    p_drop = 0.3
    dt = getattr(torch, dtype)
    g = random_case(500, *shape)
    if dt == torch.bfloat16:
        g = _rounded(g)
    gen = torch.Generator(device=cuda).manual_seed(1234)
    p_dim = 1 - math.sqrt(1 - p_drop)
    chan_keep = (torch.rand(C, device=cuda, generator=gen) > p_dim).cpu().numpy()
    time_keep = (torch.rand(T, device=cuda, generator=gen) > p_dim).cpu().numpy()
    keep = (time_keep[:, None] & chan_keep[None, :]).reshape(1, 1, T * C, 1)
    assert 0 < keep.sum() < keep.size                      # the seed drops something and keeps something
    scale = keep.astype(np.float32) / (1 - p_drop)
    gd = dict(g)
    gd["val"] = g["val"] * scale
    ref_o, _ = mo.mvpa_forward(*_oracle_args(gd), float(g["sm_scale"]))
    ref = dict(mo.mvpa_backward(*_oracle_args(gd), g["do"], float(g["sm_scale"])))
    ref["dval"] = ref["dval"] * scale                        # chain rule through the mask
    t = {k: torch.tensor(g[k], device=cuda, dtype=dt, requires_grad=True)
         for k in ("q", "u", "v", "z", "k", "r_time", "r_chan", "val")}
    o = attentions.flashmvpa(
        t["q"], t["u"].view(1, Hkv, 1, D), t["v"].view(1, Hkv, 1, D), t["z"].view(1, Hkv, 1, D),
        t["k"], t["r_time"].view(1, Hkv, T, D), t["r_chan"].view(1, Hkv, C, D), t["val"],
        causal=True, sm_scale=float(g["sm_scale"]), window_size=10, p_drop=p_drop,
        generator=torch.Generator(device=cuda).manual_seed(1234))
    tol = 3e-2 if dt == torch.bfloat16 else F32_REL           # bf16: 2e-2 on the kernel output, scaled by 1 / (1 - p)
    assert np.abs(_np(o) - ref_o).max() <= tol * max(1.0, np.abs(ref_o).max())
    o.backward(torch.tensor(g["do"], device=cuda, dtype=dt))
    for key, gk in zip(("q", "u", "v", "z", "k", "r_time", "r_chan", "val"), GRADS):
        r = ref[gk]
        err = np.abs(_np(t[key].grad).reshape(r.shape) - r).max()
        assert err <= tol * max(1.0, np.abs(r).max()), (gk, err)
