"""CPU: the model-level restatement (`oracle/mvpformer_port_torch.py`) against the fixture written from the
reference's own `MVPFormerModel`, `MVPFormerHead` and `_contrastive_logits`
(`tests/golden/make_model_golden.py`), and the wavelet front end (unpinned: `ptwt` is not installed where the
fixtures are made) through the properties of the transform."""
import os

import numpy as np
import torch

import mvpformer_port_torch as mp
from conftest import GOLDEN, PKG  # noqa: F401  (PKG is on sys.path)

import mvpa_ops


def load_model_golden():
    g = dict(np.load(os.path.join(GOLDEN, "model_tiny.npz")))
    keys = ("n_positions", "n_channels", "n_embd", "n_layer", "n_head", "n_head_kv", "n_inner")
    cfg = {k: int(v) for k, v in zip(keys, g["cfg"])}
    cfg["eps"] = float(g["eps"])
    state = {k[6:]: torch.tensor(v) for k, v in g.items() if k.startswith("state.")}
    return g, cfg, state


def test_model_port_matches_reference_model():
    g, cfg, state = load_model_golden()
    out = mp.model(torch.tensor(g["x"]), state, cfg)
    assert np.abs(out.numpy() - g["out"]).max() <= 2e-5 * np.abs(g["out"]).max()
    # the fixture's parameters make the attention matter: dropping it changes the output visibly
    no_attn = {k: (torch.zeros_like(v) if k.endswith("c_proj.weight") else v) for k, v in state.items()}
    assert np.abs(mp.model(torch.tensor(g["x"]), no_attn, cfg).numpy() - g["out"]).max() > 1e-2


def test_heads_match_reference():
    g, cfg, state = load_model_golden()
    out = torch.tensor(g["out"])
    cls = mp.classification_logits(out, torch.tensor(g["head_cls"]))
    assert np.abs(cls.numpy() - g["cls_logits"]).max() <= 1e-6
    logits = mp.contrastive_logits(torch.tensor(g["pred"]), torch.tensor(g["x"]), torch.tensor(g["neg_idx"]),
                                   float(g["temp"]))
    assert logits.shape == g["con_logits"].shape
    assert np.abs(logits.numpy() - g["con_logits"]).max() <= 1e-5


def test_db4_filters_are_the_published_wavelet():
    lo, hi = (x.astype(np.float64) for x in mvpa_ops.db4_filters())
    # first taps of the scaling filter h = dec_lo reversed (Daubechies 1988, N = 4, to 7 places)
    assert np.allclose(lo[::-1][:4], [0.2303778, 0.7148466, 0.6308808, -0.0279838], atol=2e-7)
    assert abs(lo.sum() - np.sqrt(2)) < 1e-6 and abs(hi.sum()) < 1e-6
    for shift in range(4):                                   # orthonormal under even shifts
        a = np.dot(lo[2 * shift:], lo[:8 - 2 * shift])
        assert abs(a - (1.0 if shift == 0 else 0.0)) < 1e-6
        assert abs(np.dot(lo[2 * shift:], hi[:8 - 2 * shift])) < 1e-6
    k = np.arange(8)
    for m in range(4):                                       # four vanishing moments
        assert abs(np.dot(hi, k ** m)) < 1e-4


def test_wavedec_layout_and_energy():
    lo, hi = (torch.tensor(x) for x in mvpa_ops.db4_filters())
    sizes, total = mvpa_ops.wave_sizes(2560)
    assert sizes == [1283, 645, 326, 166, 86, 46, 26, 16] and total == 2610      # `_compute_dwt_size`, 5 s at 512 Hz
    torch.manual_seed(0)
    x = torch.randn(3, 256, dtype=torch.float64)
    coef = mp.wavedec_periodic(x, lo.double(), hi.double())
    s256, t256 = mvpa_ops.wave_sizes(256)
    assert coef.shape == (3, t256) and t256 == sum(s256) + s256[-1]
    # one level on an even length: the periodic transform is orthogonal up to its redundant wrap-around
    # coefficients (n/2 + 3 per band instead of n/2): dropping the 3 repeats leaves the energy of x
    one = mp.wavedec_periodic(x[:, :16], lo.double(), hi.double())                # 16 samples: exactly one level
    a, d = one[:, :11], one[:, 11:]
    assert torch.allclose(a[:, :3], a[:, 8:], atol=1e-12) and torch.allclose(d[:, :3], d[:, 8:], atol=1e-12)
    energy = (a[:, 3:] ** 2).sum(-1) + (d[:, 3:] ** 2).sum(-1)
    assert torch.allclose(energy, (x[:, :16] ** 2).sum(-1), atol=1e-9)
    # a constant signal has no detail
    c = mp.wavedec_periodic(torch.ones(1, 64, dtype=torch.float64), lo.double(), hi.double())
    assert c[:, mvpa_ops.wave_sizes(64)[0][-1]:].abs().max() < 1e-6
