"""CPU: host logic of the layer shim (strided head views, state-dict names, return tuple) with
the oracle's torch port standing in for the CUDA operator, against the reference layer's own
output and gradients (`tests/golden/layer_*.npz`)."""
from types import SimpleNamespace as NS

import numpy as np
import pytest
import torch

import layers.mvpa as lm
import mvpa_port_torch as mp
from conftest import load_golden


def _cfg(H, Hkv, D, T):
    return NS(max_position_embeddings=T, hidden_size=H * D, num_attention_heads=H, n_head_kv=Hkv,
              n_inner=4 * H * D, global_att=True, scale_attn_weights=True,
              scale_attn_by_inverse_layer_idx=False, reorder_and_upcast_attn=False, lora=False,
              attn_pdrop=0.1, resid_pdrop=0.1)


def _cpu_op(q, u, v, z, k, rt, rc, val, causal, sm_scale, window_size=0, **kw):
    Hkv, D = k.shape[1], q.shape[-1]
    return mp.rel_attn(q, u.reshape(Hkv, D), v.reshape(Hkv, D), z.reshape(Hkv, D), k,
                       rt.reshape(Hkv, -1, D), rc.reshape(Hkv, -1, D), val, sm_scale, window_size)


@pytest.mark.parametrize("name", ["e64", "e128_mha"])
@pytest.mark.parametrize("cls", ["MVPFormerGQAFlashAttention", "MVPFormerGQAAttention"])
def test_layer_matches_reference_layer(monkeypatch, name, cls):
    g = load_golden(name, "layer")
    B, H, Hkv, T, C, D = (int(x) for x in g["dims"])
    monkeypatch.setattr(lm, "flashmvpa", _cpu_op)
    m = getattr(lm, cls)(_cfg(H, Hkv, D, T), layer_idx=0).eval()
    sd = {k[3:]: torch.tensor(v) for k, v in g.items() if k.startswith("sd.")}
    assert set(sd) == set(m.state_dict())            # same names as the reference module
    m.load_state_dict(sd, strict=True)
    x, pos, chan = (torch.tensor(g[k], requires_grad=True) for k in ("x", "pos", "chan"))
    out, present = m(x, pos, chan, use_cache=True)
    assert np.abs(out.detach().numpy() - g["out"]).max() < 2e-5
    assert np.abs(present[0].detach().numpy() - g["present_k"]).max() < 1e-6
    assert np.abs(present[1].detach().numpy() - g["present_v"]).max() < 1e-6
    out.backward(torch.tensor(g["gout"]))
    for t, k in ((x, "dx"), (pos, "dpos"), (chan, "dchan")):
        assert np.abs(t.grad.numpy() - g[k]).max() / max(1.0, np.abs(g[k]).max()) < 2e-5, k
    for k, p in m.named_parameters():
        ref = g["grad." + k]
        assert np.abs(p.grad.numpy() - ref).max() / max(1.0, np.abs(ref).max()) < 2e-5, k
    assert m(x, pos, chan, output_attentions=True)[1:] == (None, None)


def test_operator_refuses_cpu_tensors():
    import attentions
    q = torch.zeros(1, 2, 4, 16)
    b = torch.zeros(1, 2, 1, 16)
    with pytest.raises(RuntimeError, match="CUDA"):
        attentions.flashmvpa(q, b, b, b, q, torch.zeros(1, 2, 2, 16), torch.zeros(1, 2, 2, 16), q,
                             causal=True, sm_scale=0.25, window_size=10)
    with pytest.raises(NotImplementedError):   # both relative terms off: a plain windowed attention
        attentions.flashmvpa(q, b, b, b, q, torch.zeros(1, 2, 2, 16), torch.zeros(1, 2, 2, 16), q,
                             causal=True, sm_scale=0.25, window_size=10, rel_bias_time=False,
                             rel_bias_chan=False)
    with pytest.raises(ValueError):
        attentions.flashmvpa(q, b, b, b, q, torch.zeros(1, 2, 2, 16), torch.zeros(1, 2, 2, 16), q,
                             causal=True, sm_scale=0.25, window_size=10, p_drop=1.0)
    with pytest.raises(AssertionError):
        attentions.flashmvpa(q, b, b, b, q, torch.zeros(1, 2, 3, 16), torch.zeros(1, 2, 2, 16), q,
                             causal=True, sm_scale=0.25)
