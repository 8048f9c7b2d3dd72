"""GPU: the layer module on the CUDA kernels against the reference layer's own outputs and
gradients (`tests/golden/layer_*.npz`), fp32 and bf16, and its zero-copy head layout."""
from types import SimpleNamespace as NS

import numpy as np
import pytest
import torch

from conftest import load_golden

pytestmark = pytest.mark.gpu


def _cfg(H, Hkv, D, T):
    return NS(max_position_embeddings=T, hidden_size=H * D, num_attention_heads=H, n_head_kv=Hkv,
              n_inner=4 * H * D, global_att=True, scale_attn_weights=True,
              scale_attn_by_inverse_layer_idx=False, reorder_and_upcast_attn=False, lora=False,
              attn_pdrop=0.1, resid_pdrop=0.1)


@pytest.mark.parametrize("name", ["e64", "e128_mha"])
def test_layer_fp32_matches_reference_layer(cuda, name):
    import layers
    g = load_golden(name, "layer")
    B, H, Hkv, T, C, D = (int(x) for x in g["dims"])
    m = layers.MVPFormerGQAFlashAttention(_cfg(H, Hkv, D, T), layer_idx=0).eval().to(cuda)
    m.load_state_dict({k[3:]: torch.tensor(v) for k, v in g.items() if k.startswith("sd.")}, strict=True)
    x, pos, chan = (torch.tensor(g[k], device=cuda, requires_grad=True) for k in ("x", "pos", "chan"))
    out, present = m(x, pos, chan, use_cache=True)
    assert np.abs(out.detach().cpu().numpy() - g["out"]).max() <= 1e-4 * max(1.0, np.abs(g["out"]).max())
    assert np.abs(present[0].detach().cpu().numpy() - g["present_k"]).max() < 1e-5
    out.backward(torch.tensor(g["gout"], device=cuda))
    for t, k in ((x, "dx"), (pos, "dpos"), (chan, "dchan")):
        assert np.abs(t.grad.cpu().numpy() - g[k]).max() <= 1e-4 * max(1.0, np.abs(g[k]).max()), k
    for k, p in m.named_parameters():
        ref = g["grad." + k]
        assert np.abs(p.grad.cpu().numpy() - ref).max() <= 1e-4 * max(1.0, np.abs(ref).max()), k


def test_layer_bf16_tensor_core_path(cuda):
    """bf16-true as in the shipped configs (`configs/*.yaml:7`): D = 64 heads go through the
    tcgen05 kernel; output within 2e-2 of the fp32 reference layer."""
    import layers
    g = load_golden("e128_mha", "layer")
    B, H, Hkv, T, C, D = (int(x) for x in g["dims"])
    m = layers.MVPFormerGQAFlashAttention(_cfg(H, Hkv, D, T), layer_idx=0).eval().to(cuda)
    m.load_state_dict({k[3:]: torch.tensor(v) for k, v in g.items() if k.startswith("sd.")}, strict=True)
    m = m.to(torch.bfloat16)
    x, pos, chan = (torch.tensor(g[k], device=cuda, dtype=torch.bfloat16) for k in ("x", "pos", "chan"))
    with torch.no_grad():
        out, _ = m(x, pos, chan)
    assert out.dtype == torch.bfloat16 and out.is_contiguous()
    assert np.abs(out.float().cpu().numpy() - g["out"]).max() <= 2e-2 * max(1.0, np.abs(g["out"]).max())


def test_layer_bf16_backward_through_tensor_core_kernels(cuda):
    """Training path of the layer in bf16-true: the strided head views and the strided dO go through the
    tcgen05 backward; input and parameter gradients within 3e-2 * max|reference| (measured <= 1.1e-2) of the fp32 reference
    layer's (bf16 projections and bf16 gradient tensors set the error, not the attention kernels)."""
    import layers
    g = load_golden("e128_mha", "layer")
    B, H, Hkv, T, C, D = (int(x) for x in g["dims"])
    m = layers.MVPFormerGQAFlashAttention(_cfg(H, Hkv, D, T), layer_idx=0).eval().to(cuda)
    m.load_state_dict({k[3:]: torch.tensor(v) for k, v in g.items() if k.startswith("sd.")}, strict=True)
    m = m.to(torch.bfloat16)
    x, pos, chan = (torch.tensor(g[k], device=cuda, dtype=torch.bfloat16).requires_grad_(True)
                    for k in ("x", "pos", "chan"))
    out, _ = m(x, pos, chan)
    out.backward(torch.tensor(g["gout"], device=cuda, dtype=torch.bfloat16))
    worst = {}
    for t, k in ((x, "dx"), (pos, "dpos"), (chan, "dchan")):
        worst[k] = np.abs(t.grad.float().cpu().numpy() - g[k]).max() / max(1.0, np.abs(g[k]).max())
    for k, p in m.named_parameters():
        ref = g["grad." + k]
        worst[k] = np.abs(p.grad.float().cpu().numpy() - ref).max() / max(1.0, np.abs(ref).max())
    print("bf16 layer gradient errors / max|ref|:", {k: round(float(v), 4) for k, v in worst.items()})
    assert max(worst.values()) <= 3e-2, worst


def test_layer_training_mode_with_attention_dropout(cuda):
    """`model.train()` with `attn_pdrop > 0` (the shipped configs train that way): the layer passes
    `p_drop` to the operator as the reference Flash layer does (`layers/mvpa.py:391-397`); the step runs,
    gradients are finite, and the output differs from the eval-mode one."""
    import layers
    g = load_golden("e128_mha", "layer")
    B, H, Hkv, T, C, D = (int(x) for x in g["dims"])
    m = layers.MVPFormerGQAFlashAttention(_cfg(H, Hkv, D, T), layer_idx=0).to(cuda).to(torch.bfloat16)
    x, pos, chan = (torch.tensor(g[k], device=cuda, dtype=torch.bfloat16).requires_grad_(True)
                    for k in ("x", "pos", "chan"))
    m.eval()
    with torch.no_grad():
        ref, _ = m(x, pos, chan)
    m.train()
    torch.manual_seed(0)
    out, _ = m(x, pos, chan)
    out.float().square().mean().backward()
    assert torch.isfinite(out).all() and not torch.equal(out, ref)
    for t in (x, pos, chan, *m.parameters()):
        assert t.grad is not None and torch.isfinite(t.grad).all()
