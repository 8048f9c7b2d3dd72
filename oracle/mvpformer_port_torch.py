"""CPU restatement, in plain PyTorch, of the parts of MVPFormer that surround the attention.

TEST INFRASTRUCTURE ONLY: the checker for the block / encoder / head kernels and the model-level
forward, and the timed CPU stand-in of the model-level benchmark.  Nothing on the product path imports it.

What it follows:
  rmsnorm               `torch.nn.RMSNorm` as `models/mvpformer.py:5-8` selects it on a host without a
                        capability-8 GPU: x * rsqrt(mean(x^2) + eps) * weight
  block                 `MVPFormerBlock.forward` (`models/mvpformer.py:116-152`): ln_1, attention and MLP on
                        the same normalised input, h = x + MLP + Attn; the attention layer's projections and
                        head split as in `layers/mvpa.py:341-409`, attention itself by `mvpa_port_torch`
  model                 `MVPFormerModel.forward` (`models/mvpformer.py:246-261, 282-286, 296-383`):
                        embeddings of arange(T) / arange(C), the block loop, ln_f
  wavedec_periodic      `ptwt.wavedec(x, db4, mode="periodic")` as `WaveEncoder.block` calls it
                        (`models/fftencoder.py:79-88`): per level, circular padding by (2L-3)//2 on both
                        sides (one more on the right for an odd length) and a stride-2 correlation with the
                        reversed decomposition filters; coefficients concatenated coarse to fine
  wave_encoder          `WaveEncoder.forward` (`models/fftencoder.py:90-97`)
  classification_logits `ClassificationHMVPFormer.test_step` (`models/mvpformer.py:951-953`)
  contrastive_logits    `HMVPFormer._contrastive_logits` (`models/mvpformer.py:574-594`) with the negatives'
                        row indices passed in (`_get_negative_samples`, `:631-660`, draws them at random)

Parity pin: the block / model / head functions are pinned to `tests/golden/model_tiny.npz`, written by
`tests/golden/make_model_golden.py` from the reference's own `MVPFormerModel`, `MVPFormerHead` and
`_contrastive_logits`.  The wavelet transform is NOT pinned: `ptwt` / `pywt` are not installed where the
goldens were made ("parity unpinned" for `wavedec_periodic` / `wave_encoder`; they are checked through
properties of the transform: orthonormal filters, energy preservation, published db4 values).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

import mvpa_port_torch as port


def rmsnorm(x, weight, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)


def attention_layer(x, pos, chan, p, cfg):
    """x (B,T,C,E) already normalised; p: the layer's parameters by their state-dict names."""
    B, T, C, E = x.shape
    H, Hkv = cfg["n_head"], cfg["n_head_kv"]
    D = E // H
    N = T * C
    q = F.linear(x, p["q_attn.weight"]).view(B, N, H, D).permute(0, 2, 1, 3)
    kv = F.linear(x, p["c_attn.weight"]).view(B, N, 2 * Hkv, D)
    k, v = kv[:, :, :Hkv].permute(0, 2, 1, 3), kv[:, :, Hkv:].permute(0, 2, 1, 3)
    rt = F.linear(pos, p["position_net.weight"]).view(T, Hkv, D).permute(1, 0, 2)
    rc = F.linear(chan, p["channel_net.weight"]).view(C, Hkv, D).permute(1, 0, 2)
    u, vt, z = (b.view(Hkv, D) for b in p["attn_bias"].split(Hkv * D))
    o = port.rel_attn(q, u, vt, z, k, rt, rc, v, D ** -0.5, 10)            # (B,H,N,D)
    return F.linear(o.permute(0, 2, 1, 3).reshape(B, T, C, E), p["c_proj.weight"])


def block(h, pos, chan, p, cfg):
    """p: parameters of one block (`ln_1.weight`, `attn.*`, `mlp.*`)."""
    x = rmsnorm(h, p["ln_1.weight"], cfg["eps"])
    attn = attention_layer(x, pos, chan, {k[5:]: v for k, v in p.items() if k.startswith("attn.")}, cfg)
    mlp = F.linear(F.silu(F.linear(x, p["mlp.gate_proj.weight"])) * F.linear(x, p["mlp.up_proj.weight"]),
                   p["mlp.down_proj.weight"])
    return h + mlp + attn


def model(inputs_embeds, state, cfg):
    """state: `MVPFormerModel.state_dict()`; returns last_hidden_state (B,T,C,E)."""
    B, T, C, E = inputs_embeds.shape
    pos = state["positional_embedding.weight"][:T].unsqueeze(0)
    chan = state["channel_embedding.weight"][:C].unsqueeze(0)
    h = inputs_embeds
    for i in range(cfg["n_layer"]):
        pre = f"h.{i}."
        h = block(h, pos, chan, {k[len(pre):]: v for k, v in state.items() if k.startswith(pre)}, cfg)
    return rmsnorm(h, state["ln_f.weight"], cfg["eps"])


def wavedec_periodic(x, dec_lo, dec_hi):
    """x (rows, len) -> (rows, total): [cA_L, cD_L, ..., cD_1]."""
    L = dec_lo.numel()
    filt = torch.stack([dec_lo.flip(0), dec_hi.flip(0)]).unsqueeze(1).to(x.dtype)      # (2,1,L)
    levels, n = 0, x.shape[-1] // (L - 1)
    while n > 1:
        levels, n = levels + 1, n >> 1
    lo = x.unsqueeze(1)
    details = []
    for _ in range(levels):
        pad = (2 * L - 3) // 2
        padded = F.pad(lo, [pad, pad + (lo.shape[-1] % 2)], mode="circular")
        res = F.conv1d(padded, filt, stride=2)
        lo, hi = res[:, :1], res[:, 1:]
        details.append(hi.squeeze(1))
    return torch.cat([lo.squeeze(1)] + details[::-1], dim=-1)


def wave_encoder(x, dec_lo, dec_hi, ln_weight, proj_weight, eps=1e-5):
    coef = wavedec_periodic(x.float(), dec_lo, dec_hi)
    return F.linear(rmsnorm(coef, ln_weight, eps).to(proj_weight.dtype), proj_weight)


def classification_logits(out, head_weight):
    return F.linear(out[:, -1].mean(dim=1), head_weight)


def contrastive_logits(pred, positive, negatives_idx, temp):
    """pred, positive (B,T,C,E); negatives_idx (B,T,C,K) rows of positive.view(-1,E)."""
    B, T, C, E = positive.shape
    K = negatives_idx.shape[-1]
    negative = positive.reshape(-1, E).index_select(0, negatives_idx.reshape(-1).long()).view(B, T, C, K, E)[:, 1:]
    pos = positive[:, 1:]
    p = pred[:, :-1]
    target = torch.cat([pos.unsqueeze(-2), negative], dim=-2)
    logits = torch.cosine_similarity(p.unsqueeze(-2), target, dim=-1).type_as(target)
    same = (negative - pos.unsqueeze(-2)).norm(dim=-1) < 1e-8 + 1e-5 * pos.norm(dim=-1)[..., None]
    logits[..., 1:][same] = float("-inf")
    return (logits / temp).flatten(0, -2)
