"""CPU: host-side logic of the model-level package: state-dict layout against the fixture written from the
reference's `MVPFormerModel`, configuration aliases, encoder sizes, and the synthetic iEEG generator."""
import numpy as np
import torch

import models
from eeg_datasets import synthetic_ieeg
from test_model_oracle import load_model_golden


def _config(cfg, **kw):
    return models.MVPFormerConfig(n_positions=cfg["n_positions"], n_channels=cfg["n_channels"], n_embd=cfg["n_embd"],
                                  n_layer=cfg["n_layer"], n_head=cfg["n_head"], n_inner=cfg["n_inner"],
                                  n_head_kv=cfg["n_head_kv"], layer_norm_epsilon=cfg["eps"], **kw)


def test_state_dict_has_the_reference_keys_and_shapes():
    g, cfg, state = load_model_golden()
    m = models.MVPFormerModel(_config(cfg))
    own = {k: v for k, v in m.state_dict().items() if not k.endswith(("time_bias", "masked_bias"))}
    assert set(own) == set(state)
    for k, v in own.items():
        assert tuple(v.shape) == tuple(state[k].shape), k
    m.load_state_dict(state, strict=False)             # the two buffers are not in the fixture
    assert torch.equal(m.h[1].mlp.up_proj.weight, state["h.1.mlp.up_proj.weight"])


def test_config_aliases_and_task_layout():
    c = models.MVPFormerConfig(n_embd=768, n_layer=12, n_head=12, n_head_kv=4, n_inner=1728, n_positions=128)
    assert (c.hidden_size, c.num_attention_heads, c.num_hidden_layers, c.intermediate_size) == (768, 12, 12, 1728)
    assert c.max_position_embeddings == 128 and c.max_channel_embeddings == 128
    enc = models.WaveEncoder(2560, 768)
    assert enc.dwt_size == 2610 and enc.sizes == [1283, 645, 326, 166, 86, 46, 26, 16, 16]
    task = models.ClassificationHMVPFormer(models.MVPFormerConfig(n_embd=64, n_layer=1, n_head=4, n_head_kv=2, n_inner=96),
                                           models.WaveEncoder(256, 64), models.MVPFormerHead(64, 2))
    keys = set(task.state_dict())
    assert {"seizure_embeddings", "encoder.ln.weight", "encoder.proj.weight", "head.head.weight",
            "mvpformer.ln_f.weight", "mvpformer.h.0.attn.attn_bias", "mvpformer.h.0.mlp.down_proj.weight"} <= keys


def test_negative_indices_never_name_the_token_itself():
    task = models.HMVPFormer(models.MVPFormerConfig(n_embd=64, n_layer=1, n_head=4, n_head_kv=2, n_inner=96),
                             models.WaveEncoder(256, 64), models.MVPFormerHead(64), num_negatives=7)
    idx = task._negative_indices((3, 5, 4), torch.Generator().manual_seed(0))
    n = 3 * 5 * 4
    assert idx.shape == (3, 5, 4, 7) and idx.dtype == torch.int32
    assert int(idx.min()) >= 0 and int(idx.max()) < n
    own = torch.arange(n).view(3, 5, 4, 1)
    assert not (idx == own).any()


def test_synthetic_ieeg_is_seeded_pink_and_bursty():
    a = synthetic_ieeg(1, 16, 4, 512, seed=3)
    b = synthetic_ieeg(1, 16, 4, 512, seed=3)
    assert a.shape == (1, 16, 4, 512) and a.dtype == torch.float32 and torch.equal(a, b)
    assert not torch.equal(a, synthetic_ieeg(1, 16, 4, 512, seed=4))
    quiet = synthetic_ieeg(1, 16, 4, 512, seed=3, bursts=0)
    rec = quiet[0].permute(1, 0, 2).reshape(4, -1).double()                     # (channels, time)
    assert abs(float(rec.mean())) < 1e-3 and abs(float(rec.std()) - 1.0) < 1e-2  # z-scored per channel
    p = np.abs(np.fft.rfft(rec.numpy(), axis=-1)) ** 2
    f = np.fft.rfftfreq(rec.shape[-1], d=1 / 512.0)
    lo, hi = (f > 1) & (f < 4), (f > 64) & (f < 256)
    slope = np.log(p[:, hi].mean() / p[:, lo].mean()) / np.log(f[hi].mean() / f[lo].mean())
    assert -1.3 < slope < -0.7                                                   # power ~ 1/f
    assert float(a.abs().max()) > 4.0 > float(quiet.abs().max()) * 0.8           # bursts stand out of the background
