"""GPU: kernels around the attention (RMSNorm + residual, SwiGLU gate, wavelet encoder, readouts) and the
fused model-level forward, through ctypes -> C ABI.

Oracles: the reference's own `MVPFormerModel` / `MVPFormerHead` / `_contrastive_logits` outputs stored in
`tests/golden/model_tiny.npz` (fp32, 1e-4 relative), and the plain-PyTorch restatement
`oracle/mvpformer_port_torch.py` (pinned to that fixture on CPU) for shapes the tensor-core attention takes
(bf16; tolerance 3e-2 of the largest |reference| after several layers of bf16 rounding).  The wavelet front end
has no reference fixture (`ptwt` is not installed where fixtures are made): the kernel is compared with the
restatement of `ptwt.wavedec`'s procedure."""
import numpy as np
import pytest
import torch

import models
import mvpa_ops
import mvpformer_port_torch as mp
from eeg_datasets import synthetic_ieeg
from test_model_host import _config
from test_model_oracle import load_model_golden

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,width", [(torch.bfloat16, 2048), (torch.bfloat16, 768), (torch.float32, 32),
                                         (torch.float32, 2048), (torch.bfloat16, 4096)])
def test_rmsnorm_with_and_without_residual_add(cuda, dtype, width):
    g = torch.Generator().manual_seed(width)
    x, a = (torch.randn(37, width, generator=g).to(dtype).to(cuda) for _ in range(2))
    w = (1 + 0.1 * torch.randn(width, generator=g)).to(dtype).to(cuda)
    y = mvpa_ops.rmsnorm(x, w, 1e-5)
    ref = mp.rmsnorm(x.float(), w.float(), 1e-5)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (y.float() - ref).abs().max() <= tol
    h = x.clone()
    y2 = mvpa_ops.rmsnorm(h, w, 1e-5, add=a, sum_out=h)                  # residual stream updated in place
    s = (x + a)                                                          # eager sum in the element type
    assert torch.equal(h, s)
    assert (y2.float() - mp.rmsnorm(s.float(), w.float(), 1e-5)).abs().max() <= tol


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_silu_mul_on_column_blocks(cuda, dtype):
    g = torch.Generator().manual_seed(1)
    I = 1728
    big = torch.randn(50, 64 + 2 * I, generator=g).to(dtype).to(cuda)
    cat = torch.zeros(50, 128 + I, dtype=dtype, device=cuda)
    mvpa_ops.silu_mul(big[:, 64:64 + I], big[:, 64 + I:], cat[:, 128:])
    ref = torch.nn.functional.silu(big[:, 64:64 + I]) * big[:, 64 + I:]    # eager: silu rounded to dtype, then the product
    assert (cat[:, 128:].float() - ref.float()).abs().max() <= (2e-2 if dtype == torch.bfloat16 else 1e-5)
    assert cat[:, :128].abs().max() == 0                                   # the neighbouring block is untouched


@pytest.mark.parametrize("n,rows,in_dtype,out_dtype", [(2560, 9, torch.float32, torch.float32),
                                                       (2560, 5, torch.float32, torch.bfloat16),
                                                       (300, 4, torch.float32, torch.float32),
                                                       (1000, 3, torch.bfloat16, torch.bfloat16)])
def test_wave_encode_vs_restated_wavedec(cuda, n, rows, in_dtype, out_dtype):
    lo, hi = (torch.tensor(x) for x in mvpa_ops.db4_filters())
    x = synthetic_ieeg(1, rows, 1, n, seed=n)[0, :, 0].to(in_dtype)
    _, total = mvpa_ops.wave_sizes(n)
    w = (1 + 0.1 * torch.randn(total, generator=torch.Generator().manual_seed(2))).to(out_dtype)
    pad = (total + 31) // 32 * 32
    y = mvpa_ops.wave_encode(x.to(cuda), w.to(cuda), 1e-5, pad_to=pad)
    coef = mp.wavedec_periodic(x.double(), lo.double(), hi.double())
    ref = mp.rmsnorm(coef, w.double(), 1e-5)
    assert y.shape == (rows, pad) and y.dtype == out_dtype
    assert y[:, total:].abs().max() == 0 if pad > total else True
    tol = 1e-4 if out_dtype == torch.float32 else 3e-2
    assert (y[:, :total].double().cpu() - ref).abs().max() <= tol * max(1.0, float(ref.abs().max()))


def test_fused_model_forward_fp32_vs_reference_fixture(cuda):
    """The reference's `MVPFormerModel` output on the fixture's weights and input: fused inference path and
    the differentiable eager path, fp32 (attention on the CUDA-core kernels at this head dim)."""
    g, cfg, state = load_model_golden()
    m = models.MVPFormerModel(_config(cfg, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)).to(cuda).eval()
    m.load_state_dict({k: v.to(cuda) for k, v in state.items()}, strict=False)
    x = torch.tensor(g["x"], device=cuda)
    ref = g["out"]
    with torch.no_grad():
        fused = m(inputs_embeds=x).last_hidden_state
    assert np.abs(fused.cpu().numpy() - ref).max() <= 1e-4 * np.abs(ref).max()
    assert torch.equal(x, torch.tensor(g["x"], device=cuda))               # the caller's input is not modified
    eager = m(inputs_embeds=x.clone().requires_grad_(True)).last_hidden_state
    assert np.abs(eager.detach().cpu().numpy() - ref).max() <= 1e-4 * np.abs(ref).max()
    eager.sum().backward()                                                 # the eager path is differentiable


def test_readouts_vs_reference_fixture(cuda):
    g, cfg, state = load_model_golden()
    out = torch.tensor(g["out"], device=cuda)
    pooled = mvpa_ops.channel_mean(out)
    cls = torch.nn.functional.linear(pooled, torch.tensor(g["head_cls"], device=cuda))
    assert np.abs(cls.cpu().numpy() - g["cls_logits"]).max() <= 1e-5
    logits = mvpa_ops.contrastive_logits(torch.tensor(g["pred"], device=cuda), torch.tensor(g["x"], device=cuda),
                                         torch.tensor(g["neg_idx"], device=cuda).int(), float(g["temp"]))
    assert np.abs(logits.cpu().numpy() - g["con_logits"]).max() <= 1e-4


def test_contrastive_logits_mask_equal_negatives_bf16(cuda):
    B, T, C, E, K = 2, 4, 3, 256, 5
    gen = torch.Generator().manual_seed(3)
    pred, enc = (torch.randn(B, T, C, E, generator=gen).to(torch.bfloat16) for _ in range(2))
    n = B * T * C
    neg = torch.randint(0, n, (B, T, C, K), generator=gen, dtype=torch.int32)
    neg[0, 1, 0, 2] = (0 * T + 1) * C + 0                                  # a negative that is the positive itself
    ref = mp.contrastive_logits(pred.float(), enc.float(), neg, 0.1)
    got = mvpa_ops.contrastive_logits(pred.to(cuda), enc.to(cuda), neg.to(cuda), 0.1).cpu()
    assert torch.isinf(got[0 * (T - 1) * C + 0 * C + 0, 3]) and torch.isinf(ref[0, 3])
    fin = torch.isfinite(ref)
    assert torch.equal(fin, torch.isfinite(got))
    assert (got[fin] - ref[fin]).abs().max() <= 2e-2


@pytest.mark.parametrize("shape", [dict(E=256, H=4, Hkv=2, I=352, L=3, T=12, C=32, B=2),      # D 64, grouped heads
                                   dict(E=256, H=2, Hkv=1, I=512, L=2, T=6, C=100, B=1)])     # D 128, ragged channels
def test_fused_model_forward_bf16_vs_port(cuda, shape):
    E, H, Hkv, I, L, T, C, B = (shape[k] for k in ("E", "H", "Hkv", "I", "L", "T", "C", "B"))
    torch.manual_seed(5)
    cfg = models.MVPFormerConfig(n_positions=T, n_channels=C, n_embd=E, n_layer=L, n_head=H, n_inner=I, n_head_kv=Hkv)
    m = models.MVPFormerModel(cfg).eval()
    with torch.no_grad():                                                  # make the attention matter (see the fixture)
        for blk in m.h:
            for name in ("q_attn", "c_attn", "position_net", "channel_net"):
                getattr(blk.attn, name).weight.mul_(6.0)
            blk.attn.attn_bias.mul_(20.0)
        m.positional_embedding.weight.mul_(30.0)
        m.channel_embedding.weight.mul_(30.0)
    m = m.to(torch.bfloat16)
    x = torch.randn(B, T, C, E).to(torch.bfloat16)
    state = {k: v.float() for k, v in m.state_dict().items()}
    pcfg = dict(n_layer=L, n_head=H, n_head_kv=Hkv, eps=cfg.layer_norm_epsilon)
    ref = mp.model(x.float(), state, pcfg)
    with torch.no_grad():
        got = m.to(cuda)(inputs_embeds=x.to(cuda)).last_hidden_state.float().cpu()
    assert torch.isfinite(got).all()
    assert (got - ref).abs().max() <= 3e-2 * ref.abs().max(), float((got - ref).abs().max())


def test_cuda_graph_replay_equals_eager_launches(cuda):
    """The fused forward captured in a CUDA graph: same bits as the eager launches, for two different inputs
    (the second one replays the graph captured for the first), and the caller's tensors are left alone."""
    E, H, Hkv, I, L, T, C, B = 256, 4, 2, 352, 2, 12, 32, 2
    torch.manual_seed(8)
    cfg = models.MVPFormerConfig(n_positions=T, n_channels=C, n_embd=E, n_layer=L, n_head=H, n_inner=I, n_head_kv=Hkv)
    m = models.MVPFormerModel(cfg).to(torch.bfloat16).to(cuda).eval()
    xs = [torch.randn(B, T, C, E, device=cuda).to(torch.bfloat16) for _ in range(2)]
    with torch.no_grad():
        eager = [m(inputs_embeds=x).last_hidden_state.clone() for x in xs]
        m.enable_cuda_graph()
        for x, ref in zip(xs, eager):
            keep = x.clone()
            out = m(inputs_embeds=x).last_hidden_state
            assert torch.equal(out, ref)
            assert torch.equal(x, keep)
        assert len(m._graphs) == 1
        m.enable_cuda_graph(False)
        assert torch.equal(m(inputs_embeds=xs[0]).last_hidden_state, eager[0])


def test_tasks_end_to_end_on_synthetic_ieeg(cuda):
    """Encoder -> model -> heads on synthetic iEEG: classification logits and contrastive next-state logits of
    the task wrappers against the same pipeline assembled from the restatement."""
    E, H, Hkv, I, L, T, C, B, n = 128, 2, 1, 192, 2, 5, 32, 3, 512
    torch.manual_seed(6)
    cfg = models.MVPFormerConfig(n_positions=T, n_channels=C, n_embd=E, n_layer=L, n_head=H, n_inner=I, n_head_kv=Hkv)
    x = synthetic_ieeg(B, T, C, n, seed=3)
    lo, hi = (torch.tensor(v) for v in mvpa_ops.db4_filters())
    pcfg = dict(n_layer=L, n_head=H, n_head_kv=Hkv, eps=cfg.layer_norm_epsilon)
    for cls in (True, False):
        head = models.MVPFormerHead(E, 2 if cls else None)
        task = (models.ClassificationHMVPFormer if cls else models.HMVPFormer)(cfg, models.WaveEncoder(n, E), head,
                                                                                num_negatives=6)
        with torch.no_grad():
            task.encoder.proj.weight.mul_(30.0)                            # unit-scale embeddings from unit-scale coefficients
        task = task.to(torch.bfloat16).eval()
        st = {k: v.float() for k, v in task.state_dict().items()}
        enc = mp.wave_encoder(x.reshape(-1, n), lo, hi, st["encoder.ln.weight"], st["encoder.proj.weight"]).view(B, T, C, E)
        out = mp.model(enc, {k[10:]: v for k, v in st.items() if k.startswith("mvpformer.")}, pcfg)
        task = task.to(cuda)
        if cls:
            ref = mp.classification_logits(out, st["head.head.weight"])
            got = task.classify(x.to(cuda)).float().cpu()
            assert got.shape == (B, 2)
        else:
            neg = task._negative_indices((B, T, C), torch.Generator(device=cuda).manual_seed(1))
            ref = mp.contrastive_logits(torch.nn.functional.linear(out, st["head.head.weight"]), enc, neg.cpu(), task.temp)
            got = task.next_state_logits(x.to(cuda), negatives=neg).cpu()
            assert got.shape == (B * (T - 1) * C, 7)
        assert torch.isfinite(got).all()
        assert (got - ref).abs().max() <= 5e-2 * max(1.0, float(ref.abs().max())), float((got - ref).abs().max())
