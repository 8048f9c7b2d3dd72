"""GPU: size-independent properties at BASELINE's full kernel configurations, where the CPU
oracle would take minutes: row-stochasticity, linearity in V, causality, batch/head
independence, and agreement of the tensor-core path with the fp32 CUDA-core path on one slice."""
import numpy as np
import pytest
import torch

import mvpa_oracle as mo

pytestmark = pytest.mark.gpu


def make(dev, seed, B, H, Hkv, T, C, D, dtype=torch.bfloat16):
    g = torch.Generator(device="cpu").manual_seed(seed)
    N = T * C
    r = lambda *s: torch.randn(*s, generator=g).to(dtype).to(dev)
    return dict(q=r(B, H, N, D), u=r(1, Hkv, 1, D), v=r(1, Hkv, 1, D), z=r(1, Hkv, 1, D),
                k=r(B, Hkv, N, D), rt=r(1, Hkv, T, D), rc=r(1, Hkv, C, D), val=r(B, Hkv, N, D))


def run(t, **over):
    import attentions
    a = dict(t, **over)
    D = a["q"].shape[-1]
    return attentions.flashmvpa(a["q"], a["u"], a["v"], a["z"], a["k"], a["rt"], a["rc"], a["val"],
                                causal=True, sm_scale=D ** -0.5, window_size=10)


CFG2 = (4, 16, 16, 64, 64, 64)     # BASELINE config 2 (MHA)
CFG2_GQA = (4, 16, 8, 64, 64, 64)
CFG3 = (8, 16, 16, 128, 32, 64)    # BASELINE config 3
LONG = (1, 4, 2, 128, 128, 128)    # 16k tokens, D=128 (per-sample slice of config 5)


@pytest.mark.parametrize("cfg", [CFG2, CFG2_GQA, CFG3, LONG])
def test_rows_sum_to_one_and_linearity(cuda, cfg):
    t = make(cuda, 1, *cfg)
    ones = torch.ones_like(t["val"])
    o1 = run(t, val=ones).float()
    assert (o1 - 1).abs().max() <= 1e-2            # softmax rows sum to one
    a = run(t).float()
    b = run(t, val=(2 * t["val"])).float()
    assert (b - 2 * a).abs().max() <= 2e-2         # exact scaling of V by 2 commutes with rounding
    assert torch.isfinite(a).all()


@pytest.mark.parametrize("cfg", [CFG2, LONG])
def test_causality_and_batch_independence(cuda, cfg):
    B, H, Hkv, T, C, D = cfg
    t = make(cuda, 2, *cfg)
    a = run(t)
    t_cut = T // 2
    k2, v2 = t["k"].clone(), t["val"].clone()
    k2[:, :, t_cut * C:] += 1.0                     # change every key/value of the later half
    v2[:, :, t_cut * C:] *= -1.0
    b = run(t, k=k2, val=v2)
    assert torch.equal(a[:, :, : t_cut * C], b[:, :, : t_cut * C])
    assert not torch.equal(a[:, :, t_cut * C:], b[:, :, t_cut * C:])
    if B > 1:                                       # batch elements do not interact
        perm = torch.arange(B - 1, -1, -1, device=cuda)
        c = run(t, q=t["q"][perm].contiguous(), k=t["k"][perm].contiguous(),
                val=t["val"][perm].contiguous())
        assert torch.equal(c[perm], a)


@pytest.mark.parametrize("cfg", [CFG2, CFG3, LONG])
def test_tensor_core_path_vs_fp32_path_on_a_slice(cuda, cfg):
    """One (batch, kv-group) slice: bf16 tensor-core result vs the fp32 CUDA-core kernels fed the
    same bf16-rounded values (the fp32 path itself is pinned to the oracle in test_gpu_op)."""
    B, H, Hkv, T, C, D = cfg
    g = H // Hkv
    t = make(cuda, 3, *cfg)
    a = run(t)[:1, :g].float()
    sl = dict(q=t["q"][:1, :g], k=t["k"][:1, :1], val=t["val"][:1, :1], u=t["u"][:, :1],
              v=t["v"][:, :1], z=t["z"][:, :1], rt=t["rt"][:, :1], rc=t["rc"][:, :1])
    b = run({k: x.float().contiguous() for k, x in sl.items()})
    assert (a - b).abs().max() <= 2e-2


def test_oracle_on_rows_of_config2(cuda):
    """A few query rows of config 2 against the numpy oracle (row-chunked, one head)."""
    B, H, Hkv, T, C, D = CFG2
    t = make(cuda, 4, *CFG2)
    o = run(t)[0, 0].float().cpu().numpy()
    f = lambda x: x.float().cpu().numpy()
    ref, _ = mo.mvpa_forward(f(t["q"][:1, :1]), f(t["u"][0, :1, 0]), f(t["v"][0, :1, 0]), f(t["z"][0, :1, 0]),
                             f(t["k"][:1, :1]), f(t["rt"][0, :1]), f(t["rc"][0, :1]), f(t["val"][:1, :1]),
                             D ** -0.5, row_chunk=512)
    assert np.abs(o - ref[0, 0]).max() <= 2e-2


def _oracle_inputs(t, b, hk, g):
    """One batch element x one kv group of a case, as float32 numpy arrays in the oracle's argument order."""
    f = lambda x: x.float().cpu().numpy()
    hs = slice(hk * g, (hk + 1) * g)
    return (f(t["q"][b:b + 1, hs]), f(t["u"][0, hk:hk + 1, 0]), f(t["v"][0, hk:hk + 1, 0]), f(t["z"][0, hk:hk + 1, 0]),
            f(t["k"][b:b + 1, hk:hk + 1]), f(t["rt"][0, hk:hk + 1]), f(t["rc"][0, hk:hk + 1]),
            f(t["val"][b:b + 1, hk:hk + 1]))


def _group_slice(t, b, hk, g):
    hs = slice(hk * g, (hk + 1) * g)
    return dict(q=t["q"][b:b + 1, hs].contiguous(), k=t["k"][b:b + 1, hk:hk + 1].contiguous(),
                val=t["val"][b:b + 1, hk:hk + 1].contiguous(), u=t["u"][:, hk:hk + 1].contiguous(),
                v=t["v"][:, hk:hk + 1].contiguous(), z=t["z"][:, hk:hk + 1].contiguous(),
                rt=t["rt"][:, hk:hk + 1].contiguous(), rc=t["rc"][:, hk:hk + 1].contiguous())


ORACLE_BWD_CASES = [
    ("config 3", CFG3, 2),                       # BASELINE config 3: T 128, C 32, D 64 (MHA), seed 2
    ("config 2, grouped heads", CFG2_GQA, 1),    # BASELINE config 2 with two query heads per kv head
    ("T 128, C 32, D 128", (1, 4, 2, 128, 32, 128), 8),   # the long model's head dim at an oracle-sized N
]


@pytest.mark.parametrize("name,cfg,seed", ORACLE_BWD_CASES)
def test_tensor_core_forward_and_backward_vs_oracle_at_baseline_sizes(cuda, name, cfg, seed):
    """One batch element x one kv group at BASELINE's own shapes, tensor-core kernels against the numpy
    oracle itself (not against this library's fp32 kernels): forward and all eight gradients.  This is
    BASELINE config 3's wording: "dQ/dK/dV checked against autograd through the reference PyTorch MVPA"
    (`layers/mvpa.py:173-278`, which the oracle restates and is pinned to).  bf16 tolerance: 2e-2 absolute
    on o, 2e-2 of max(1, max|reference|) on each gradient."""
    B, H, Hkv, T, C, D = cfg
    g = H // Hkv
    t = make(cuda, seed, *cfg)
    b, hk = B - 1, Hkv - 1                       # the last batch element and kv group: largest offsets
    sl = _group_slice(t, b, hk, g)
    gout = torch.randn(sl["q"].shape, generator=torch.Generator().manual_seed(seed + 50)).to(torch.bfloat16).to(cuda)
    leaves = {n: x.detach().clone().requires_grad_(True) for n, x in sl.items()}
    o = run(leaves)
    o.backward(gout)
    args = _oracle_inputs(t, b, hk, g)
    ref_o, _ = mo.mvpa_forward(*args, D ** -0.5)
    assert np.abs(o.detach().float().cpu().numpy() - ref_o).max() <= 2e-2
    ref = mo.mvpa_backward(*args, gout.float().cpu().numpy(), D ** -0.5)
    for leaf, key in (("q", "dq"), ("u", "du"), ("v", "dv"), ("z", "dz"), ("k", "dk"), ("rt", "dr_time"),
                      ("rc", "dr_chan"), ("val", "dval")):
        r = ref[key]
        got = leaves[leaf].grad.float().cpu().numpy().reshape(r.shape)
        err = np.abs(got - r).max()
        assert err <= 2e-2 * max(1.0, np.abs(r).max()), (name, key, float(err), float(np.abs(r).max()))
    # the same rows inside the full-size call: bit-identical forward (batch elements and kv groups are independent)
    full = run(t)
    assert torch.equal(full[b:b + 1, hk * g:(hk + 1) * g], o.detach())


def test_16k_tokens_head_dim_128_forward_vs_oracle(cuda):
    """The 16k-token point (T 128, C 128, D 128, two query heads per kv head): one query head of one kv
    group against the numpy oracle, row-chunked, in float32 (a float64 pass takes half a minute)."""
    B, H, Hkv, T, C, D = LONG
    g = H // Hkv
    t = make(cuda, 9, *LONG)
    o = run(t)
    hk = Hkv - 1
    args = list(_oracle_inputs(t, 0, hk, g))
    args[0] = args[0][:, 1:2]                    # the group's second query head
    ref, lse = mo.mvpa_forward(*args, D ** -0.5, row_chunk=512, dtype=np.float32)
    got = o[0, hk * g + 1].float().cpu().numpy()
    assert np.abs(got - ref[0, 0]).max() <= 2e-2


BWD_CASES = [(1, 16, 16, 128, 32, 64),   # config 3's shape, one batch element: several CTAs per SM in a row
             (1, 4, 2, 128, 128, 128),   # 16k tokens, grouped heads, head_dim 128
             (2, 4, 4, 64, 64, 64),      # config 2's shape, two batch elements
             # ragged channel / segment counts with many tiles outside the window, one per kernel variant:
             (2, 4, 2, 50, 22, 64),      # 32 channel slots, head_dim 64, grouped heads
             (1, 4, 4, 40, 100, 64),     # 128 channel slots at head_dim 64
             (1, 2, 1, 30, 60, 128),     # 64 channel slots at head_dim 128
             (1, 2, 2, 128, 7, 128)]     # 32 channel slots at head_dim 128


@pytest.mark.parametrize("cfg", BWD_CASES)
def test_backward_tensor_core_vs_fp32_path_full_size(cuda, cfg):
    """Backward at the benchmark shapes (many key tiles outside the content window, more CTAs than SMs):
    all eight gradients of the bf16 tensor-core kernels against the fp32 CUDA-core kernels fed the same
    bf16-rounded values; the latter are pinned to the oracle at small sizes in test_gpu_op.
    Tolerance: 3e-2 of the largest magnitude of each gradient (bf16 operands, fp32 accumulation)."""
    t = make(cuda, 5, *cfg)
    gout = torch.randn(t["q"].shape, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16).to(cuda)
    grads = []
    for dtype in (torch.bfloat16, torch.float32):
        leaves = {n: x.to(dtype).detach().clone().requires_grad_(True) for n, x in t.items()}
        run(leaves).backward(gout.to(dtype))
        grads.append({n: x.grad.float() for n, x in leaves.items()})
    torch.cuda.synchronize()
    for n in grads[0]:
        a, b = grads[0][n], grads[1][n]
        assert torch.isfinite(a).all(), n
        assert (a - b).abs().max() <= 3e-2 * b.abs().max() + 1e-6, (n, float((a - b).abs().max()), float(b.abs().max()))


@pytest.mark.parametrize("cfg", [(1, 16, 16, 128, 32, 64), (2, 4, 2, 64, 128, 128), (1, 4, 2, 40, 100, 64)])
def test_backward_is_bit_identical_from_run_to_run(cuda, cfg):
    """All eight gradients of the bf16 tensor-core backward, twice on the same inputs with thousands of CTAs
    adding into the per-kv-head accumulators in whatever order they finish: identical bits.  (The partial
    sums are added in 64-bit fixed point, and integer addition is associative.)"""
    t = make(cuda, 11, *cfg)
    gout = torch.randn(t["q"].shape, generator=torch.Generator().manual_seed(12)).to(torch.bfloat16).to(cuda)
    runs = []
    for _ in range(2):
        leaves = {n: x.detach().clone().requires_grad_(True) for n, x in t.items()}
        run(leaves).backward(gout)
        torch.cuda.synchronize()
        runs.append({n: x.grad.clone() for n, x in leaves.items()})
        # different work on the GPU in between, so that the two backward passes do not meet the same timing
        torch.randn(1 << 22, device=cuda).sort()
    for n in runs[0]:
        assert torch.equal(runs[0][n], runs[1][n]), n


@pytest.mark.parametrize("gain", [4.0, 40.0])
def test_forward_with_score_jumps_between_key_tiles(cuda, gain):
    """The temporal keys of the most recent lags are scaled up, so the row maximum jumps from one key
    tile to the next (tiles are visited oldest first), by about ten or by more than sixty binary orders
    of magnitude: the running reference of the online softmax has to follow.  (The temporal products
    use the raw bf16 q, so both paths see identical scores up to fp32 summation order.)  bf16
    tensor-core result vs the fp32 CUDA-core kernels on the same values; 2e-2 of the largest |o|."""
    B, H, Hkv, T, C, D = 1, 2, 2, 16, 64, 64
    t = make(cuda, 7, B, H, Hkv, T, C, D)
    rt = t["rt"].clone()
    rt[:, :, T - 4:] *= gain                # slots T-1-dt of the lags dt = 0 .. 3
    t = dict(t, rt=rt)
    a = run(t).float()
    b = run({n: x.float().contiguous() for n, x in t.items()})
    assert torch.isfinite(a).all()
    assert (a - b).abs().max() <= 2e-2 * b.abs().max(), float((a - b).abs().max())


def test_config5_full_batch_last_element_equals_single_sample_run(cuda):
    """The largest configuration BASELINE names (config 5: B 32 x 16 heads / 8 kv heads x 16384 tokens,
    D 128, bf16; q alone is 2.1 GB, byte offsets pass 2^31): forward and backward of the whole batch,
    then the last and a middle batch element again as single-sample calls on the same data — O, dq, dk,
    dv must be bit-identical (batch elements do not interact; any 32-bit offset overflow would show).
    At this size the kernels take their CTAs kv-head-major instead of tile-major, so this also checks that
    order, including the per-CTA partial sums behind the bias gradients."""
    import attentions
    B, H, Hkv, T, C, D = 32, 16, 8, 128, 128, 128
    N = T * C
    g = torch.Generator(device=cuda).manual_seed(5)
    r = lambda *s: torch.randn(*s, generator=g, device=cuda, dtype=torch.bfloat16)
    q, k, v, do = r(B, H, N, D), r(B, Hkv, N, D), r(B, Hkv, N, D), r(B, H, N, D)
    small = [r(1, Hkv, 1, D) for _ in range(3)] + [r(1, Hkv, T, D), r(1, Hkv, C, D)]
    kw = dict(causal=True, sm_scale=D ** -0.5, window_size=10)

    def step(qq, kk, vv, dd):
        qq, kk, vv = (x.detach().requires_grad_(True) for x in (qq, kk, vv))
        sm = [x.detach().requires_grad_(True) for x in small]
        o = attentions.flashmvpa(qq, sm[0], sm[1], sm[2], kk, sm[3], sm[4], vv, **kw)
        o.backward(dd)
        return (o.detach(), qq.grad, kk.grad, vv.grad), [x.grad.float() for x in sm]

    full, full_small = step(q, k, v, do)
    assert all(torch.isfinite(x).all() for x in full)
    acc = [torch.zeros_like(x) for x in full_small]
    for b in range(B):
        one, one_small = step(q[b:b + 1], k[b:b + 1], v[b:b + 1], do[b:b + 1])
        for a, x in zip(acc, one_small):
            a += x
        if b in (B - 1, B // 2):
            for name, a, c in zip(("o", "dq", "dk", "dv"), full, one):
                assert torch.equal(a[b:b + 1], c), (b, name)
    # bias and relative-key gradients are sums over the batch: whole-batch call vs the sum of the
    # single-sample calls (each rounded to bf16 once, hence the tolerance)
    for name, a, c in zip(("du", "dv_bias", "dz", "dr_time", "dr_chan"), full_small, acc):
        assert (a - c).abs().max() <= 2e-2 * max(1.0, c.abs().max().item()), name
