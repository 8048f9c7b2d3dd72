"""Generate the golden fixtures in this directory from the reference itself.

Run once, in a container that has the reference checked out:

    python tests/golden/make_golden.py [/path/to/reference]

It imports the reference's own PyTorch attention layer
(`layers/mvpa.py`, class `MVPFormerGQAAttention`) with a stub for the unused
`loralib` import, runs `_rel_attn` / `forward` on seeded inputs in fp32 on the
CPU, and stores inputs, outputs and autograd gradients as `.npz`.  The tests
only read the `.npz` files; they never import the reference.
"""
import os
import sys
import types
from types import SimpleNamespace as NS

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MVPA_REFERENCE_DIR", "reference")
HERE = os.path.dirname(os.path.abspath(__file__))
sys.modules.setdefault("loralib", types.ModuleType("loralib"))
sys.path.insert(0, REF)
from layers.mvpa import MVPFormerGQAAttention  # noqa: E402


def make_layer(H, Hkv, D, t_max):
    cfg = NS(max_position_embeddings=t_max, hidden_size=H * D, num_attention_heads=H,
             n_head_kv=Hkv, n_inner=4 * H * D, global_att=True, scale_attn_weights=True,
             scale_attn_by_inverse_layer_idx=False, reorder_and_upcast_attn=False,
             lora=False, attn_pdrop=0.1, resid_pdrop=0.1)
    return MVPFormerGQAAttention(cfg, layer_idx=0).eval()


def op_case(name, seed, B, H, Hkv, T, C, D, stress, grads):
    """One operator-level case.  Draw order: module, q, k, v, pos_emb, chan_emb[, dO];
    the stress variant then overwrites the relative keys and u/v/z with N(0,1)."""
    torch.manual_seed(seed)
    m = make_layer(H, Hkv, D, max(T, 1))
    E = H * D
    q = torch.randn(B, H, T, C, D)
    k = torch.randn(B, Hkv, T, C, D)
    v = torch.randn(B, Hkv, T, C, D)
    pos = torch.randn(1, T, E)
    chan = torch.randn(1, C, E)
    do = torch.randn(B, H, T, C, D)
    with torch.no_grad():
        tk = m._split_heads(m.position_net(pos).unsqueeze(2), Hkv, D)   # (1,Hkv,T,1,D)
        ck = m._split_heads(m.channel_net(chan).unsqueeze(1), Hkv, D)   # (1,Hkv,1,C,D)
        if stress:
            tk = torch.randn_like(tk)
            ck = torch.randn_like(ck)
            m.attn_bias.data = torch.randn_like(m.attn_bias)
    leaves = [q, k, v, tk, ck]
    for t in leaves:
        t.requires_grad_(grads)
    m.attn_bias.requires_grad_(grads)
    out, _ = m._rel_attn(q, k, tk, ck, v)
    N = T * C
    u, vb, z = m.attn_bias.detach().split(Hkv * D)
    rec = dict(
        q=q.detach().reshape(B, H, N, D), k=k.detach().reshape(B, Hkv, N, D),
        val=v.detach().reshape(B, Hkv, N, D),
        u=u.reshape(Hkv, D), v=vb.reshape(Hkv, D), z=z.reshape(Hkv, D),
        r_time=tk.detach().reshape(Hkv, T, D), r_chan=ck.detach().reshape(Hkv, C, D),
        o=out.detach().reshape(B, H, N, D),
        dims=np.array([B, H, Hkv, T, C, D]), sm_scale=np.float64(1.0 / D ** 0.5),
    )
    if grads:
        out.backward(do)
        du, dv, dz = m.attn_bias.grad.split(Hkv * D)
        rec.update(
            do=do.reshape(B, H, N, D), dq=q.grad.reshape(B, H, N, D),
            dk=k.grad.reshape(B, Hkv, N, D), dval=v.grad.reshape(B, Hkv, N, D),
            du=du.reshape(Hkv, D), dv=dv.reshape(Hkv, D), dz=dz.reshape(Hkv, D),
            dr_time=tk.grad.reshape(Hkv, T, D), dr_chan=ck.grad.reshape(Hkv, C, D),
        )
    rec = {k_: (v_.numpy() if torch.is_tensor(v_) else v_) for k_, v_ in rec.items()}
    np.savez_compressed(os.path.join(HERE, f"op_{name}.npz"), **rec)
    print(name, "ok", {k_: getattr(v_, "shape", None) for k_, v_ in rec.items() if k_ == "o"})


def layer_case(name, seed, B, H, Hkv, T, C, D):
    """Module-level case: full `forward` with its state_dict, for the layer shim."""
    torch.manual_seed(seed)
    m = make_layer(H, Hkv, D, T)
    with torch.no_grad():
        m.attn_bias.data = 0.5 * torch.randn_like(m.attn_bias)
    E = H * D
    x = torch.randn(B, T, C, E, requires_grad=True)
    pos = torch.randn(1, T, E, requires_grad=True)
    chan = torch.randn(1, C, E, requires_grad=True)
    out, present = m(x, pos, chan, use_cache=True)
    gout = torch.randn_like(out)
    out.backward(gout)
    rec = {f"sd.{k_}": v_.detach().numpy() for k_, v_ in m.state_dict().items()}
    rec.update({f"grad.{k_}": p.grad.numpy() for k_, p in m.named_parameters()})
    rec.update(x=x.detach().numpy(), pos=pos.detach().numpy(), chan=chan.detach().numpy(),
               out=out.detach().numpy(), gout=gout.numpy(), dx=x.grad.numpy(),
               dpos=pos.grad.numpy(), dchan=chan.grad.numpy(),
               present_k=present[0].detach().numpy(), present_v=present[1].detach().numpy(),
               dims=np.array([B, H, Hkv, T, C, D]))
    np.savez_compressed(os.path.join(HERE, f"layer_{name}.npz"), **rec)
    print("layer", name, "ok", out.shape)


if __name__ == "__main__":
    # name, seed, B, H, Hkv, T, C, D, stress, grads
    op_case("cfg1", 0, 1, 4, 4, 32, 16, 64, False, False)       # BASELINE config 1 (fp32, CPU)
    op_case("gqa2_t24_c5", 11, 2, 4, 2, 24, 5, 16, True, True)  # GQA, last-row exception
    op_case("gqa3_t13_c3", 12, 1, 3, 1, 13, 3, 16, True, True)  # g=3, just past window edge
    op_case("t1_c7", 13, 1, 2, 2, 1, 7, 16, True, True)         # single time step
    op_case("t12_c1", 14, 1, 2, 2, 12, 1, 16, True, True)       # single channel
    op_case("t11_c4", 15, 1, 2, 1, 11, 4, 32, True, True)       # T == W+1
    op_case("t16_c16_d64", 16, 1, 2, 2, 16, 16, 64, True, True) # power-of-two tile shapes
    op_case("t6_c22_d64", 17, 1, 2, 1, 6, 22, 64, True, True)   # ragged channel count
    op_case("t2_c128_d128", 18, 1, 1, 1, 2, 128, 128, True, True)
    op_case("t14_c32_init", 19, 1, 2, 2, 14, 32, 64, False, True)  # model-init magnitudes
    layer_case("e64", 21, 2, 4, 2, 6, 5, 16)
    layer_case("e128_mha", 22, 1, 2, 2, 13, 4, 64)
