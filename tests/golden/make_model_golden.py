"""Generate `model_tiny.npz` from the reference's own model classes.

Run once, in a container that has the reference checked out:

    python tests/golden/make_model_golden.py [/path/to/reference]

`models/mvpformer.py` cannot be imported as it stands on a CPU-only host: it asks the GPU for its
capability at import time and imports the training stack (Lightning, DeepSpeed, torchtune,
torchmetrics, the dataset and logger packages).  None of that is on the path this fixture pins, so the
script stubs those modules, answers the capability query with (7, 0) (which makes the reference choose
`torch.nn.RMSNorm` and its PyTorch attention layer, `models/mvpformer.py:5-8, 109-112`), and restores
`get_head_mask`, which the installed `transformers` no longer provides (the reference pins 4.43.3, where
`get_head_mask(None, n)` returns `[None] * n`).  Everything computed is the reference's code:
`MVPFormerModel.forward`, `MVPFormerHead`, the readout of `ClassificationHMVPFormer.test_step`
(`out[:, -1].mean(dim=1)`), and `HMVPFormer._contrastive_logits` + `_get_negative_samples` (the function
under its `torch.compile` decorator).  fp32, CPU.
"""
import os
import sys
import types

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MVPA_REFERENCE_DIR", "reference")
HERE = os.path.dirname(os.path.abspath(__file__))


class _Any:
    def __init__(self, *a, **k):
        pass

    def __call__(self, *a, **k):
        return self

    def __getattr__(self, n):
        return _Any()


def _stub(name, **attrs):
    m = types.ModuleType(name)
    m.__dict__.update(attrs)
    sys.modules[name] = m


_stub("loralib")
for n in ("deepspeed", "deepspeed.ops", "deepspeed.runtime", "deepspeed.runtime.activation_checkpointing", "loggers",
          "pytorch_lightning.utilities", "torchmetrics", "torchtune", "torchtune.modules"):
    _stub(n)
_stub("deepspeed.ops.adam", FusedAdam=_Any)
_stub("deepspeed.runtime.activation_checkpointing.checkpointing", checkpoint=lambda f, *a: f(*a))
_stub("eeg_datasets", EEGBatch=_Any)
_stub("loggers.patient_logger", PatientLogger=_Any, PredictiveLogger=_Any)
_stub("pytorch_lightning", LightningModule=torch.nn.Module)
_stub("pytorch_lightning.utilities.types", STEP_OUTPUT=object)
_stub("torchmetrics.classification", BinaryAccuracy=_Any, BinaryF1Score=_Any, BinaryStatScores=_Any)
_stub("torchtune.modules.peft", get_adapter_params=_Any, set_trainable_params=_Any)
torch.cuda.get_device_capability = lambda *a: (7, 0)
sys.path.insert(0, REF)
import models.mvpformer as M  # noqa: E402

M.MVPFormerModel.get_head_mask = lambda self, head_mask, n, *a, **k: [None] * n

CFG = dict(n_positions=12, n_channels=8, n_embd=32, n_layer=2, n_head=2, n_head_kv=1, n_inner=48)
B, T, C, K = 3, 7, 5, 4


def main():
    torch.manual_seed(11)
    cfg = M.MVPFormerConfig(resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0, **CFG)
    model = M.MVPFormerModel(cfg).eval()
    # the reference initialises every Linear / Embedding with std 0.02, which makes the attention nearly
    # uniform; widen the parameters the attention scores depend on so that a wrong index map shows
    with torch.no_grad():
        for blk in model.h:
            for name in ("q_attn", "c_attn", "position_net", "channel_net"):
                getattr(blk.attn, name).weight.mul_(12.0)
            blk.attn.attn_bias.mul_(20.0)
            blk.ln_1.weight.copy_(1 + 0.2 * torch.randn_like(blk.ln_1.weight))
        model.ln_f.weight.copy_(1 + 0.2 * torch.randn_like(model.ln_f.weight))
        model.positional_embedding.weight.mul_(30.0)
        model.channel_embedding.weight.mul_(30.0)
    E = CFG["n_embd"]
    x = torch.randn(B, T, C, E)
    head_cls = M.MVPFormerHead(E, 2)
    head_gen = M.MVPFormerHead(E)
    with torch.no_grad():
        out = model(input_ids=None, inputs_embeds=x).last_hidden_state
        cls = head_cls(out[:, -1].mean(dim=1))
        pred = head_gen(out)
        fake = types.SimpleNamespace(num_negatives=K, device=torch.device("cpu"))
        drawn = {}

        def negatives(positive):  # `_get_negative_samples` with its draws recorded
            bsz, seg_n, ch, _ = positive.shape
            torch.manual_seed(12)
            idx = torch.randint((bsz - 1) * (ch * seg_n), (bsz * seg_n * ch * K,), dtype=torch.int)
            torch.manual_seed(12)
            neg = M.HMVPFormer._get_negative_samples(fake, positive)
            cand = torch.arange(bsz * ch * seg_n).unsqueeze(-1).expand(-1, K).flatten()
            idx[idx >= cand] += 1
            drawn["idx"] = idx.view(bsz, seg_n, ch, K)
            return neg

        fake._get_negative_samples = negatives
        fn = M.HMVPFormer._contrastive_logits
        fn = getattr(fn, "_torchdynamo_orig_callable", fn)
        logits = fn(fake, pred, x, 0.1)
    state = {k: v.numpy() for k, v in model.state_dict().items() if not k.endswith(("time_bias", "masked_bias"))}
    np.savez_compressed(
        os.path.join(HERE, "model_tiny.npz"), x=x.numpy(), out=out.numpy(), cls_logits=cls.numpy(),
        head_cls=head_cls.head.weight.detach().numpy(), head_gen=head_gen.head.weight.detach().numpy(),
        pred=pred.numpy(), neg_idx=drawn["idx"].numpy(), con_logits=logits.numpy(), temp=np.float32(0.1),
        cfg=np.array([CFG[k] for k in ("n_positions", "n_channels", "n_embd", "n_layer", "n_head", "n_head_kv", "n_inner")]),
        eps=np.float32(cfg.layer_norm_epsilon), **{"state." + k: v for k, v in state.items()})
    print("wrote model_tiny.npz", out.shape, logits.shape, float(out.abs().mean()))


if __name__ == "__main__":
    main()
