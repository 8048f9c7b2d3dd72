"""MVPFormer around the MVPA layer: configuration, parallel block, model loop, head and the two task
wrappers, with the reference's class names, constructor arguments and state-dict keys
(`models/mvpformer.py:37-188, 405-485, 596-607, 951-953, 979-989`), without Lightning / DeepSpeed /
transformers.  Training-loop code (optimizer, loggers, metrics, checkpoint plumbing) is not here.

Inference runs a fused form of the parallel block (`models/mvpformer.py:132-147`,
h = x + MLP(ln_1 x) + Attn(ln_1 x)) built for B200:

  * one RMSNorm kernel that also adds the previous block's branch sum to the residual stream
    (`mvpa_rmsnorm` with `add`): one pass over the hidden state where eager PyTorch makes three;
  * ONE projection GEMM per block for q, k, v, gate and up (their weights concatenated once): the
    normalised input is read once; the attention kernels take q / k / v as strided views of its output;
  * the attention writes its output straight into the left column block of the buffer whose right block
    the SwiGLU kernel fills (`mvpa_silu_mul`), so `c_proj` and `down_proj` become ONE GEMM with the
    concatenated weight [c_proj | down_proj]: the two branch outputs are summed in the GEMM's fp32
    accumulator instead of two bf16 additions;
  * the relative keys of all layers (`position_net`, `channel_net` of the embeddings, which do not depend
    on the input) come from one GEMM each per forward.

With gradients enabled the blocks run the reference's op order through differentiable torch
expressions and the differentiable `attentions.flashmvpa`.
"""
from __future__ import annotations

from types import SimpleNamespace
from typing import Optional

import torch
import torch.nn.functional as F

import mvpa_ops
from attentions import flash_mvpa_into
from layers import MVPFormerGQAFlashAttention
from models import BrainDecider


class MVPFormerConfig:
    """Same constructor arguments and attribute aliases as the reference's `MVPFormerConfig(GPT2Config)`
    (`models/mvpformer.py:37-101`)."""

    attribute_map = {"hidden_size": "n_embd", "max_position_embeddings": "n_positions",
                     "max_channel_embeddings": "n_channels", "num_attention_heads": "n_head",
                     "num_hidden_layers": "n_layer", "intermediate_size": "n_inner",
                     "hidden_act": "activation_function"}

    def __init__(self, n_positions=100, n_channels=128, n_embd=768, n_layer=12, n_head=12, n_inner=2048,
                 n_head_kv=12, global_att=True, activation_function="silu", resid_pdrop=0.1, embd_pdrop=0.1,
                 attn_pdrop=0.1, layer_norm_epsilon=0.00001, initializer_range=0.02, scale_attn_weights=True,
                 use_cache=False, scale_attn_by_inverse_layer_idx=False, reorder_and_upcast_attn=False, lora=False,
                 lora_alpha=16, lora_rank=8, lora_dropout=0, lora_merge=True):
        if activation_function != "silu":
            raise NotImplementedError("MVPFormerConfig: the MLP kernels implement the shipped activation, silu")
        for k, v in list(locals().items()):
            if k != "self":
                setattr(self, k, v)
        self.pretraining_tp, self.mlp_bias = 1, False

    def __getattr__(self, name):
        alias = type(self).attribute_map.get(name)
        if alias is None:
            raise AttributeError(name)
        return getattr(self, alias)


class RMSNorm(torch.nn.Module):
    """x * rsqrt(mean(x^2) + eps) * weight in fp32 (`models/mvpformer.py:5-8` takes flash-attn's or torch's)."""

    def __init__(self, hidden_size, eps=1e-5):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.ones(hidden_size))
        self.eps = eps

    def forward(self, x):
        if torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad):
            xf = x.float()
            return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()).to(x.dtype)
        return mvpa_ops.rmsnorm(x.contiguous(), self.weight.detach().to(x.dtype), self.eps)


class LlamaMLP(torch.nn.Module):
    """SwiGLU MLP with the parameter names of `transformers`' `LlamaMLP`, which the reference block uses
    (`models/mvpformer.py:34, 114`): down_proj(silu(gate_proj(x)) * up_proj(x)), no biases."""

    def __init__(self, config):
        super().__init__()
        self.gate_proj = torch.nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.up_proj = torch.nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.down_proj = torch.nn.Linear(config.intermediate_size, config.hidden_size, bias=False)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class MVPFormerBlock(torch.nn.Module):
    def __init__(self, config, layer_idx=None):
        super().__init__()
        self.ln_1 = RMSNorm(config.hidden_size, eps=config.layer_norm_epsilon)
        self.attn = MVPFormerGQAFlashAttention(config, layer_idx=layer_idx)
        self.ln_2 = RMSNorm(config.hidden_size, eps=config.layer_norm_epsilon)   # unused, as in the reference
        self.mlp = LlamaMLP(config)
        self._fused = None

    def forward(self, hidden_states, positional_embedding, channel_embedding, layer_past=None, attention_mask=None,
                head_mask=None, encoder_hidden_states=None, encoder_attention_mask=None, use_cache=False,
                output_attentions=False):
        """The reference's op order (`models/mvpformer.py:132-152`); differentiable."""
        residual = hidden_states
        hidden_states = self.ln_1(hidden_states)
        attn_outputs = self.attn(hidden_states, positional_embedding, channel_embedding, layer_past=layer_past,
                                 attention_mask=attention_mask, head_mask=head_mask, use_cache=use_cache,
                                 output_attentions=output_attentions)
        outputs = attn_outputs[1:]
        hidden_states = residual + self.mlp(hidden_states) + attn_outputs[0]
        return (hidden_states,) + (outputs if use_cache else outputs[1:])

    # ---- fused inference path -------------------------------------------------------------------
    def fused_weights(self):
        """[q | k v | gate up] (rows) and [c_proj | down_proj] (columns), concatenated once per weight version."""
        ws = (self.attn.q_attn.weight, self.attn.c_attn.weight, self.mlp.gate_proj.weight, self.mlp.up_proj.weight,
              self.attn.c_proj.weight, self.mlp.down_proj.weight)
        tag = tuple((w._version, w.data_ptr(), w.dtype) for w in ws)
        if self._fused is None or self._fused[0] != tag:
            w_in = torch.cat([w.detach() for w in ws[:4]], dim=0).contiguous()
            w_out = torch.cat([ws[4].detach(), ws[5].detach()], dim=1).contiguous()
            self._fused = (tag, w_in, w_out)
        return self._fused[1], self._fused[2]

    @torch.no_grad()
    def fused_branches(self, x, r_time, r_chan, B, T, C):
        """x (B*T*C, E): the block's normalised input.  Returns MLP(x) + Attn(x), (B*T*C, E)."""
        a = self.attn
        E, H, Hkv, D = a.embed_dim, a.num_heads, a.num_kv_heads, a.head_dim
        I = self.mlp.gate_proj.out_features
        N, KV = T * C, Hkv * D
        w_in, w_out = self.fused_weights()
        big = F.linear(x, w_in)                                          # (M, E + 2 KV + 2 I)
        q4 = big[:, :E].view(B, N, H, D).permute(0, 2, 1, 3)
        k4 = big[:, E:E + KV].view(B, N, Hkv, D).permute(0, 2, 1, 3)
        v4 = big[:, E + KV:E + 2 * KV].view(B, N, Hkv, D).permute(0, 2, 1, 3)
        cat = torch.empty((x.shape[0], E + I), dtype=x.dtype, device=x.device)
        u, vt, z = (b.view(Hkv, D).to(x.dtype) for b in a.attn_bias.detach().split(KV))
        flash_mvpa_into(cat[:, :E].view(B, N, H, D).permute(0, 2, 1, 3), q4, u, vt, z, k4, r_time, r_chan, v4,
                        1.0 / (D ** 0.5), 10)
        g0 = E + 2 * KV
        mvpa_ops.silu_mul(big[:, g0:g0 + I], big[:, g0 + I:g0 + 2 * I], cat[:, E:])
        return F.linear(cat, w_out)

    @torch.no_grad()
    def fused_branches_time_sharded(self, x, r_time, r_chan, T, C, rows, group, transport):
        """The same for ONE sample whose time axis is spread over the ranks of `group` (`mvpa_shard`): x holds
        this rank's tokens, its two zig-zag chunks one after the other (`rows` = tokens per chunk).  Everything
        but the attention is local to a token; K and V of the other ranks' tokens are gathered per layer while
        the MLP's gate runs, and the rank's two query ranges write straight into the buffer the output
        projection reads."""
        import mvpa_shard
        a = self.attn
        E, H, Hkv, D = a.embed_dim, a.num_heads, a.num_kv_heads, a.head_dim
        I = self.mlp.gate_proj.out_features
        KV = Hkv * D
        w_in, w_out = self.fused_weights()
        big = F.linear(x, w_in)                                          # (rows of this rank, E + 2 KV + 2 I)
        cat = torch.empty((x.shape[0], E + I), dtype=x.dtype, device=x.device)
        u, vt, z = (b.view(Hkv, D).to(x.dtype) for b in a.attn_bias.detach().split(KV))
        bounds = [(0, rows[0]), (rows[0], rows[0] + rows[1])]
        part = lambda lo, hi, c0, heads: big[lo:hi, c0:c0 + heads * D].view(1, hi - lo, heads, D) if hi > lo else None
        q_loc = [part(lo, hi, 0, H) for lo, hi in bounds]
        kv_loc = [part(lo, hi, E, 2 * Hkv) for lo, hi in bounds]         # K and V side by side: fused along the head axis
        if transport == "nccl":
            kv_loc = [t.contiguous() if t is not None else None for t in kv_loc]
        outs = iter([cat[lo:hi, :E].view(1, hi - lo, H, D).permute(0, 2, 1, 3) for lo, hi in bounds if hi > lo])

        def op(q, u_, vt_, z_, k, rt, rc, v, causal, sm_scale, window_size, q_time_range):
            return flash_mvpa_into(next(outs), q, u_, vt_, z_, k, rt, rc, v, sm_scale, window_size, q_time_range)

        g0 = E + 2 * KV
        mvpa_shard.time_sharded_attention(
            op, q_loc, u, vt, z, kv_loc, r_time, r_chan, None, T, C, 1.0 / (D ** 0.5), 10, group=group,
            overlap=lambda: mvpa_ops.silu_mul(big[:, g0:g0 + I], big[:, g0 + I:g0 + 2 * I], cat[:, E:]),
            transport=transport)
        return F.linear(cat, w_out)


class MVPFormerModel(torch.nn.Module):
    def __init__(self, config, gradient_checkpointing=False):
        super().__init__()
        self.config = config
        self.embed_dim = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.num_kv_heads = config.n_head_kv
        self.head_dim = self.embed_dim // self.num_heads
        self.embed_kv_dim = self.head_dim * self.num_kv_heads
        self.drop = torch.nn.Dropout(config.embd_pdrop)
        self.h = torch.nn.ModuleList([MVPFormerBlock(config, layer_idx=i) for i in range(config.num_hidden_layers)])
        self.ln_f = RMSNorm(self.embed_dim, eps=config.layer_norm_epsilon)
        self.positional_embedding = torch.nn.Embedding(config.max_position_embeddings, self.embed_dim)
        self.channel_embedding = torch.nn.Embedding(config.max_channel_embeddings, self.embed_dim)
        self.gradient_checkpointing = gradient_checkpointing
        self._rel = None
        self._use_graph, self._graphs = False, {}
        std = config.initializer_range                                     # `_init_weights` (`:179-188`)
        for m in self.modules():
            if isinstance(m, (torch.nn.Linear, torch.nn.Embedding)):
                m.weight.data.normal_(mean=0.0, std=std)

    def _rel_weights(self):
        ws = [b.attn.position_net.weight for b in self.h] + [b.attn.channel_net.weight for b in self.h]
        tag = tuple((w._version, w.data_ptr(), w.dtype) for w in ws)
        if self._rel is None or self._rel[0] != tag:
            L = len(self.h)
            self._rel = (tag, torch.cat([w.detach() for w in ws[:L]], dim=0).contiguous(),
                         torch.cat([w.detach() for w in ws[L:]], dim=0).contiguous())
        return self._rel[1], self._rel[2]

    def forward(self, input_ids=None, past_key_values=None, attention_mask=None, token_type_ids=None,
                position_ids=None, channel_ids=None, head_mask=None, inputs_embeds=None, encoder_hidden_states=None,
                encoder_attention_mask=None, use_cache=None, output_attentions=None, output_hidden_states=None,
                return_dict=None):
        """`inputs_embeds` (B,T,C,E) -> namespace with `last_hidden_state` (B,T,C,E)
        (`models/mvpformer.py:190-402`; token ids, KV cache, masks and cross attention are not supported,
        as in every shipped configuration)."""
        if inputs_embeds is None or input_ids is not None:
            raise NotImplementedError("MVPFormerModel takes inputs_embeds only, as the reference does")
        if past_key_values is not None or attention_mask is not None or head_mask is not None or use_cache:
            raise NotImplementedError("KV cache, attention_mask and head_mask are not supported by the MVPA kernels")
        B, T, C, E = inputs_embeds.shape
        dev = inputs_embeds.device
        if position_ids is None:
            position_ids = torch.arange(T, dtype=torch.long, device=dev).unsqueeze(0)
        if channel_ids is None:
            channel_ids = torch.arange(C, dtype=torch.long, device=dev).unsqueeze(0)
        hidden = self.drop(inputs_embeds)
        if torch.is_grad_enabled() or self.training:
            position_embeds = self.positional_embedding(position_ids)      # (1,T,E)
            channel_embeds = self.channel_embedding(channel_ids)           # (1,C,E)
            for block in self.h:
                hidden = block(hidden, position_embeds, channel_embeds)[0]
            hidden = self.ln_f(hidden)
        elif self._use_graph:
            hidden = self._graphed_forward(hidden, position_ids, channel_ids)
        else:
            hidden = self._fused_forward(hidden, position_ids, channel_ids)
        return SimpleNamespace(last_hidden_state=hidden.view(B, T, C, E), past_key_values=None, hidden_states=None,
                               attentions=None, cross_attentions=None)

    @torch.no_grad()
    def forward_time_sharded(self, embeds_local, T: int, C: int, group=None, transport: str = "p2p", graph: bool = False):
        """Inference on ONE sample of T x C tokens whose time axis is spread over the ranks of `group`
        (one process per GPU; no counterpart in the reference).  `embeds_local` (n*C, E) holds the encoder
        outputs of this rank's tokens: the time steps of its two zig-zag chunks (`mvpa_shard.zigzag_chunks(T,
        C, world)[rank]`), first chunk first, token = t*C + c inside a chunk.  Returns the last hidden state
        of the same tokens, (n*C, E).  Norms, projections and the MLP are local to a token; per layer only
        K and V travel (`transport`: "p2p", this library's peer-load kernels, or "nccl").  `graph=True` (peer-load
        transport, frozen weights): the whole forward is captured in a CUDA graph on first use and replayed -
        its step counters live on the device, so every replay orders itself against the other ranks' replays;
        the result is the graph's own buffer, overwritten by the next call."""
        if graph and transport == "p2p":
            key = ("sharded", tuple(embeds_local.shape), embeds_local.dtype, embeds_local.device.index, T, C, id(group))
            entry = self._graphs.get(key)
            if entry is None:
                static_in = embeds_local.clone()
                cur = torch.cuda.current_stream(embeds_local.device)
                side = torch.cuda.Stream(device=embeds_local.device)
                side.wait_stream(cur)
                with torch.cuda.stream(side):              # warm-up: builds the send buffers and mappings (collective)
                    self.forward_time_sharded(static_in, T, C, group, transport)
                cur.wait_stream(side)
                import mvpa_shard as _ms
                _ms.PeerKV.forget_events()                 # events of earlier work cannot be waited for inside a capture
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    static_out = self.forward_time_sharded(static_in, T, C, group, transport)
                _ms.PeerKV.forget_events()                 # ... nor those of the capture outside it
                entry = (g, static_in, static_out)
                self._graphs[key] = entry
            g, static_in, static_out = entry
            static_in.copy_(embeds_local)
            g.replay()
            return static_out
        import mvpa_shard
        import torch.distributed as dist
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        plan = mvpa_shard.zigzag_chunks(T, C, world)
        rows = [n * C for _, n in plan[rank]]
        if embeds_local.shape[0] != sum(rows):
            raise ValueError(f"rank {rank} owns {sum(rows)} tokens of this sample, got {embeds_local.shape[0]}")
        dev = embeds_local.device
        position_embeds = self.positional_embedding(torch.arange(T, dtype=torch.long, device=dev))
        channel_embeds = self.channel_embedding(torch.arange(C, dtype=torch.long, device=dev))
        L, Hkv, D = len(self.h), self.num_kv_heads, self.head_dim
        w_pos, w_chan = self._rel_weights()
        r_time = F.linear(position_embeds.to(embeds_local.dtype), w_pos).view(T, L, Hkv, D).permute(1, 2, 0, 3).contiguous()
        r_chan = F.linear(channel_embeds.to(embeds_local.dtype), w_chan).view(C, L, Hkv, D).permute(1, 2, 0, 3).contiguous()
        h = embeds_local.contiguous().clone()                             # the residual stream is updated in place
        branches = None
        import attentions.attn as attn_mod
        check = attn_mod._CHECK_STATUS
        attn_mod._CHECK_STATUS = False      # reading a status word back after every launch would stall the overlap
        try:
            for i, block in enumerate(self.h):
                w = block.ln_1.weight.detach().to(h.dtype)
                x = mvpa_ops.rmsnorm(h, w, block.ln_1.eps, add=branches, sum_out=h if branches is not None else None)
                branches = block.fused_branches_time_sharded(x, r_time[i], r_chan[i], T, C, rows, group, transport)
        finally:
            attn_mod._CHECK_STATUS = check
        return mvpa_ops.rmsnorm(h, self.ln_f.weight.detach().to(h.dtype), self.ln_f.eps, add=branches, sum_out=h)

    def enable_cuda_graph(self, flag: bool = True):
        """Inference with frozen weights: capture the fused forward of each input shape in a CUDA graph on
        first use and replay it afterwards (one launch from the host instead of about ten per block, which
        matters when a rank's share of the batch is small).  The returned tensor is the graph's own output
        buffer: it is overwritten by the next call with the same shape.  Call again (or `reset_cuda_graphs`)
        after changing or moving the weights."""
        self._use_graph = bool(flag)
        self._graphs = {}
        return self

    def reset_cuda_graphs(self):
        self._graphs = {}

    @torch.no_grad()
    def _graphed_forward(self, hidden, position_ids, channel_ids):
        import attentions.attn as attn_mod
        key = (tuple(hidden.shape), hidden.dtype, hidden.device.index, tuple(position_ids.shape), tuple(channel_ids.shape))
        entry = self._graphs.get(key)
        if entry is None:
            static_in = hidden.clone()
            pos, chan = position_ids.clone(), channel_ids.clone()
            cur = torch.cuda.current_stream(hidden.device)
            side = torch.cuda.Stream(device=hidden.device)
            side.wait_stream(cur)
            check = attn_mod._CHECK_STATUS
            attn_mod._CHECK_STATUS = False                 # reading the status word back synchronises: not under capture
            try:
                with torch.cuda.stream(side):              # warm-up: lazy initialisations, allocator, fused weights
                    self._fused_forward(static_in, pos, chan)
                cur.wait_stream(side)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    static_out = self._fused_forward(static_in, pos, chan)
            finally:
                attn_mod._CHECK_STATUS = check
            # the graph reads these buffers on every replay: the index tensors stay alive with it
            entry = (graph, static_in, static_out, pos, chan)
            self._graphs[key] = entry
        graph, static_in, static_out = entry[:3]
        static_in.copy_(hidden)
        graph.replay()
        return static_out

    @torch.no_grad()
    def _fused_forward(self, hidden, position_ids, channel_ids):
        position_embeds = self.positional_embedding(position_ids)          # (1,T,E)
        channel_embeds = self.channel_embedding(channel_ids)               # (1,C,E)
        B, T, C, E = hidden.shape
        L, Hkv, D = len(self.h), self.num_kv_heads, self.head_dim
        w_pos, w_chan = self._rel_weights()
        # relative keys of every layer at once: (T, L, Hkv, D) -> per layer (Hkv, T, D)
        r_time = F.linear(position_embeds[0].to(hidden.dtype), w_pos).view(T, L, Hkv, D).permute(1, 2, 0, 3).contiguous()
        r_chan = F.linear(channel_embeds[0].to(hidden.dtype), w_chan).view(C, L, Hkv, D).permute(1, 2, 0, 3).contiguous()
        h = hidden.reshape(B * T * C, E).contiguous()
        if h.data_ptr() == hidden.data_ptr():
            h = h.clone()                                                  # the residual stream is updated in place
        branches = None
        for i, block in enumerate(self.h):
            w = block.ln_1.weight.detach().to(h.dtype)
            x = mvpa_ops.rmsnorm(h, w, block.ln_1.eps, add=branches, sum_out=h if branches is not None else None)
            branches = block.fused_branches(x, r_time[i], r_chan[i], B, T, C)
        return mvpa_ops.rmsnorm(h, self.ln_f.weight.detach().to(h.dtype), self.ln_f.eps, add=branches, sum_out=h)


class MVPFormerHead(BrainDecider):
    def __init__(self, size: int, size_out: Optional[int] = None):
        super().__init__()
        self.head = torch.nn.Linear(size, size_out if size_out is not None else size, bias=False)

    def forward(self, x):
        return self.head(x)


class HMVPFormer(torch.nn.Module):
    """The generative task's forward computations (`models/mvpformer.py:405-485, 574-607, 631-660`):
    encoder -> MVPFormerModel -> head -> contrastive next-state logits.  Attribute names (`mvpformer`,
    `encoder`, `head`, `seizure_embeddings`) are the reference's, so its checkpoints address the same keys."""

    def __init__(self, gpt_config, encoder, head, num_negatives=20, temp=0.1, **_unused_training_arguments):
        super().__init__()
        self.gpt_config = gpt_config
        self.mvpformer = MVPFormerModel(gpt_config)
        self.head = head
        self.encoder = encoder
        self.num_negatives = num_negatives
        self.temp = temp
        self.seizure_embeddings = torch.nn.Parameter(
            torch.normal(mean=0, std=1.0 / encoder.size_input, size=(3, encoder.size_input)))

    def _common_forward(self, batch):
        """batch (bsz, seg, ch, len) -> (last hidden state, encoder output), both (bsz, seg, ch, E)."""
        bsz, seg_n, ch, _ = batch.shape
        out_enc = self.encoder(batch.reshape(bsz * seg_n * ch, -1))
        input_embeds = out_enc.view(bsz, seg_n, ch, -1)
        out = self.mvpformer(input_ids=None, inputs_embeds=input_embeds).last_hidden_state
        return out, input_embeds

    def _negative_indices(self, shape, generator=None):
        """The draws of `_get_negative_samples` (`:631-660`): for every token, `num_negatives` rows of the
        flattened batch other than the token itself.  (B,T,C,K) int32."""
        bsz, seg_n, ch = shape
        dev = generator.device if generator is not None else self.head.head.weight.device
        n = bsz * seg_n * ch
        idx = torch.randint((bsz - 1) * (ch * seg_n), (n * self.num_negatives,), device=dev, dtype=torch.int,
                            generator=generator)
        cand = torch.arange(n, device=dev).unsqueeze(-1).expand(-1, self.num_negatives).flatten()
        idx[idx >= cand] += 1
        return idx.view(bsz, seg_n, ch, self.num_negatives)

    def _contrastive_logits(self, pred, positive, temp, negatives=None, generator=None):
        if negatives is None:
            negatives = self._negative_indices(positive.shape[:3], generator)
        return mvpa_ops.contrastive_logits(pred.contiguous(), positive.contiguous(), negatives.contiguous(), temp)

    @torch.no_grad()
    def next_state_logits(self, x, negatives=None, generator=None):
        """Forward of `training_step` up to the logits (`:677-690`): (B*(T-1)*C, 1 + num_negatives) fp32."""
        out, out_enc = self._common_forward(x)
        return self._contrastive_logits(self.head(out), out_enc, self.temp, negatives, generator)


class ClassificationHMVPFormer(HMVPFormer):
    @torch.no_grad()
    def classify(self, x):
        """Forward of `test_step` (`models/mvpformer.py:947-953`): logits (B, size_out)."""
        out, _ = self._common_forward(x)
        return self.head(mvpa_ops.channel_mean(out.contiguous()))
