"""MVPA attention layer with the reference's module API (`layers/mvpa.py`).

Constructor arguments, config fields read, parameter / buffer names and shapes,
`forward` signature and return tuple are those of the reference, so
`MVPFormerBlock` (`models/mvpformer.py:104-152`) and reference checkpoints work
unchanged.  The attention itself always runs through the sm_100a library
(`attentions.flashmvpa`); there is no materialised-N x N PyTorch path here.

Unlike the reference Flash layer (`layers/mvpa.py:360-399`), heads are not split
by permute + `.contiguous()` copies: the projection outputs are handed to the
kernels as strided (B, H, N, D) views and the attention output is written
straight into the (B, T, C, H*D) layout `c_proj` reads.
"""
from __future__ import annotations

from typing import List, Optional, Tuple, Union

import torch

from attentions import flashmvpa


class MVPFormerGQAAttention(torch.nn.Module):
    """Parameters and buffers as in `layers/mvpa.py:9-84`."""

    def __init__(self, config, is_cross_attention=False, layer_idx=None):
        super().__init__()
        max_timesteps = config.max_position_embeddings
        # Unused by the computation; kept so reference checkpoints load strictly.
        self.register_buffer(
            "time_bias",
            torch.ones((max_timesteps, max_timesteps), dtype=torch.bool).tril().view(
                1, 1, max_timesteps, max_timesteps),
        )
        self.register_buffer("masked_bias", torch.tensor(-1e4))
        self.embed_dim = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.num_kv_heads = config.n_head_kv
        self.num_kv_groups = self.num_heads // self.num_kv_heads
        self.head_dim = self.embed_dim // self.num_heads
        self.embed_kv_dim = self.head_dim * self.num_kv_heads
        self.split_size = self.embed_dim
        self.inner_dim = config.n_inner
        self.global_att = config.global_att
        if self.head_dim * self.num_heads != self.embed_dim:
            raise ValueError(
                f"`embed_dim` must be divisible by num_heads (got `embed_dim`: {self.embed_dim} and "
                f"`num_heads`: {self.num_heads}).")
        self.scale_attn_weights = config.scale_attn_weights
        self.is_cross_attention = is_cross_attention
        self.scale_attn_by_inverse_layer_idx = config.scale_attn_by_inverse_layer_idx
        self.layer_idx = layer_idx
        self.reorder_and_upcast_attn = config.reorder_and_upcast_attn
        if getattr(config, "lora", False):
            import loralib as lora  # only needed for LoRA fine-tuning (`layers/mvpa.py:43-62`)

            self.q_attn = lora.Linear(
                self.embed_dim, self.embed_dim, lora_dropout=config.lora_dropout, r=config.lora_rank,
                lora_alpha=config.lora_alpha, bias=False, merge_weights=config.lora_merge)
            self.c_attn = lora.MergedLinear(
                self.embed_dim, 2 * self.embed_kv_dim, enable_lora=[False, True],
                lora_dropout=config.lora_dropout, r=config.lora_rank, lora_alpha=config.lora_alpha,
                bias=False, merge_weights=config.lora_merge)
        else:
            self.q_attn = torch.nn.Linear(self.embed_dim, self.embed_dim, bias=False)
            self.c_attn = torch.nn.Linear(self.embed_dim, 2 * self.embed_kv_dim, bias=False)
        self.position_net = torch.nn.Linear(self.embed_dim, self.embed_kv_dim, bias=False)
        self.channel_net = torch.nn.Linear(self.embed_dim, self.embed_kv_dim, bias=False)
        self.c_proj = torch.nn.Linear(self.embed_dim, self.embed_dim, bias=False)
        self.attn_bias = torch.nn.Parameter(torch.empty(3 * self.embed_kv_dim))  # u, v, z
        torch.nn.init.normal_(self.attn_bias, std=0.02)
        self.attn_dropout = torch.nn.Dropout(config.attn_pdrop)
        self.resid_dropout = torch.nn.Dropout(config.resid_pdrop)

    def adapter_params(self) -> List[str]:
        return ["q_attn.lora_A", "q_attn.lora_B", "c_attn.lora_A", "c_attn.lora_B"]

    def _check_supported(self, layer_past, attention_mask, head_mask, encoder_hidden_states):
        # Options the reference's PyTorch layer has but its Flash layer ignores
        # (`layers/mvpa.py:188-266,314-317`); all are off in every shipped config.
        if not self.global_att or not self.scale_attn_weights or self.scale_attn_by_inverse_layer_idx:
            raise NotImplementedError(
                "MVPA kernels implement global_att=True, scale_attn_weights=True, "
                "scale_attn_by_inverse_layer_idx=False (the shipped configuration)")
        if layer_past is not None or encoder_hidden_states is not None:
            raise NotImplementedError("KV cache / cross attention are not part of the MVPA kernels")
        if attention_mask is not None or head_mask is not None:
            raise NotImplementedError("attention_mask / head_mask are not supported by the MVPA kernels")

    def forward(
        self,
        hidden_states: Optional[Tuple[torch.FloatTensor]],
        positional_embedding: Optional[Tuple[torch.FloatTensor]],
        channel_embedding: Optional[Tuple[torch.FloatTensor]],
        layer_past: Optional[Tuple[torch.Tensor]] = None,
        attention_mask: Optional[torch.FloatTensor] = None,
        head_mask: Optional[torch.FloatTensor] = None,
        encoder_hidden_states: Optional[torch.Tensor] = None,
        encoder_attention_mask: Optional[torch.FloatTensor] = None,
        use_cache: Optional[bool] = False,
        output_attentions: Optional[bool] = False,
    ) -> Tuple[Union[torch.Tensor, Tuple[torch.Tensor]], ...]:
        self._check_supported(layer_past, attention_mask, head_mask, encoder_hidden_states)
        return self._mvpa_forward(hidden_states, positional_embedding, channel_embedding, use_cache,
                                  output_attentions)

    def _mvpa_forward(self, hidden_states, positional_embedding, channel_embedding, use_cache,
                      output_attentions):
        B, T, C, E = hidden_states.shape
        H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        N = T * C
        query = self.q_attn(hidden_states)                       # (B,T,C,E)
        kv = self.c_attn(hidden_states)                          # (B,T,C,2*Hkv*D)
        time_key = self.position_net(positional_embedding)       # (1,T,Hkv*D)
        channel_key = self.channel_net(channel_embedding)        # (1,C,Hkv*D)
        # Strided (B, heads, N, D) views of the projection outputs: no copies.
        q4 = query.view(B, N, H, D).permute(0, 2, 1, 3)
        k4 = kv.view(B, N, 2 * Hkv, D)[:, :, :Hkv].permute(0, 2, 1, 3)
        v4 = kv.view(B, N, 2 * Hkv, D)[:, :, Hkv:].permute(0, 2, 1, 3)
        rt = time_key.view(1, T, Hkv, D).permute(0, 2, 1, 3)     # (1,Hkv,T,D)
        rc = channel_key.view(1, C, Hkv, D).permute(0, 2, 1, 3)  # (1,Hkv,C,D)
        u, v, z = (b.view(1, Hkv, 1, D).to(query.dtype) for b in self.attn_bias.split(self.embed_kv_dim))
        attn = flashmvpa(
            q4, u, v, z, k4, rt, rc, v4,
            causal=True,
            sm_scale=1.0 / (D ** 0.5),
            window_size=10,
            p_drop=self.attn_dropout.p if self.training else 0,
            rel_bias_chan=True,
            rel_bias_time=True,
        )                                                         # (B,H,N,D), laid out (B,N,H,D)
        attn = attn.permute(0, 2, 1, 3).reshape(B, T, C, E)       # free: matches the memory layout
        attn = self.resid_dropout(self.c_proj(attn))
        present = None
        if use_cache is True:  # same shapes as the reference: (B,Hkv,T,C,D) (`layers/mvpa.py:402-405`)
            present = (k4.reshape(B, Hkv, T, C, D), v4.reshape(B, Hkv, T, C, D))
        outputs = (attn, present)
        if output_attentions:
            outputs += (None,)
        return outputs


class MVPFormerGQAFlashAttention(MVPFormerGQAAttention):
    """Like the reference Flash layer (`layers/mvpa.py:340-409`), the unsupported
    arguments are accepted and ignored."""

    def forward(
        self,
        hidden_states: Tuple[torch.FloatTensor] | None,
        positional_embedding: Tuple[torch.FloatTensor] | None,
        channel_embedding: Tuple[torch.FloatTensor] | None,
        layer_past: Tuple[torch.Tensor] | None = None,
        attention_mask: torch.FloatTensor | None = None,
        head_mask: torch.FloatTensor | None = None,
        encoder_hidden_states: torch.Tensor | None = None,
        encoder_attention_mask: torch.FloatTensor | None = None,
        use_cache: bool | None = False,
        output_attentions: bool | None = False,
    ) -> Tuple[torch.Tensor | Tuple[torch.Tensor], ...]:
        return self._mvpa_forward(hidden_states, positional_embedding, channel_embedding, use_cache,
                                  output_attentions)
