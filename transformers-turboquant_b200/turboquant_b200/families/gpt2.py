"""GPT-2 adapter (reference families/gpt2.py:17-119): fused c_attn projection, learned
positions (no rotary), head_dim 64 for every published size."""

from __future__ import annotations

import torch.nn as nn

from ..compressors import compress_kv, fused_attention
from ..plugin import TurboQuantAttentionBase, register_family
from ._cached import CompressedCacheMixin


@register_family("gpt2")
class TurboQuantGPT2Attention(CompressedCacheMixin, TurboQuantAttentionBase):
    ATTENTION_CLASS_NAMES = ("GPT2Attention",)

    @classmethod
    def from_original(cls, original: nn.Module, key_compressor, val_compressor):
        self = cls.__new__(cls)
        nn.Module.__init__(self)
        self.c_attn, self.c_proj = original.c_attn, original.c_proj
        self.attn_dropout, self.resid_dropout = original.attn_dropout, original.resid_dropout
        self.embed_dim, self.num_heads, self.head_dim = original.embed_dim, original.num_heads, original.head_dim
        self.layer_idx = getattr(original, "layer_idx", None)
        self.key_compressor, self.val_compressor = key_compressor, val_compressor
        return self

    def forward(self, hidden_states, past_key_values=None, cache_position=None, attention_mask=None,
                head_mask=None, encoder_hidden_states=None, encoder_attention_mask=None,
                output_attentions=False, **kwargs):
        if output_attentions:
            raise NotImplementedError("the fused kernel never materialises attention probabilities; "
                                      "output_attentions is not available on the compressed path")
        if self.training and self.attn_dropout.p > 0 and not getattr(self, "_warned_dropout", False):
            import warnings
            warnings.warn(f"attention-probability dropout (attn_pdrop={self.attn_dropout.p}) is not applied on the "
                          "compressed path: fine-tuning differs from the reference's adapter, which drops "
                          "probabilities (families/gpt2.py:104); set attn_pdrop=0 to make them agree")
            self._warned_dropout = True
        B, T, _ = hidden_states.shape
        q, k, v = self.c_attn(hidden_states).split(self.embed_dim, dim=2)
        q, k, v = (t.view(B, T, self.num_heads, self.head_dim).transpose(1, 2) for t in (q, k, v))
        if self.kv_cache_capacity is not None and past_key_values is not None:
            # generation against a persistent compressed cache (an extension: the reference runs cache-less)
            out = self._attend_cached(q, k, v, past_key_values, attention_mask)
            return self.resid_dropout(self.c_proj(out.transpose(1, 2).reshape(B, T, self.embed_dim))), None
        ck, cv = compress_kv(k, v, self.key_compressor, self.val_compressor)
        # attention-probability dropout (attn_pdrop) has no counterpart in the fused kernel; it is
        # inactive in eval mode and warned about above in train mode
        out = fused_attention(q, ck, cv, self.key_compressor, self.val_compressor, causal=True,
                              attention_mask=attention_mask)
        out = out.transpose(1, 2).reshape(B, T, self.embed_dim)
        return self.resid_dropout(self.c_proj(out)), None
