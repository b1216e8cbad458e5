"""Shared body of the LLaMA-style adapters (separate q/k/v/o projections, rotary
position embeddings handed in as (cos, sin), grouped-query attention).

Differences from the reference adapters (families/llama.py:36-122), all needed to run under
transformers >= 5: head counts come from the module's config (the `num_heads` attributes
are gone), `forward` returns the 2-tuple decoder layers unpack, attention is causal even
when HF passes no mask (its sdpa path does), keys/values are compressed once per KV head
instead of after `repeat_interleave`, and `.to()` moves the compressors without touching
attributes the value compressor does not have.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from ..compressors import compress_kv, fused_attention
from ..plugin import TurboQuantAttentionBase
from ._cached import CompressedCacheMixin


class RopeGQAAttention(CompressedCacheMixin, TurboQuantAttentionBase):
    ATTENTION_CLASS_NAMES = ()

    @staticmethod
    def _rotary(q, k, cos, sin):
        """apply_rotary_pos_emb of the reference's adapters (families/llama.py:98), in one launch of the
        library's own kernel where it applies (same bits); HF's function otherwise (partial rotary widths)."""
        from ..rotary import rope, rope_applies
        if rope_applies(q, k, cos, sin):
            return rope(q, k, cos, sin)
        from transformers.models.llama.modeling_llama import apply_rotary_pos_emb
        return apply_rotary_pos_emb(q, k, cos, sin)

    @classmethod
    def from_original(cls, original: nn.Module, key_compressor, val_compressor):
        self = cls.__new__(cls)
        nn.Module.__init__(self)
        for proj in ("q_proj", "k_proj", "v_proj", "o_proj"):
            setattr(self, proj, getattr(original, proj))
        cfg = getattr(original, "config", None)
        self.head_dim = int(getattr(original, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads)
        heads = getattr(original, "num_heads", None) or cfg.num_attention_heads
        kv_heads = getattr(original, "num_key_value_heads", None) or getattr(cfg, "num_key_value_heads", heads)
        self.num_heads, self.num_key_value_heads = int(heads), int(kv_heads)
        self.num_key_value_groups = self.num_heads // self.num_key_value_heads
        self.hidden_size = int(getattr(original, "hidden_size", None) or cfg.hidden_size)
        self.layer_idx = getattr(original, "layer_idx", None)
        self.key_compressor, self.val_compressor = key_compressor, val_compressor
        return self

    def forward(self, hidden_states: torch.Tensor, position_embeddings=None, attention_mask=None,
                past_key_values=None, **kwargs):
        B, T, _ = hidden_states.shape
        shape = (B, T, -1, self.head_dim)
        q = self.q_proj(hidden_states).view(shape).transpose(1, 2)
        k = self.k_proj(hidden_states).view(shape).transpose(1, 2)
        v = self.v_proj(hidden_states).view(shape).transpose(1, 2)
        cos, sin = position_embeddings
        q, k = self._rotary(q, k, cos, sin)
        if self.kv_cache_capacity is not None and past_key_values is not None:
            out = self._attend_cached(q, k, v, past_key_values, attention_mask)
            return self.o_proj(out.transpose(1, 2).reshape(B, T, self.num_heads * self.head_dim)), None
        ck, cv = compress_kv(k, v, self.key_compressor, self.val_compressor)
        out = fused_attention(q, ck, cv, self.key_compressor, self.val_compressor, causal=True,
                              attention_mask=attention_mask)
        out = out.transpose(1, 2).reshape(B, T, self.num_heads * self.head_dim)
        return self.o_proj(out), None
