"""Qwen2 adapter (reference families/qwen2.py:18-31); q/k/v projections carry biases,
which ride along with the copied Linear modules."""
from ..plugin import register_family
from ._rope_gqa import RopeGQAAttention


@register_family("qwen2")
class TurboQuantQwen2Attention(RopeGQAAttention):
    ATTENTION_CLASS_NAMES = ("Qwen2Attention", "Qwen2SdpaAttention", "Qwen2FlashAttention2")

    @staticmethod
    def _rotary(q, k, cos, sin):
        from transformers.models.qwen2.modeling_qwen2 import apply_rotary_pos_emb
        return apply_rotary_pos_emb(q, k, cos, sin)
