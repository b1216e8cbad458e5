"""DeepSeek (V1, LLaMA-like MHA/GQA) adapter (reference families/deepseek.py:22-37).

The V2/V3 names stay registered as in the reference, but those models use multi-head
latent attention without separate q/k/v projections; `from_original` says so instead of
failing later with an AttributeError."""
from ..plugin import register_family
from ._rope_gqa import RopeGQAAttention


@register_family("deepseek", "deepseek_v2", "deepseek_v3")
class TurboQuantDeepSeekAttention(RopeGQAAttention):
    ATTENTION_CLASS_NAMES = ("DeepseekAttention", "DeepseekSdpaAttention", "DeepseekFlashAttention2",
                             "DeepseekV2Attention", "DeepseekV3Attention")

    @classmethod
    def from_original(cls, original, key_compressor, val_compressor):
        if not all(hasattr(original, p) for p in ("q_proj", "k_proj", "v_proj", "o_proj")):
            raise NotImplementedError(
                f"{type(original).__name__} has no separate q/k/v projections (multi-head latent "
                "attention); only LLaMA-style DeepSeek attention can be replaced")
        return super().from_original(original, key_compressor, val_compressor)
