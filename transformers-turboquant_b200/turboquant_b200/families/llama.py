"""LLaMA / Mistral adapter (reference families/llama.py:18-35)."""
from ..plugin import register_family
from ._rope_gqa import RopeGQAAttention


@register_family("llama", "mistral")
class TurboQuantLlamaAttention(RopeGQAAttention):
    ATTENTION_CLASS_NAMES = ("LlamaAttention", "LlamaSdpaAttention", "LlamaFlashAttention2",
                             "MistralAttention", "MistralSdpaAttention", "MistralFlashAttention2")
